"""The table of tensors a configuration expects, by safetensors name."""

from __future__ import annotations

from ..config.model_config import STANDARD_ROLES, ModelConfig
from ..config.registry import ARCHITECTURES, TensorNames
from ..parts.base import ParamSpec, part_class

LAYER_ROLES = STANDARD_ROLES   # the four parts of a pre-norm layer; a layer may list more (LayerSpec.extra)


def tensor_names(config: ModelConfig) -> TensorNames:
    return ARCHITECTURES[config.architecture].tensor_names(config)


def expected_tensors(config: ModelConfig) -> dict[str, ParamSpec]:
    """Every tensor the model reads: the parameters each part class declares for its spec, under
    the names the architecture gives them.  The head's matrix is listed even when it is tied to
    the embedding; the loader lets a tied model leave it out."""
    names = tensor_names(config)
    table: dict[str, ParamSpec] = {}
    for local, param in part_class("embedding", config.embedding.kind).parameters(config.embedding).items():
        table[names.embedding_name(local)] = param
    for index, layer in enumerate(config.layers):
        for role, category, spec in layer.roles():
            prefix = names.layer_part(index, role)
            for local, param in part_class(category, spec.kind).parameters(spec).items():
                table[prefix + local] = param
    norm = config.final_norm
    for local, param in part_class("norm", norm.kind).parameters(norm).items():
        table[names.final_norm_prefix + local] = param
    for local, param in part_class("head", config.head.kind).parameters(config.head).items():
        table[names.head_name(local)] = param
    return table
