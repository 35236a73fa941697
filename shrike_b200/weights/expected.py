"""The table of tensors a configuration expects, by safetensors name."""

from __future__ import annotations

from ..config.model_config import ModelConfig
from ..config.registry import ARCHITECTURES, TensorNames
from ..parts.base import ParamSpec, part_class

LAYER_ROLES = (
    ("mixer", "mixer"),
    ("mixer_norm", "norm"),
    ("feed_forward", "feed_forward"),
    ("feed_forward_norm", "norm"),
)


def tensor_names(config: ModelConfig) -> TensorNames:
    return ARCHITECTURES[config.architecture].tensor_names(config)


def expected_tensors(config: ModelConfig) -> dict[str, ParamSpec]:
    """Every tensor the model reads.  The LM head is listed even when tied; the
    loader lets a tied model leave it out."""
    names = tensor_names(config)
    table: dict[str, ParamSpec] = {
        names.embedding: ParamSpec((config.vocab_size, config.hidden_size), "table")
    }
    for index, layer in enumerate(config.layers):
        for role, category in LAYER_ROLES:
            spec = getattr(layer, role)
            prefix = names.layer_part(index, role)
            for local, param in part_class(category, spec.kind).parameters(spec).items():
                table[prefix + local] = param
    norm = config.final_norm
    for local, param in part_class("norm", norm.kind).parameters(norm).items():
        table[names.final_norm_prefix + local] = param
    table[names.lm_head] = ParamSpec((config.vocab_size, config.hidden_size), "matrix")
    return table
