"""One registry: architecture name (config.json `architectures[0]`) -> architecture.

An `Architecture` knows two things and nothing about kernels: how to turn its own
config.json keys into a `ModelConfig`, and which safetensors name each parameter
of each part has.  Azimml/shrike has one hard-wired model class
(shrike/models/qwen.py:167) and a registry of checkpoint ids only
(shrike/config.py:21-25); dispatch by architecture name is this engine's design.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class TensorNames:
    """Where an architecture keeps its tensors.

    `layer_part(layer, role)` gives the prefix for a layer's part, role being one of
    "mixer", "mixer_norm", "feed_forward", "feed_forward_norm" (or a role the layer lists
    in `extra`); a part's own parameter names (e.g. "q_proj.weight") are appended to it.
    `embedding` and `lm_head` are the full names of the token table and the output
    matrix: the parameter "weight" of the embedding part and of the head part.  Further
    parameters of those two parts (an embedding that also holds a position table, say) are
    named `embedding_prefix + local` and `head_prefix + local`; the prefixes default to the
    two names without their trailing "weight".
    """

    embedding: str
    final_norm_prefix: str
    lm_head: str
    layer_part: Callable[[int, str], str]
    embedding_prefix: str | None = None
    head_prefix: str | None = None

    def embedding_name(self, local: str) -> str:
        return self.embedding if local == "weight" else _prefix(self.embedding_prefix, self.embedding) + local

    def head_name(self, local: str) -> str:
        return self.lm_head if local == "weight" else _prefix(self.head_prefix, self.lm_head) + local


def _prefix(given: str | None, weight_name: str) -> str:
    if given is not None:
        return given
    return weight_name[: -len("weight")] if weight_name.endswith("weight") else weight_name + "."


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], ModelConfig]
    tensor_names: Callable[[ModelConfig], TensorNames]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    ARCHITECTURES[arch.name] = arch
    return arch


def _register_builtin() -> None:
    """The package's own architectures register themselves on import."""
    from .. import models  # noqa: F401


def architecture_of(raw: dict) -> Architecture:
    _register_builtin()
    names = raw.get("architectures")
    if not names or not isinstance(names, list):
        raise ConfigError(
            "config.json lacks `architectures`; known: " + ", ".join(sorted(ARCHITECTURES))
        )
    if names[0] not in ARCHITECTURES:
        raise ConfigError(
            f"architecture {names[0]!r} is not registered; known: "
            + ", ".join(sorted(ARCHITECTURES))
        )
    return ARCHITECTURES[names[0]]


def parse_config(raw: dict) -> ModelConfig:
    config = architecture_of(raw).parse_config(raw)
    config.validate()
    return config


def load_config(model_dir) -> ModelConfig:
    return parse_config(read_config_json(model_dir))
