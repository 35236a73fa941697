"""Typed model configuration.

A `ModelConfig` is what an architecture's `parse_config` makes of the keys of its
own `config.json`: the widths, and for every layer a `LayerSpec` that names the
parts the layer is put together from (mixer, feed-forward, norm, position
encoding) with their sizes and constants.  The order in which layers run is data
too (`order`, a list of `LayerRun`).  Nothing here knows a model by name; no size
appears in code outside the values read from `config.json`.

Reference: Azimml/shrike reads a flat set of keys into `QwenConfig`
(shrike/models/qwen.py:23-49); the per-layer specs are this engine's own design so
that another architecture can choose other parts layer by layer.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


@dataclass(frozen=True)
class PartSpec:
    """Base of all part specifications: `kind` selects the implementation."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding (shrike/models/qwen.py:77-101)."""

    head_dim: int
    theta: float
    kind: str = field(init=False, default="rotary")


@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """Root-mean-square norm with a plain weight (shrike/models/qwen.py:64-74)."""

    width: int
    eps: float
    kind: str = field(init=False, default="rmsnorm")


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Grouped-query softmax attention over a paged key/value cache.

    `window` is the number of most recent keys a query sees (None: all of them).
    `scale` multiplies the scores before the softmax.
    """

    width: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qkv_bias: bool
    out_bias: bool
    window: int | None
    position: PartSpec | None
    kind: str = field(init=False, default="attention")

    def __post_init__(self):
        if self.num_heads % self.num_kv_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_heads} is not a multiple of "
                f"num_key_value_heads={self.num_kv_heads}"
            )
        if self.window is not None and self.window < 1:
            raise ConfigError(f"attention window must be >= 1, got {self.window}")


@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x)) (shrike/models/qwen.py:128-136)."""

    width: int
    intermediate: int
    activation: str
    kind: str = field(init=False, default="gated_mlp")


@dataclass(frozen=True)
class TokenEmbeddingSpec(PartSpec):
    """One table row per token id, copied into the residual (shrike/models/qwen.py:161)."""

    vocab: int
    width: int
    kind: str = field(init=False, default="token_embedding")


@dataclass(frozen=True)
class LMHeadSpec(PartSpec):
    """Normed hidden rows times a [vocab, width] matrix, which may be the embedding's table
    (shrike/models/qwen.py:192,211-212)."""

    width: int
    vocab: int
    tied: bool = False
    kind: str = field(init=False, default="lm_head")


STANDARD_ROLES = (
    ("mixer", "mixer"),
    ("mixer_norm", "norm"),
    ("feed_forward", "feed_forward"),
    ("feed_forward_norm", "norm"),
)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which parts, and how they are arranged (`block`).

    The four named parts are what a pre-norm block takes.  A block that arranges more parts
    (norms after its branches, a third branch) lists them in `extra` as (role, category, spec);
    the block class is built with every role as a keyword and the architecture names the
    tensors of every role.
    """

    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec
    block: str = "pre_norm"
    extra: tuple = ()

    def roles(self):
        """(role, category, spec) of every part of the layer."""
        for role, category in STANDARD_ROLES:
            yield role, category, getattr(self, role)
        yield from self.extra


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    `layer` indexes `ModelConfig.layers` (weights); `cache` is the id of the cache
    (pages or state) this run uses.  A run with `writes_cache=False` reads the cache
    that an earlier run with the same `cache` id wrote in this step.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass
class ModelConfig:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list[LayerSpec]
    order: list[LayerRun]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: list[int]
    dtype: str  # "bfloat16" | "float32": what config.json asks for
    raw: dict[str, Any] = field(default_factory=dict, repr=False)
    # how token ids become the residual and how normed rows become logits: parts like the others,
    # chosen by `kind`.  None: one table, and a plain (or tied) matrix, from the sizes above.
    embedding: PartSpec | None = None
    head: PartSpec | None = None

    def __post_init__(self):
        if self.embedding is None:
            self.embedding = TokenEmbeddingSpec(vocab=self.vocab_size, width=self.hidden_size)
        if self.head is None:
            self.head = LMHeadSpec(width=self.hidden_size, vocab=self.vocab_size, tied=self.tie_word_embeddings)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @property
    def num_caches(self) -> int:
        return 1 + max(run.cache for run in self.order) if self.order else 0

    def validate(self) -> None:
        writers: dict[int, int] = {}
        for index, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"run {index} names layer {run.layer}, model has {len(self.layers)}")
            if run.writes_cache:
                if run.cache in writers:
                    raise ConfigError(
                        f"runs {writers[run.cache]} and {index} both write cache {run.cache}"
                    )
                writers[run.cache] = index
            elif run.cache not in writers:
                raise ConfigError(f"run {index} reads cache {run.cache} before any run wrote it")


DTYPE_NAMES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "float": "float32",
}


def normalise_dtype(name: str) -> str:
    try:
        return DTYPE_NAMES[str(name).replace("torch.", "")]
    except KeyError:
        raise ConfigError(
            f"dtype {name!r} is not served; this engine runs bfloat16 or float32"
        ) from None


def require(raw: dict, key: str, kind=None):
    """A key that config.json must hold; a clear error when it does not."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks the key {key!r}")
    value = raw[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int) or value < 1):
        raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
    if kind is float and (isinstance(value, bool) or not isinstance(value, (int, float))):
        raise ConfigError(f"config.json: {key} must be a number, got {value!r}")
    return value


def read_config_json(model_dir: str | Path) -> dict:
    """The raw dictionary; missing file is a FileNotFoundError with a hint
    (shrike/models/qwen.py:25-31)."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(
            f"no config.json under {str(model_dir)!r}; point --model (or SHRIKE_B200_MODEL_DIR) at "
            "a folder with config.json and *.safetensors, or write one with "
            "`python -m shrike_b200.weights.random_init`"
        )
    return json.loads(path.read_text())
