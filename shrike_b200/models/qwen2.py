"""Qwen2 dense decoder: config.json keys -> parts, and its tensor names.

Keys and defaults follow Azimml/shrike's `QwenConfig` (shrike/models/qwen.py:33-49):
`head_dim` is optional (else hidden_size // num_attention_heads), `rms_norm_eps`
and `rope_theta` have no default, `tie_word_embeddings` defaults to false,
`eos_token_id` is an int or a list.  q/k/v carry a bias and o_proj none
(qwen.py:111-114); the activation is SiLU (qwen.py:136); the score scale is
head_dim^-0.5 (shrike/engine/model_runner.py:131).

Beyond the reference, which never reads them: `use_sliding_window` with
`sliding_window` and `max_window_layers` gives the layers from index
`max_window_layers` on a key window (a query sees the `sliding_window` most recent
keys, itself included), and a non-null `rope_scaling` is refused instead of being
ignored.
"""

from __future__ import annotations

from ..config.model_config import (
    AttentionSpec,
    ConfigError,
    GatedMLPSpec,
    LayerRun,
    LayerSpec,
    ModelConfig,
    RMSNormSpec,
    RotarySpec,
    normalise_dtype,
    require,
)
from ..config.registry import Architecture, TensorNames, register_architecture


def parse_qwen2(raw: dict) -> ModelConfig:
    hidden = require(raw, "hidden_size", int)
    inter = require(raw, "intermediate_size", int)
    num_layers = require(raw, "num_hidden_layers", int)
    heads = require(raw, "num_attention_heads", int)
    kv_heads = require(raw, "num_key_value_heads", int)
    head_dim = raw.get("head_dim") or hidden // heads
    vocab = require(raw, "vocab_size", int)
    eps = float(require(raw, "rms_norm_eps", float))
    theta = float(require(raw, "rope_theta", float))
    if raw.get("rope_scaling") is not None:
        raise ConfigError("config.json: rope_scaling is not supported for Qwen2ForCausalLM here")
    activation = raw.get("hidden_act", "silu")
    if activation != "silu":
        raise ConfigError(f"config.json: hidden_act={activation!r}; Qwen2 here runs 'silu'")

    window_from = num_layers
    window = None
    if raw.get("use_sliding_window", False):
        window = require(raw, "sliding_window", int)
        window_from = int(raw.get("max_window_layers", num_layers))

    eos = raw.get("eos_token_id")
    eos_ids = list(eos) if isinstance(eos, list) else ([] if eos is None else [int(eos)])

    rotary = RotarySpec(head_dim=head_dim, theta=theta)
    norm = RMSNormSpec(width=hidden, eps=eps)
    layers = []
    for index in range(num_layers):
        mixer = AttentionSpec(
            width=hidden,
            num_heads=heads,
            num_kv_heads=kv_heads,
            head_dim=head_dim,
            scale=head_dim**-0.5,
            qkv_bias=True,
            out_bias=False,
            window=window if index >= window_from else None,
            position=rotary,
        )
        ffn = GatedMLPSpec(width=hidden, intermediate=inter, activation=activation)
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm, feed_forward=ffn, feed_forward_norm=norm))

    return ModelConfig(
        architecture="Qwen2ForCausalLM",
        hidden_size=hidden,
        vocab_size=vocab,
        layers=layers,
        order=[LayerRun(layer=i, cache=i) for i in range(num_layers)],
        final_norm=norm,
        tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
        max_position_embeddings=int(raw.get("max_position_embeddings", 0)) or 1 << 30,
        eos_token_ids=eos_ids,
        dtype=normalise_dtype(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
        raw=dict(raw),
    )


_ROLE_PREFIX = {
    "mixer": "self_attn.",
    "mixer_norm": "input_layernorm.",
    "feed_forward": "mlp.",
    "feed_forward_norm": "post_attention_layernorm.",
}


def qwen2_tensor_names(config: ModelConfig) -> TensorNames:
    return TensorNames(
        embedding="model.embed_tokens.weight",
        final_norm_prefix="model.norm.",
        lm_head="lm_head.weight",
        layer_part=lambda layer, role: f"model.layers.{layer}.{_ROLE_PREFIX[role]}",
    )


QWEN2 = register_architecture(
    Architecture(name="Qwen2ForCausalLM", parse_config=parse_qwen2, tensor_names=qwen2_tensor_names)
)
