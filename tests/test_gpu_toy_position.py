"""Another position encoding, defined here: rotary with interleaved pairs (element 2j with
2j + 1) instead of the halves, applied by the part's own code.  It has no table for the
fused kernel, so the attention part takes its unfused path: bias into q / k / v buffers,
`position.apply`, then the key/value store as a kernel of its own.  Registered, built and
stepped without a change to the package."""

from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

from shrike_b200.config import Architecture, LayerSpec, TensorNames, parse_config, register_architecture
from shrike_b200.config.model_config import AttentionSpec, PartSpec
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.models.qwen2 import parse_qwen2, qwen2_tensor_names
from shrike_b200.parts import register_part
from shrike_b200.weights import random_tensors
from tests.gpu_common import TOL, assert_close, cuda_ops
from tests.helpers import random_tokens
from tests.plain import plain_model as pm
from tests.tiny_configs import TINY_B

pytestmark = pytest.mark.gpu
DEV = "cuda"


@dataclass(frozen=True)
class InterleavedRotarySpec(PartSpec):
    head_dim: int
    theta: float
    kind: str = field(init=False, default="interleaved_rotary")


def interleaved(x, positions, head_dim, theta):
    """x [n, heads, D]: pair (2j, 2j + 1) turns by position * theta^(-2j/D)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=x.device).float() / head_dim))
    angle = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = angle.cos()[:, None, :].to(x.dtype), angle.sin()[:, None, :].to(x.dtype)
    even, odd = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = even * cos - odd * sin
    out[..., 1::2] = odd * cos + even * sin
    return out


class InterleavedRotary:
    @staticmethod
    def parameters(spec):
        return {}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec

    def rotary_table(self):
        return None   # nothing the fused kernel could apply

    def apply(self, q, k, positions):
        q.copy_(interleaved(q.float(), positions, self.spec.head_dim, self.spec.theta).to(q.dtype))
        k.copy_(interleaved(k.float(), positions, self.spec.head_dim, self.spec.theta).to(k.dtype))


def parse_toy(raw):
    config = parse_qwen2(dict(raw, architectures=["Qwen2ForCausalLM"]))
    layers = []
    for layer in config.layers:
        m = layer.mixer
        position = InterleavedRotarySpec(head_dim=m.head_dim, theta=m.position.theta)
        mixer = AttentionSpec(width=m.width, num_heads=m.num_heads, num_kv_heads=m.num_kv_heads, head_dim=m.head_dim,
                              scale=m.scale, qkv_bias=m.qkv_bias, out_bias=m.out_bias, window=m.window, position=position)
        layers.append(LayerSpec(mixer=mixer, mixer_norm=layer.mixer_norm, feed_forward=layer.feed_forward,
                                feed_forward_norm=layer.feed_forward_norm))
    config.architecture = "ToyPositionForCausalLM"
    config.layers = layers
    return config


def plain_toy(raw, weights, ids):
    sizes = pm.config_sizes(raw)
    w = {k: v.double() for k, v in weights.items()}
    n = len(ids)
    positions = torch.arange(n)
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    for layer in range(sizes["layers"]):
        p = f"model.layers.{layer}"
        a = pm.rms_norm(x, w[f"{p}.input_layernorm.weight"], sizes["eps"])
        H, Hkv, D = sizes["heads"], sizes["kv_heads"], sizes["head_dim"]
        q = (a @ w[f"{p}.self_attn.q_proj.weight"].T + w[f"{p}.self_attn.q_proj.bias"]).view(n, H, D)
        k = (a @ w[f"{p}.self_attn.k_proj.weight"].T + w[f"{p}.self_attn.k_proj.bias"]).view(n, Hkv, D)
        v = (a @ w[f"{p}.self_attn.v_proj.weight"].T + w[f"{p}.self_attn.v_proj.bias"]).view(n, Hkv, D)
        q, k = interleaved(q, positions, D, sizes["theta"]), interleaved(k, positions, D, sizes["theta"])
        x = x + pm.causal_attention(q, k, v).reshape(n, -1) @ w[f"{p}.self_attn.o_proj.weight"].T
        m = pm.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], sizes["eps"])
        x = x + pm.mlp(m, w, f"{p}.mlp", pm.Rounder(()))
    return (pm.rms_norm(x, w["model.norm.weight"], sizes["eps"]) @ w["lm_head.weight"].T).numpy()


def test_position_encoding_without_a_table_takes_the_unfused_path():
    register_part("position", "interleaved_rotary", InterleavedRotary)
    register_architecture(Architecture("ToyPositionForCausalLM", parse_toy, qwen2_tensor_names))
    raw = dict(TINY_B, architectures=["ToyPositionForCausalLM"])
    config = parse_config(raw)
    weights = random_tensors(config, 9)
    runner = ModelRunner(config, {k: v.to(DEV) for k, v in weights.items()}, cuda_ops(torch.float32), DEV,
                         "float32", page_size=8, num_pages=16, max_slots=2)
    ids = random_tokens(raw["vocab_size"], 50, 4)
    want = plain_toy(raw, weights, ids)
    cache, pos, rows = runner.cache.open(), 0, []
    for n in (19, 1, 1, 2, 27):
        runner.cache.append(cache, pos, n)
        rows.append(runner.step([StepEntry(cache, ids[pos:pos + n], pos, list(range(n)))]).cpu().numpy().copy())
        pos += n
    assert_close(np.concatenate(rows), want, TOL["float32"], "interleaved rotary through the unfused path")
    halves = pm.forward(TINY_B, weights, ids).numpy()
    assert np.abs(halves - want).max() > 1e-3, "the toy encoding must differ from the built-in one"
