"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases
(shrike/models/qwen.py:128-136).  Gate and up are one matrix product (rows of Wg
then Wu, stacked at load); the activation product is formed in 32-bit."""

from __future__ import annotations

import torch

from .base import ParamSpec, register_part


class GatedMLP:
    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {
            "gate_proj.weight": ParamSpec((spec.intermediate, spec.width), "matrix"),
            "up_proj.weight": ParamSpec((spec.intermediate, spec.width), "matrix"),
            "down_proj.weight": ParamSpec((spec.width, spec.intermediate), "matrix"),
        }

    def __init__(self, spec, tensors, ops, runtime):
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward activation {spec.activation!r} has no kernel; known: silu")
        self.spec = spec
        self.ops = ops
        self.runtime = runtime
        self.w_gate_up = torch.cat([tensors.pop("gate_proj.weight"), tensors.pop("up_proj.weight")]).contiguous()
        self.w_down = tensors.pop("down_proj.weight").contiguous()

    def forward(self, x, ctx):
        spec, rt, ops = self.spec, self.runtime, self.ops
        n = x.shape[0]
        gate_up = rt.buffer("gate_up", (n, 2 * spec.intermediate), rt.act_dtype)
        ops.linear(x, self.w_gate_up, gate_up)
        act = rt.buffer("ffn_act", (n, spec.intermediate), rt.act_dtype)
        ops.silu_mul(gate_up, act)
        delta = rt.buffer("ffn_delta", (n, spec.width), torch.float32)
        return ops.linear(act, self.w_down, delta, allow_partials=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
