"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases
(shrike/models/qwen.py:128-136).  Gate and up are one matrix product (rows of Wg and
Wu stacked at load: all gate rows then all up rows, or, where the kernels can apply the
activation inside the product, runs of gate rows each followed by the up rows of the same
features); the activation product is formed in 32-bit."""

from __future__ import annotations

import torch

from .base import ParamSpec, register_part


class GatedMLP:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

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
        gate, up = tensors.pop("gate_proj.weight"), tensors.pop("up_proj.weight")
        run = getattr(ops, "gated_rows", 0)
        self.run = run if run and spec.intermediate % run == 0 else 0
        if self.run:
            blocks = spec.intermediate // self.run
            stacked = torch.stack([gate.view(blocks, self.run, -1), up.view(blocks, self.run, -1)], dim=1)
            self.w_gate_up = stacked.reshape(2 * spec.intermediate, -1).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up]).contiguous()
        self.w_down = tensors.pop("down_proj.weight").contiguous()

    def forward(self, x, ctx):
        spec, rt, ops = self.spec, self.runtime, self.ops
        n = x.shape[0]
        act = rt.buffer("ffn_act", (n, spec.intermediate), rt.act_dtype)
        if not (self.run and ops.linear_gated(x, self.w_gate_up, act)):
            gate_up = rt.buffer("gate_up", (n, 2 * spec.intermediate), rt.act_dtype)
            ops.linear(x, self.w_gate_up, gate_up)
            if self.run:
                ops.silu_mul(gate_up, act, block=self.run)
            else:
                ops.silu_mul(gate_up, act)
        delta = rt.buffer("ffn_delta", (n, spec.width), torch.float32)
        return ops.linear(act, self.w_down, delta, allow_partials=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
