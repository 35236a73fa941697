"""RMSNorm, fused with the residual sum.

y = x * rsqrt(mean(x^2) + eps) * w with a plain weight, all in 32-bit, one
rounding at the end (shrike/models/qwen.py:64-74).  The residual stream is kept in
float32; `add_norm` first adds the pending branch output to it, so the sum that
Azimml/shrike does in the model dtype (qwen.py:148-149) is a 32-bit sum here and
costs no pass of its own.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, register_part


class RMSNorm:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.width,), "norm")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec
        self.ops = ops
        self.runtime = runtime
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def add_norm(self, resid, delta, out_name="normed"):
        out = self.runtime.buffer(out_name, (resid.shape[0], self.spec.width), self.runtime.act_dtype)
        self.ops.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out)
        return out

    def gather_norm(self, resid, delta, rows, out_name="normed_rows"):
        out = self.runtime.buffer(out_name, (rows.shape[0], self.spec.width), self.runtime.act_dtype)
        self.ops.gather_add_rmsnorm(resid, delta, rows, self.weight, self.spec.eps, out)
        return out


register_part("norm", "rmsnorm", RMSNorm)
