"""Rotary position encoding, rotate-half pairing (j with j + D/2).

inv_freq[j] = 1 / theta^(2j/D) evaluated in float32 exactly as
shrike/models/qwen.py:80 does; the angle is float32(position) * inv_freq[j]
(qwen.py:86) and q' = q cos + rotate_half(q) sin in float32 with one rounding
(qwen.py:91-101).  The table of inverse frequencies is all the fused
rotate-and-store kernel needs, so that is what this part hands to a mixer.
"""

from __future__ import annotations

import torch

from .base import register_part


class Rotary:
    @staticmethod
    def parameters(spec) -> dict:
        return {}

    def __init__(self, spec, tensors, ops, runtime):
        if spec.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {spec.head_dim}")
        self.spec = spec
        exponent = torch.arange(0, spec.head_dim, 2).float() / spec.head_dim
        self.inv_freq = (1.0 / (spec.theta ** exponent)).to(runtime.device)

    def rotary_table(self) -> torch.Tensor:
        return self.inv_freq


register_part("position", "rotary", Rotary)
