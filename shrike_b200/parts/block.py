"""Pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
(shrike/models/qwen.py:147-150).  The residual `resid` is float32; a branch output
is handed on as `delta` and added by the next norm kernel."""

from __future__ import annotations

from .base import register_part


class PreNormBlock:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    def __init__(self, mixer, mixer_norm, feed_forward, feed_forward_norm):
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm

    def forward(self, resid, delta, ctx, run):
        hidden = self.mixer_norm.add_norm(resid, delta)
        delta = self.mixer.forward(hidden, ctx, run)
        hidden = self.feed_forward_norm.add_norm(resid, delta)
        delta = self.feed_forward.forward(hidden, ctx)
        return resid, delta


register_part("block", "pre_norm", PreNormBlock)
