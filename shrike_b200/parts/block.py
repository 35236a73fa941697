"""Pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
(shrike/models/qwen.py:147-150).  The residual `resid` is float32; a branch output
is handed on as `delta` and added by the next norm kernel.

When the kernels offer a native issue of whole layers (`ops.layer_program()`) and the four parts
are ones it serves, the layer's launches are issued by one native call instead of part by part:
the same kernels with the same arguments in the same order, without the interpreter between them."""

from __future__ import annotations

from .base import register_part


class PreNormBlock:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    def __init__(self, mixer, mixer_norm, feed_forward, feed_forward_norm):
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm
        self._program = None
        self._asked = False
        self._native_constants: dict = {}   # what the native issue keeps per run of this layer

    def _native(self):
        if not self._asked:
            self._asked = True
            offer = getattr(getattr(self.mixer, "ops", None), "layer_program", None)
            program = offer() if offer is not None else None
            if program is not None and program.serves(self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm):
                self._program = program
        return self._program

    def prepare(self) -> None:
        """Called once when the model is built: settles how the layer is issued, so that what that
        takes (the native library's set-up) does not fall into a request's first step."""
        self._native()

    def forward(self, resid, delta, ctx, run):
        program = self._native()
        if program is not None and getattr(program.ops, "native_layers", False):
            return resid, program.run(self._native_constants, self.mixer, self.mixer_norm, self.feed_forward,
                                      self.feed_forward_norm, resid, delta, ctx, run)
        hidden = self.mixer_norm.add_norm(resid, delta)
        delta = self.mixer.forward(hidden, ctx, run)
        hidden = self.feed_forward_norm.add_norm(resid, delta)
        delta = self.feed_forward.forward(hidden, ctx)
        return resid, delta


register_part("block", "pre_norm", PreNormBlock)
