"""Token embedding and output head: how ids enter the residual stream and how it leaves as logits.

The embedding copies one table row per token into the float32 residual
(shrike/models/qwen.py:161); the head multiplies the final norm's output at the wanted
rows by a [vocab, width] matrix, the embedding's own table when the model ties them
(qwen.py:192,211-212), into float32 logits.  Both are parts like the others, chosen by the
`kind` of `ModelConfig.embedding` and `ModelConfig.head`: an architecture that scales its
embedding, adds a learned position table or caps its logits registers a part of its own
instead of changing the model class.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, register_part


class TokenEmbedding:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "table")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.table = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        resid = self.runtime.buffer("resid", (ctx.num_tokens, self.spec.width), torch.float32)
        self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens)
        return resid


class LMHead:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "matrix")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.weight = tensors["weight"]

    def forward(self, hidden) -> torch.Tensor:
        logits = self.runtime.buffer("logits", (hidden.shape[0], self.spec.vocab), torch.float32)
        if hidden.shape[0]:
            self.ops.linear(hidden, self.weight, logits)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
