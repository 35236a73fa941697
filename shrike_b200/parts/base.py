"""What a part is, and the registries that map a spec's `kind` to its class.

A layer is put together from four kinds of part, chosen by the configuration layer
by layer: a mixer (attention here), a feed-forward, a norm and a position encoding,
arranged by a block.  A part is built from its spec alone; it never learns which
model it is in.  Azimml/shrike hard-wires these as nn.Modules
(shrike/models/qwen.py:64-150) and injects only the attention backend
(qwen.py:52-61); the split into registered parts is this engine's design.

Interfaces (duck-typed; `parameters` and `cache_needs` are static so that weights can
be checked and the cache sized before anything is put on the device):

  every part class
      parameters(spec) -> {local name: ParamSpec}
      __init__(spec, tensors: {local name: Tensor}, ops, runtime)
  norm
      add_norm(resid_f32[N,W], delta | None) -> normed[N,W]
          resid += delta (32-bit), then the normalised rows in the activation dtype;
          delta is [N,W], or a stack [P,N,W] of partial sums that the kernel adds in order
          (what `ops.linear(..., allow_partials=True)` may return)
      gather_norm(resid_f32, delta, rows_i32[R]) -> normed[R,W]   (only the wanted rows)
  position encoding
      rotary_table() -> float32 [D/2] inverse frequencies, when the mixer's fused
          kernel can apply it; else None and
      apply(q[N,H,D], k[N,Hkv,D], positions_i32[N]) rotates in place
  mixer
      cache_needs(spec) -> [KVNeed | StateNeed]
      forward(x[N,W], ctx: StepContext, run: LayerRun) -> delta[N,W]
  feed-forward
      forward(x[N,W], ctx) -> delta[N,W]
  block
      __init__(**parts by role)   ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm"
          and whatever further roles the layer's spec lists in `extra`)
      forward(resid_f32, delta, ctx, run) -> (resid_f32, delta)
          `delta` is a sum not yet added to the residual; the next norm adds it.
  embedding
      forward(ctx) -> resid_f32[N,W]   the residual stream of the step's tokens.  A token id of
          -1 - r stands for `ctx.previous_tokens[r]` (what the step before drew in its row r).
      `table`: the [vocab, W] tensor a tied head may share, or None
  head
      forward(hidden[R,W]) -> float32 logits [R, vocab]   (hidden: the final norm's output on the
          wanted rows); built with tensors {"weight": ...}, the embedding's table when tied

A part may declare the class attribute `capture_safe = True`.  It then promises that forward()
launches the same kernels with the same sizes for the same batch shape, whatever the positions,
slots and pages of the step (so a recorded launch sequence can be replayed), and that it leaves
rows alone whose cache slot and state slot are -1: the step function pads batches of single
tokens with such rows up to a few fixed sizes.  A model is treated so only if all its parts say so.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part expects: its shape and how random weights fill it.

    init: "matrix" | "table" (N(0, 0.02)), "bias" (N(0, 0.02)), "norm" (1 + N(0, 0.1)).
    """

    shape: tuple[int, ...]
    init: str


@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages: `window` None keeps all, else the last `window`."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, one slot per live request."""

    shape: tuple[int, ...]
    dtype: str = "float32"


MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITIONS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}
EMBEDDINGS: dict[str, type] = {}
HEADS: dict[str, type] = {}

_CATEGORIES = {
    "embedding": EMBEDDINGS,
    "head": HEADS,
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position": POSITIONS,
    "block": BLOCKS,
}


def register_part(category: str, kind: str, cls: type) -> type:
    """Adds a part class; `category` is one of mixer, feed_forward, norm, position, block,
    embedding, head."""
    _CATEGORIES[category][kind] = cls
    return cls


def part_class(category: str, kind: str) -> type:
    table = _CATEGORIES[category]
    if kind not in table:
        raise KeyError(f"no {category} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind]
