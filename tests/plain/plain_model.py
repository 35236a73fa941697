"""Plain, slow, whole-sequence implementation of the Qwen2 dense decoder.

It rests on the formulas of Azimml/shrike's model code (each function cites the
file and lines it restates); `tests/golden/make_golden.py` compares it once with
that code run on the CPU.  It keeps no cache, runs whole sequences only, has one
function per part and shares no code with the `shrike_b200` package: it reads the
raw `config.json` dictionary and a name -> tensor dictionary itself.

Two things go beyond the reference, because the engine's parts are more general
than the one model and the tests need an oracle for them:
  * `windows`: a per-layer key window (query i sees keys j with i - j < window);
  * `order`: the list of layer runs, each `(layer, cache_source)`; a layer may be
    named twice, and `cache_source` names an earlier run whose keys and values this
    run attends over instead of its own.
`rounding` emulates where the bfloat16 engine rounds activations (norm output,
rotated q/k, v, attention output, gate/up, activation product); sums, softmax,
norm statistics and the residual stay in the working precision.
"""

from __future__ import annotations

import math

import torch

ROUNDING_POINTS = ("norm_out", "q", "k", "v", "attn_out", "gate_up", "act")


def _round_bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


class Rounder:
    """Applies bfloat16 rounding at the named points, or nothing."""

    def __init__(self, points=()):
        self.points = set(points)

    def __call__(self, name: str, x: torch.Tensor) -> torch.Tensor:
        return _round_bf16(x) if name in self.points else x


def config_sizes(raw: dict) -> dict:
    """Sizes as shrike reads them (shrike/models/qwen.py:33-49)."""
    hidden = raw["hidden_size"]
    heads = raw["num_attention_heads"]
    return dict(
        hidden=hidden,
        inter=raw["intermediate_size"],
        layers=raw["num_hidden_layers"],
        heads=heads,
        kv_heads=raw["num_key_value_heads"],
        head_dim=raw.get("head_dim") or hidden // heads,
        vocab=raw["vocab_size"],
        eps=raw["rms_norm_eps"],
        theta=raw["rope_theta"],
        tied=raw.get("tie_word_embeddings", False),
    )


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """shrike/models/qwen.py:70-74: x * rsqrt(mean(x^2) + eps) * w, plain w."""
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight.to(x.dtype)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> tuple:
    """shrike/models/qwen.py:80,86-88: inv_freq in float32, angles = pos * inv_freq,
    duplicated to the full head size; the angle is formed in float32 as the
    reference does, whatever the working precision."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    freqs = torch.outer(positions.float(), inv_freq.to(positions.device))
    emb = torch.cat((freqs, freqs), dim=-1)
    if dtype == torch.float64:
        emb = emb.double()
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """shrike/models/qwen.py:91-93."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """shrike/models/qwen.py:96-101, for one of q or k: x [n, heads, D]."""
    return x * cos.unsqueeze(1) + rotate_half(x) * sin.unsqueeze(1)


def causal_attention(q, k, v, window: int | None = None) -> torch.Tensor:
    """Scores, scale, mask, softmax and PV for a whole sequence.

    shrike/engine/model_runner.py:129-136 (grouped heads: q head i uses kv head
    i // G; scale D^-0.5; softmax in the working precision) with the causal mask
    of shrike/models/qwen.py:243-248.  q [m, H, D], k/v [n, Hkv, D] -> [m, H, D].
    With m < n the queries are the last m positions of the sequence, as the
    reference's mask is aligned to the end of the keys (model_runner.py:137-147).
    Runs on the device of its inputs.
    """
    m, heads, dim = q.shape
    n, kv_heads = k.shape[0], k.shape[1]
    group = heads // kv_heads
    qg = q.view(m, kv_heads, group, dim)
    scores = torch.einsum("nkgd,skd->kgns", qg, k) * dim**-0.5
    i = torch.arange(n - m, n, device=q.device)[:, None]
    j = torch.arange(n, device=q.device)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (i - j >= window)
    scores = scores.masked_fill(hidden[None, None], float("-inf"))
    probs = scores.softmax(-1)
    out = torch.einsum("kgns,skd->nkgd", probs, v)
    return out.reshape(m, heads, dim)


def attention_inputs(x, w, prefix, sizes, cos, sin, rnd: Rounder):
    """q/k/v projections with bias and RoPE (shrike/models/qwen.py:120-123)."""
    n = x.shape[0]
    H, Hkv, D = sizes["heads"], sizes["kv_heads"], sizes["head_dim"]

    def proj(name):
        y = x @ w[f"{prefix}.{name}.weight"].T
        bias = w.get(f"{prefix}.{name}.bias")
        return y + bias if bias is not None else y

    q = proj("q_proj").view(n, H, D)
    k = proj("k_proj").view(n, Hkv, D)
    v = proj("v_proj").view(n, Hkv, D)
    q = rnd("q", apply_rope(q, cos, sin))
    k = rnd("k", apply_rope(k, cos, sin))
    v = rnd("v", v)
    return q, k, v


def mlp(x, w, prefix, rnd: Rounder):
    """shrike/models/qwen.py:136: down(silu(gate(x)) * up(x)), no biases."""
    g = rnd("gate_up", x @ w[f"{prefix}.gate_proj.weight"].T)
    u = rnd("gate_up", x @ w[f"{prefix}.up_proj.weight"].T)
    act = rnd("act", g * torch.sigmoid(g) * u)
    return act @ w[f"{prefix}.down_proj.weight"].T


def forward(
    raw_config: dict,
    weights: dict,
    token_ids,
    dtype=torch.float64,
    rounding=(),
    windows: dict | None = None,
    order: list | None = None,
) -> torch.Tensor:
    """Logits [n, vocab] for one whole sequence.

    Embedding (qwen.py:161), the layers in `order` as pre-norm residual blocks
    (qwen.py:148-149), final norm (qwen.py:164) and LM head, tied to the
    embedding when the configuration says so and the file has no head
    (qwen.py:192,211-212).
    """
    sizes = config_sizes(raw_config)
    rnd = Rounder(rounding)
    w = {name: t.to(dtype) for name, t in weights.items()}
    device = next(iter(w.values())).device
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    n = ids.shape[0]
    cos, sin = rope_tables(torch.arange(n, device=device), sizes["head_dim"], sizes["theta"], dtype)
    cos, sin = cos.to(dtype), sin.to(dtype)
    windows = windows or {}
    if order is None:
        order = [(layer, None) for layer in range(sizes["layers"])]

    x = w["model.embed_tokens.weight"][ids]
    kv_of_run: list = []
    for layer, source in order:
        p = f"model.layers.{layer}"
        a = rnd("norm_out", rms_norm(x, w[f"{p}.input_layernorm.weight"], sizes["eps"]))
        q, k, v = attention_inputs(a, w, f"{p}.self_attn", sizes, cos, sin, rnd)
        if source is not None:
            k, v = kv_of_run[source]
        kv_of_run.append((k, v))
        o = rnd("attn_out", causal_attention(q, k, v, windows.get(layer)))
        x = x + o.reshape(n, -1) @ w[f"{p}.self_attn.o_proj.weight"].T
        m = rnd("norm_out", rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], sizes["eps"]))
        x = x + mlp(m, w, f"{p}.mlp", rnd)
    hidden = rnd("norm_out", rms_norm(x, w["model.norm.weight"], sizes["eps"]))
    head = w.get("lm_head.weight")
    if head is None:
        if not sizes["tied"]:
            raise KeyError("lm_head.weight")
        head = w["model.embed_tokens.weight"]
    return hidden @ head.T


def greedy_continue(raw_config, weights, prompt, num_new, dtype=torch.float64, **kw):
    """Greedy tokens, recomputing the whole sequence for each one (no cache);
    ties go to the lowest index as in shrike/engine/sampler.py:15-17."""
    seq = list(prompt)
    margins = []
    for _ in range(num_new):
        logits = forward(raw_config, weights, seq, dtype=dtype, **kw)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        seq.append(int(torch.argmax(logits)))
    return seq[len(prompt):], margins


def softmax_with_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """shrike/engine/sampler.py:21-22: softmax(float(logits) / T)."""
    return torch.softmax(logits.double() / temperature, dim=-1)


def top_p_keep(probs: torch.Tensor, top_p: float) -> torch.Tensor:
    """shrike/engine/sampler.py:24-28: sort descending, keep a token while the
    mass strictly before it is below top_p (the largest is always kept).
    Returns a boolean mask in vocabulary order."""
    sorted_probs, sorted_idx = probs.sort(-1, descending=True)
    before = sorted_probs.cumsum(-1) - sorted_probs
    keep_sorted = before < top_p
    keep = torch.zeros_like(keep_sorted)
    keep[sorted_idx] = keep_sorted
    return keep


def blocks_for(tokens: int, block_size: int) -> int:
    """shrike/engine/block_manager.py:60-70: ceil(tokens / block_size)."""
    return math.ceil(tokens / block_size)
