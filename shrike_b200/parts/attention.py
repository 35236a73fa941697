"""Grouped-query attention over the paged cache.

The formulas are Azimml/shrike's: q/k/v projections with optional bias, heads as
consecutive column blocks (shrike/models/qwen.py:111-122), position encoding on q
and k (qwen.py:123), new keys and values stored before attention reads
(shrike/engine/model_runner.py:69-70), q head i on kv head i // G, scores * scale,
a query at position p sees keys <= p (model_runner.py:129-150), softmax and PV in
32-bit, then the output projection (qwen.py:125).  The three projections are one
matrix product here (rows of Wq, Wk, Wv stacked at load), bias and rotation are
applied to its 32-bit result and rounded once, and one kernel serves single tokens
and portions alike.  Optional `window`: a query sees only the `window` latest keys.
"""

from __future__ import annotations

import torch

from .base import KVNeed, ParamSpec, part_class, register_part


class PagedAttention:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out = spec.num_heads * spec.head_dim
        kv_out = spec.num_kv_heads * spec.head_dim
        params = {
            "q_proj.weight": ParamSpec((q_out, spec.width), "matrix"),
            "k_proj.weight": ParamSpec((kv_out, spec.width), "matrix"),
            "v_proj.weight": ParamSpec((kv_out, spec.width), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, q_out), "matrix"),
        }
        if spec.qkv_bias:
            params["q_proj.bias"] = ParamSpec((q_out,), "bias")
            params["k_proj.bias"] = ParamSpec((kv_out,), "bias")
            params["v_proj.bias"] = ParamSpec((kv_out,), "bias")
        if spec.out_bias:
            params["o_proj.bias"] = ParamSpec((spec.width,), "bias")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        return [KVNeed(spec.num_kv_heads, spec.head_dim, spec.window)]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec
        self.ops = ops
        self.runtime = runtime
        ops.check_head_dim(spec.head_dim)
        self.w_qkv = torch.cat(
            [tensors.pop("q_proj.weight"), tensors.pop("k_proj.weight"), tensors.pop("v_proj.weight")]
        ).contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.b_qkv = None
        if spec.qkv_bias:
            self.b_qkv = torch.cat(
                [tensors.pop("q_proj.bias"), tensors.pop("k_proj.bias"), tensors.pop("v_proj.bias")]
            ).to(torch.float32).contiguous()
        self.b_o = tensors.pop("o_proj.bias").to(torch.float32).contiguous() if spec.out_bias else None
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, ops, runtime)
        self.q_width = spec.num_heads * spec.head_dim
        self.qkv_width = (spec.num_heads + 2 * spec.num_kv_heads) * spec.head_dim

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        n = x.shape[0]
        qkv = rt.buffer("qkv", (n, self.qkv_width), torch.float32)
        qkv = ops.linear(x, self.w_qkv, qkv, allow_partials=True)
        group, keys, values = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, self.q_width), rt.act_dtype)
        table = self.position.rotary_table() if self.position is not None else None
        fused = self.position is None or table is not None
        if fused:
            ops.rope_kv_write(
                qkv, self.b_qkv, ctx.positions, table, q,
                keys if run.writes_cache else None, values if run.writes_cache else None,
                view.slot_mapping, spec.num_heads, spec.num_kv_heads, spec.head_dim,
            )
        else:  # a position encoding with no table: rotate q and k with its own code, then store
            kv_width = spec.num_kv_heads * spec.head_dim
            k_new = rt.buffer("k_new", (n, kv_width), rt.act_dtype)
            v_new = rt.buffer("v_new", (n, kv_width), rt.act_dtype)
            ops.rope_kv_write(
                qkv, self.b_qkv, ctx.positions, None, q, None, None, view.slot_mapping,
                spec.num_heads, spec.num_kv_heads, spec.head_dim, k_out=k_new, v_out=v_new,
            )
            self.position.apply(
                q.view(n, spec.num_heads, spec.head_dim),
                k_new.view(n, spec.num_kv_heads, spec.head_dim),
                ctx.positions,
            )
            if run.writes_cache:
                ops.kv_write(k_new, v_new, keys, values, view.slot_mapping)
        attn = rt.buffer("attn_out", (n, self.q_width), rt.act_dtype)
        ops.paged_attention(
            q, keys, values, view.block_table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.scale, spec.window, attn,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
        )
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(attn, self.w_o, delta, bias=self.b_o, allow_partials=True)


register_part("mixer", "attention", PagedAttention)
