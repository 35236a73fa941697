"""A stand-in for the CUDA kernels, for tests that run without a GPU.

It has the interface of `shrike_b200.ops.cuda_ops.CudaOps` and the same meaning for
every argument, written with plain torch on the CPU, one loop at a time.  Host
logic (batch metadata, block tables, slots, the scheduler, the engine loop) can so
be driven end to end here; the kernels themselves are tested on the GPU.  Nothing
in the package imports this file.
"""

from __future__ import annotations

import math

import torch

from shrike_b200.sampling.rng import gumbel_noise_host


class EmulatedOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype
        self.launches = 0

    def check_head_dim(self, head_dim):
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head size {head_dim} is not served")

    def embed(self, ids, table, out, previous=None):
        ids = ids.long()
        if previous is not None and (ids < 0).any():
            ids = torch.where(ids < 0, previous.long()[(-1 - ids).clamp(min=0, max=previous.numel() - 1)], ids)
        out.copy_(table[ids].float())

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        if delta is not None:
            resid.add_(delta.float().sum(0) if delta.dim() == 3 else delta.float())
        var = resid.pow(2).mean(-1, keepdim=True)
        out.copy_((resid * torch.rsqrt(var + eps) * weight).to(out.dtype))

    def gather_add_rmsnorm(self, resid, delta, rows, weight, eps, out):
        x = resid[rows.long()]
        if delta is not None:
            summed = delta.float().sum(0) if delta.dim() == 3 else delta.float()
            x = x + summed[rows.long()]
        var = x.pow(2).mean(-1, keepdim=True)
        out.copy_((x * torch.rsqrt(var + eps) * weight).to(out.dtype))

    def linear(self, x, w, out, bias=None, allow_partials=False):
        y = x.float() @ w.float().T
        if bias is not None:
            y = y + bias
        out.copy_(y.to(out.dtype))
        if allow_partials and out.dtype == torch.float32 and x.shape[0] <= 4:
            # as the K-split tensor-core product does for few tokens: a stack whose sum is the result
            return torch.stack([0.5 * out, 0.25 * out, 0.25 * out])
        return out

    def rope_kv_write(self, qkv, bias, positions, inv_freq, q_out, keys, values, slots,
                      num_heads, num_kv_heads, head_dim, k_out=None, v_out=None):
        if qkv.dim() == 3:
            qkv = qkv.sum(0)
        n = qkv.shape[0]
        x = qkv.float()
        if bias is not None:
            x = x + bias
        qw, kw = num_heads * head_dim, num_kv_heads * head_dim
        q = x[:, :qw].view(n, num_heads, head_dim)
        k = x[:, qw:qw + kw].view(n, num_kv_heads, head_dim)
        v = x[:, qw + kw:].view(n, num_kv_heads, head_dim)
        if inv_freq is not None:
            angle = positions.float()[:, None] * inv_freq[None, :]
            cos = torch.cat([angle.cos(), angle.cos()], -1)[:, None]
            sin = torch.cat([angle.sin(), angle.sin()], -1)[:, None]

            def rot(t):
                a, b = t.chunk(2, -1)
                return t * cos + torch.cat([-b, a], -1) * sin

            q, k = rot(q), rot(k)
        q_out.copy_(q.reshape(n, -1).to(q_out.dtype))
        if k_out is not None:
            k_out.copy_(k.reshape(n, -1).to(k_out.dtype))
            v_out.copy_(v.reshape(n, -1).to(v_out.dtype))
        if keys is not None:
            self.kv_write(k.reshape(n, -1), v.reshape(n, -1), keys, values, slots)

    def kv_write(self, k_new, v_new, keys, values, slots):
        n = k_new.shape[0]
        flat_k = keys.view(-1, keys.shape[-2], keys.shape[-1])
        flat_v = values.view(-1, values.shape[-2], values.shape[-1])
        flat_k[slots.long()] = k_new.view(n, *flat_k.shape[1:]).to(flat_k.dtype)
        flat_v[slots.long()] = v_new.view(n, *flat_v.shape[1:]).to(flat_v.dtype)

    def paged_attention(self, q, keys, values, block_table, q_start, ctx_len, seq_of_token,
                        num_heads, num_kv_heads, head_dim, scale, window, out,
                        max_q_len=0, max_ctx_len=0, min_q_len=0, q_lens=None):
        page = keys.shape[1]
        group = num_heads // num_kv_heads
        n = q.shape[0]
        for token in range(n):
            s = int(seq_of_token[token])
            t = token - int(q_start[s])
            q_len = int(q_start[s + 1]) - int(q_start[s])
            last = int(ctx_len[s]) - q_len + t
            first = 0 if not window else max(0, last - window + 1)
            idx = torch.arange(first, last + 1)
            pages = block_table[s].long()[idx // page]
            assert (pages >= 0).all(), "attention read a page that was given back"
            k = keys[pages, idx % page].float()  # [c, Hkv, D]
            v = values[pages, idx % page].float()
            qt = q[token].float().view(num_kv_heads, group, head_dim)
            scores = torch.einsum("kgd,ckd->kgc", qt, k) * scale
            probs = scores.softmax(-1)
            o = torch.einsum("kgc,ckd->kgd", probs, v)
            out[token] = o.reshape(-1).to(out.dtype)

    def silu_mul(self, gate_up, out):
        inter = out.shape[1]
        g = gate_up[:, :inter].float()
        u = gate_up[:, inter:].float()
        out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def sample(self, logits, temperature, top_p, seeds, out):
        for row in range(logits.shape[0]):
            temp = float(temperature[row])
            if temp == 0.0:
                out[row] = int(torch.argmax(logits[row]))
                continue
            scaled = logits[row].double() / temp
            probs = torch.softmax(scaled, -1)
            p = float(top_p[row])
            keep = torch.ones_like(probs, dtype=torch.bool)
            if p < 1.0:
                sorted_probs, order = probs.sort(descending=True)
                before = sorted_probs.cumsum(-1) - sorted_probs
                keep = torch.zeros_like(keep)
                keep[order] = before < p
            noise = torch.from_numpy(gumbel_noise_host(int(seeds[row]), logits.shape[1])).double()
            score = torch.where(keep, scaled + noise, torch.full_like(scaled, -math.inf))
            out[row] = int(torch.argmax(score))
