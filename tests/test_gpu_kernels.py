"""Each kernel alone against a plain float64 reference of the same operation, at
sizes other than the engine's tiny models: widths and vocabularies that are no
power of two, head sizes 16..256, odd head counts and groups, context lengths
around page edges."""

import math

import numpy as np
import pytest
import torch

from tests.gpu_common import cuda_ops
from tests.plain import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, atol, rtol=0.0, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all(), what
    bound = atol + rtol * want.abs()
    worst = ((got - want).abs() - bound).max().item()
    assert worst <= 0, f"{what}: exceeds tolerance by {worst:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    ops = cuda_ops(dtype)
    table = rnd(331, 200, dtype=dtype)
    ids = torch.tensor([0, 330, 7, 7, 129], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 200, device=DEV)
    ops.embed(ids, table, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [48, 200, 3584 + 16, 5000, 8192, 8200])
def test_add_rmsnorm(dtype, width):
    ops = cuda_ops(dtype)
    n, eps = 7, 3e-6
    resid, weight = rnd(n, width, seed=1, scale=3.0), 1 + 0.1 * rnd(width, seed=2)
    for delta in (None, rnd(n, width, seed=3), rnd(n, width, seed=4, dtype=torch.bfloat16)):
        x = resid.clone()
        out = torch.empty(n, width, dtype=dtype, device=DEV)
        ops.add_rmsnorm(x, delta, weight, eps, out)
        summed = resid.double() + (0 if delta is None else delta.double())
        close(x, summed, 1e-6, 1e-6, "residual sum")
        want = pm.rms_norm(summed, weight.double(), eps)
        tol = 1e-5 if dtype == torch.float32 else 0.0
        close(out, want, tol, 0 if dtype == torch.float32 else 2 ** -8, f"norm width {width}")
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
        x2 = resid.clone()
        picked = torch.empty(3, width, dtype=dtype, device=DEV)
        ops.gather_add_rmsnorm(x2, delta, rows, weight, eps, picked)
        assert torch.equal(x2, resid), "gather form must not write the residual"
        assert torch.equal(picked, out[rows.long()])


@pytest.mark.parametrize("width", [3584, 5120, 8192, 16384, 1030])
@pytest.mark.parametrize("partials", [3, 8, 11])
@pytest.mark.parametrize("n", [2, 300])
def test_add_rmsnorm_adds_a_stack_of_partials_in_order(width, partials, n):
    """Every form of the kernel (one, two or eight groups per thread, few and many rows, the scalar
    path) adds the slices of a K-split product in ascending order, then the residual: bitwise."""
    ops = cuda_ops(torch.bfloat16)
    resid, weight = rnd(n, width, seed=1, scale=3.0), 1 + 0.1 * rnd(width, seed=2)
    stack = rnd(partials, n, width, seed=5)
    x, out = resid.clone(), torch.empty(n, width, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(x, stack, weight, 1e-6, out)
    total = stack[0].clone()
    for p in range(1, partials):
        total += stack[p]
    total = resid + total
    assert torch.equal(x, total)
    close(out, pm.rms_norm(total.double(), weight.double(), 1e-6), 0.0, 2 ** -8, f"norm of a stack, width {width}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,inter", [(5, 176 + 3), (3, 176), (300, 320), (1, 18944)])   # odd rows: scalar path
def test_silu_mul(dtype, n, inter):
    ops = cuda_ops(dtype)
    gate_up = rnd(n, 2 * inter, dtype=dtype, scale=3.0)
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops.silu_mul(gate_up, out)
    g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    want = g * torch.sigmoid(g) * u
    # bfloat16: one rounding to 8 bits (2^-8) of a float32 value that is itself good to about 2^-20
    close(out, want, 1e-6 if dtype == torch.float32 else 0, 1e-6 if dtype == torch.float32 else 2 ** -8 + 2 ** -20)


@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (33, 65, 17), (64, 64, 16), (70, 331, 240), (130, 96, 1000), (3, 500, 3)])
def test_gemm_fp32_is_true_fp32(m, n, k):
    ops = cuda_ops(torch.float32)
    x, w, bias = rnd(m, k, seed=1), rnd(n, k, seed=2), rnd(n, seed=3)
    out = torch.empty(m, n, device=DEV)
    ops.linear(x, w, out, bias=bias)
    want = x.double() @ w.double().T + bias.double()
    # float32 summation of k terms: the probabilistic rounding bound is
    # sqrt(k) * u * sum|a_i b_i| with u = 2^-24 (Higham & Mary 2019); products rounded to
    # TF32 would be off by about 2^-11 * sqrt(sum (a_i b_i)^2), far above it
    products = x.double().abs() @ w.double().abs().T + bias.double().abs()
    bound = math.sqrt(k) * 2.0 ** -24 * products
    excess = ((out.double() - want).abs() - bound).max().item()
    assert excess <= 0, f"gemm {m}x{n}x{k}: exceeds the float32 bound by {excess:.3e}"
    if k >= 64:
        tf32_error = 2.0 ** -11 * math.sqrt(k) * float((x.double() ** 2).mean().sqrt() * (w.double() ** 2).mean().sqrt())
        assert 5 * bound.mean().item() < tf32_error, "the bound would not tell float32 from TF32"
    # a row's result does not depend on the rows beside it
    alone = torch.empty(1, n, device=DEV)
    ops.linear(x[m - 1:m].contiguous(), w, alone, bias=bias)
    assert torch.equal(alone[0], out[m - 1])


def test_linear_bf16():
    ops = cuda_ops(torch.bfloat16)
    x, w = rnd(9, 240, dtype=torch.bfloat16), rnd(331, 240, dtype=torch.bfloat16)
    wide, narrow = torch.empty(9, 331, device=DEV), torch.empty(9, 331, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, w, wide)
    ops.linear(x, w, narrow)
    want = x.double() @ w.double().T
    close(wide, want, 1e-3, 1e-4)
    close(narrow, want, 1e-3, 2 ** -7)


@pytest.mark.parametrize("tokens,n,k", [(1, 64, 64), (8, 384, 192), (3, 331, 240), (16, 130, 320), (17, 4608, 3584),
                                        (33, 3584, 1000), (64, 256, 18944), (5, 1188, 136), (64, 37888, 3584),
                                        (8, 5120, 5120), (8, 5120, 13824), (4, 1152, 896), (8, 1536, 8960), (2, 10240, 8192)])
def test_gemm_tcgen05(tokens, n, k):
    """The tensor-core product for few tokens (TMA + tcgen05, accumulator in tensor memory):
    float32 and bfloat16 outputs, bias, and the K-split stack of partial results."""
    ops = cuda_ops(torch.bfloat16)
    x, w, bias = rnd(tokens, k, dtype=torch.bfloat16, seed=1), rnd(n, k, dtype=torch.bfloat16, seed=2), rnd(n, seed=3)
    want = x.double() @ w.double().T
    products = x.double().abs() @ w.double().abs().T
    bound = math.sqrt(k) * 2.0 ** -24 * products + 1e-30     # float32 accumulation of exact bf16 products

    def check(got, reference, what, extra=0.0):
        excess = ((got.double() - reference).abs() - bound - extra * reference.abs()).max().item()
        assert excess <= 0, f"gemm_tcgen05 {tokens}x{n}x{k} {what}: exceeds the bound by {excess:.3e}"

    wide = torch.full((tokens, n), float("nan"), device=DEV)
    assert ops.linear(x, w, wide) is wide
    check(wide, want, "float32")
    biased = torch.full((tokens, n), float("nan"), device=DEV)
    ops.linear(x, w, biased, bias=bias)
    check(biased, want + bias.double(), "bias", extra=2.0 ** -23)
    narrow = torch.full((tokens, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear(x, w, narrow)
    check(narrow, want, "bfloat16", extra=2.0 ** -8)
    stack = ops.linear(x, w, wide, bias=bias, allow_partials=True)
    if stack.dim() == 3:
        assert stack.dtype == torch.float32 and stack.shape[1:] == (tokens, n) and stack.shape[0] > 1
        total = stack[0].clone()
        for part in stack[1:]:
            total += part
        check(total, want + bias.double(), "partial stack", extra=2.0 ** -22)
        resid = torch.zeros(tokens, n, device=DEV)
        out = torch.empty(tokens, n, device=DEV)
        ops.add_rmsnorm(resid, stack, torch.ones(n, device=DEV), 1e-6, out)
        assert torch.equal(resid, total), "the norm kernel must add the partials in order"
    ops.check_status()


def test_gemm_tcgen05_splits_keep_their_bounds():
    """How the product cuts K: no empty cut, at least three k-blocks (of 64) a cut, at most 16 cuts, the
    grid of 128-row tiles times cuts resident at once (two CTAs per SM) unless there is a single cut;
    and the choice depends on the matrix alone, never on the number of tokens, so that a position's
    logits do not depend on what else is in the batch."""
    ops = cuda_ops(torch.bfloat16)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    seen = set()
    for n in (64, 128, 896, 1152, 1536, 2048, 2560, 3584, 4608, 5120, 7168, 8192, 10240, 18944, 152064):
        for k in (64, 136, 192, 896, 1000, 1536, 3584, 4864, 5120, 8192, 8960, 13824, 18944, 29568):
            cuts = ops.gemm_tc.shrike_gemm_tc_splits(8, n, k)
            assert all(ops.gemm_tc.shrike_gemm_tc_splits(t, n, k) == cuts for t in (1, 17, 64))
            tiles, kblocks = -(-n // 128), -(-k // 64)
            each = -(-kblocks // cuts)
            assert 1 <= cuts <= 16 and -(-kblocks // each) == cuts
            assert cuts == 1 or (each >= 3 and tiles * cuts <= 2 * sms)
            seen.add(cuts)
    assert ops.gemm_tc.shrike_gemm_tc_splits(8, 3584, 18944) == 8 and ops.gemm_tc.shrike_gemm_tc_splits(8, 5120, 13824) == 7
    assert len(seen) >= 6


def interleave_rows(gate, up, run):
    blocks = gate.shape[0] // run
    return torch.stack([gate.view(blocks, run, -1), up.view(blocks, run, -1)], dim=1).reshape(2 * gate.shape[0], -1).contiguous()


@pytest.mark.parametrize("tokens,inter,k", [(1, 64, 64), (8, 176, 192), (3, 320, 240), (17, 2368, 3584), (33, 1184, 1000),
                                            (64, 128, 18944), (8, 18944, 3584), (64, 18944, 3584)])
def test_gemm_tcgen05_with_the_activation_in_its_epilogue(tokens, inter, k):
    """silu(x Wg^T) * (x Wu^T) in one kernel, over a gate/up matrix whose rows come in runs of 16
    gate rows and their 16 up rows: bit for bit what the product followed by the activation
    kernel gives (on the interleaved and on the plain layout), and close to the exact value."""
    ops = cuda_ops(torch.bfloat16)
    run = ops.gated_rows
    assert run == 16
    x = rnd(tokens, k, dtype=torch.bfloat16, seed=1)
    gate, up = rnd(inter, k, dtype=torch.bfloat16, seed=2, scale=0.05), rnd(inter, k, dtype=torch.bfloat16, seed=3, scale=0.05)
    mixed = interleave_rows(gate, up, run)
    fused = torch.full((tokens, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.linear_gated(x, mixed, fused)
    # the product, then the activation kernel told about the interleaving
    both = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, mixed, both)
    stepwise = torch.empty_like(fused)
    ops.silu_mul(both, stepwise, block=run)
    assert torch.equal(fused, stepwise), "fused epilogue and activation kernel must agree bit for bit"
    # the plain layout: gate rows, then up rows
    plain_both = torch.empty_like(both)
    ops.linear(x, torch.cat([gate, up]).contiguous(), plain_both)
    plain = torch.empty_like(fused)
    ops.silu_mul(plain_both, plain)
    assert torch.equal(fused, plain), "the interleaving must not change a bit"
    # the arithmetic of the epilogue: from the product's own bfloat16 gate and up values (the product
    # itself is checked in test_gemm_tcgen05), one rounding of a float32 value good to about 2^-20
    g, u = plain_both[:, :inter].double(), plain_both[:, inter:].double()
    want = g * torch.sigmoid(g) * u
    assert ((fused.double() - want).abs() <= (2.0 ** -8 + 2.0 ** -20) * want.abs() + 1e-30).all()
    ops.check_status()


def test_activation_kernel_on_interleaved_columns():
    for dtype in (torch.float32, torch.bfloat16):
        ops = cuda_ops(dtype)
        n, inter, run = 37, 320, 16
        gate, up = rnd(n, inter, dtype=dtype, seed=4, scale=2.0), rnd(n, inter, dtype=dtype, seed=5)
        plain = torch.empty(n, inter, dtype=dtype, device=DEV)
        ops.silu_mul(torch.cat([gate, up], dim=1).contiguous(), plain)
        mixed = torch.stack([gate.view(n, inter // run, run), up.view(n, inter // run, run)], dim=2).reshape(n, 2 * inter).contiguous()
        got = torch.empty_like(plain)
        ops.silu_mul(mixed, got, block=run)
        assert torch.equal(got, plain)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim", [(5, 1, 48), (14, 2, 64), (3, 3, 16), (4, 2, 256)])
def test_rope_kv_write(dtype, heads, kv_heads, dim):
    ops = cuda_ops(dtype)
    n, pages, page = 6, 5, 4
    width = (heads + 2 * kv_heads) * dim
    qkv, bias = rnd(n, width, seed=1), rnd(width, seed=2)
    positions = torch.tensor([0, 1, 2, 17, 4000, 123456], dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, dim, 2).float() / dim))).to(DEV)
    slots = torch.tensor([3, 0, 19, 7, 8, 12], dtype=torch.int32, device=DEV)
    keys = torch.full((pages, page, kv_heads, dim), 9.0, dtype=dtype, device=DEV)
    values = torch.full_like(keys, 9.0)
    q = torch.empty(n, heads * dim, dtype=dtype, device=DEV)
    ops.rope_kv_write(qkv, bias, positions, inv_freq, q, keys, values, slots, heads, kv_heads, dim)
    x = (qkv.double() + bias.double()).cpu()
    cos, sin = pm.rope_tables(positions.cpu(), dim, 1e6, torch.float64)
    want_q = pm.apply_rope(x[:, : heads * dim].view(n, heads, dim), cos, sin)
    want_k = pm.apply_rope(x[:, heads * dim: (heads + kv_heads) * dim].view(n, kv_heads, dim), cos, sin)
    want_v = x[:, (heads + kv_heads) * dim:].view(n, kv_heads, dim)
    # the angle is formed in float32 from a float32 table; at position 123456 one ulp of
    # the angle is 8e-3 rad, which bounds how close any float32 implementation can be
    atol = 2e-5 if dtype == torch.float32 else 4e-2
    close(q.view(n, heads, dim)[:4], want_q[:4], atol, 0 if dtype == torch.float32 else 2 ** -8, "q")
    flat_k, flat_v = keys.view(-1, kv_heads, dim), values.view(-1, kv_heads, dim)
    close(flat_k[slots.long()][:4], want_k[:4], atol, 0 if dtype == torch.float32 else 2 ** -8, "k in cache")
    close(flat_v[slots.long()], want_v, 1e-6 if dtype == torch.float32 else 0, 0 if dtype == torch.float32 else 2 ** -8, "v in cache")
    # far positions: compare with the same float32 angle
    angle = positions.float().cpu()[:, None] * inv_freq.cpu()[None, :]
    cos32, sin32 = torch.cat([angle.cos(), angle.cos()], -1).double(), torch.cat([angle.sin(), angle.sin()], -1).double()
    far_q = pm.apply_rope(x[:, : heads * dim].view(n, heads, dim), cos32, sin32)
    close(q.view(n, heads, dim), far_q, 1e-4 if dtype == torch.float32 else 4e-2, 0 if dtype == torch.float32 else 2 ** -8, "q far")
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[slots.long().cpu()] = False
    assert (flat_k[untouched.to(DEV)] == 9.0).all() and (flat_v[untouched.to(DEV)] == 9.0).all()
    # without rotation and without a cache: bias only, into q / k_out / v_out
    k_out = torch.empty(n, kv_heads * dim, dtype=dtype, device=DEV)
    v_out = torch.empty_like(k_out)
    ops.rope_kv_write(qkv, None, positions, None, q, None, None, slots, heads, kv_heads, dim, k_out=k_out, v_out=v_out)
    close(q, qkv[:, : heads * dim], 0, 0 if dtype == torch.float32 else 2 ** -8, "plain q")
    close(k_out, qkv[:, heads * dim: (heads + kv_heads) * dim], 0, 0 if dtype == torch.float32 else 2 ** -8, "plain k")
    keys2, values2 = torch.zeros_like(keys), torch.zeros_like(values)
    ops.kv_write(k_out, v_out, keys2, values2, slots)
    assert torch.equal(keys2.view(-1, kv_heads * dim)[slots.long()], k_out)
    assert torch.equal(values2.view(-1, kv_heads * dim)[slots.long()], v_out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,with_bias", [(5, 1, 48, True), (28, 4, 128, True), (3, 3, 16, False), (4, 2, 256, True)])
def test_rope_kv_write_whole_rows(dtype, heads, kv_heads, dim, with_bias):
    """Many tokens take the form with one block per token, a shared angle table and 16-byte
    accesses; its result is the one the few-token form gives, token by token, bit for bit."""
    ops = cuda_ops(dtype)
    n, page = 300, 16
    pages = -(-n // page) + 2
    width = (heads + 2 * kv_heads) * dim
    qkv, bias = rnd(n, width, seed=5), (rnd(width, seed=6) if with_bias else None)
    g = torch.Generator().manual_seed(7)
    positions = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32).to(DEV)
    slots = torch.randperm(pages * page, generator=g)[:n].to(torch.int32).to(DEV)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, dim, 2).float() / dim))).to(DEV)

    def run(rows):
        keys = torch.full((pages, page, kv_heads, dim), 9.0, dtype=dtype, device=DEV)
        values = torch.full_like(keys, 9.0)
        q = torch.empty(n, heads * dim, dtype=dtype, device=DEV)
        for lo in range(0, n, rows):
            hi = min(n, lo + rows)
            ops.rope_kv_write(qkv[lo:hi].contiguous(), bias, positions[lo:hi].contiguous(), inv_freq, q[lo:hi], keys, values,
                              slots[lo:hi].contiguous(), heads, kv_heads, dim)
        return q, keys, values

    whole, few = run(n), run(7)
    for got, want, what in zip(whole, few, ("q", "keys", "values")):
        assert torch.equal(got, want), what
    x = qkv.double().cpu() + (bias.double().cpu() if with_bias else 0)
    angle = positions.float().cpu()[:, None] * inv_freq.cpu()[None, :]
    cos32, sin32 = torch.cat([angle.cos(), angle.cos()], -1).double(), torch.cat([angle.sin(), angle.sin()], -1).double()
    want_q = pm.apply_rope(x[:, : heads * dim].view(n, heads, dim), cos32, sin32)
    close(whole[0].view(n, heads, dim), want_q, 1e-4 if dtype == torch.float32 else 4e-2, 0 if dtype == torch.float32 else 2 ** -8, "q")


def paged_case(dtype, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=0):
    """Random sequences scattered over distinct, shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-c // page) for c in ctx_lens) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    keys = torch.full((total_pages, page, kv_heads, dim), float("nan"), dtype=dtype)
    values = torch.full_like(keys, float("nan"))
    max_blocks = max(-(-c // page) for c in ctx_lens)
    table = torch.full((len(ctx_lens), max_blocks), -1, dtype=torch.int32)
    seqs, q_rows, seq_of, q_start = [], [], [], [0]
    for s, (ctx, q_len) in enumerate(zip(ctx_lens, q_lens)):
        k = torch.randn(ctx, kv_heads, dim, generator=g).to(dtype)
        v = torch.randn(ctx, kv_heads, dim, generator=g).to(dtype)
        q = torch.randn(ctx, heads, dim, generator=g).to(dtype)
        for b in range(-(-ctx // page)):
            pid = order.pop()
            table[s, b] = pid
            rows = slice(b * page, min(ctx, (b + 1) * page))
            keys[pid, : rows.stop - rows.start] = k[rows]
            values[pid, : rows.stop - rows.start] = v[rows]
        seqs.append((q, k, v))
        q_rows.append(q[ctx - q_len:])
        seq_of += [s] * q_len
        q_start.append(q_start[-1] + q_len)
    return dict(
        keys=keys.to(DEV), values=values.to(DEV), table=table.to(DEV), seqs=seqs,
        q=torch.cat(q_rows).reshape(-1, heads * dim).contiguous().to(DEV),
        q_start=torch.tensor(q_start, dtype=torch.int32, device=DEV),
        ctx_len=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
        seq_of=torch.tensor(seq_of, dtype=torch.int32, device=DEV),
    )


def run_attention(ops, case, heads, kv_heads, dim, window, q_lens, ctx_lens):
    out = torch.empty_like(case["q"])
    ops.paged_attention(case["q"], case["keys"], case["values"], case["table"], case["q_start"], case["ctx_len"],
                        case["seq_of"], heads, kv_heads, dim, dim ** -0.5, window, out,
                        max_q_len=max(q_lens), max_ctx_len=max(ctx_lens), min_q_len=min(q_lens),
                        q_lens=list(q_lens) if sum(ctx_lens) % 2 else None)   # with and without the exact CTA count
    want = []
    for (q, k, v), q_len in zip(case["seqs"], q_lens):   # the oracle runs on the GPU in float64: plain torch all the same
        want.append(pm.causal_attention(q[len(q) - q_len:].double().to(DEV), k.double().to(DEV), v.double().to(DEV), window))
    return out, torch.cat(want).reshape(out.shape)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,page", [(14, 2, 64, 16), (5, 1, 48, 16), (6, 3, 32, 8), (2, 2, 256, 16), (7, 7, 16, 4), (28, 4, 128, 16),
                                                     (34, 2, 32, 16), (40, 1, 80, 3)])
def test_paged_attention_single_tokens_around_page_edges(dtype, heads, kv_heads, dim, page):
    ops = cuda_ops(dtype)
    ctx_lens = [1, 15, 16, 17, 100, 333, 512, 7]   # shrike tests/test_triton_attention.py:35-37
    q_lens = [1] * len(ctx_lens)
    case = paged_case(dtype, heads, kv_heads, dim, page, ctx_lens, q_lens)
    got, want = run_attention(ops, case, heads, kv_heads, dim, None, q_lens, ctx_lens)
    close(got, want, 2e-5 if dtype == torch.float32 else 2e-2, 0, "decode attention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 1, 16, 50])
@pytest.mark.parametrize("heads,kv_heads,dim,page", [(6, 2, 64, 16), (17, 1, 112, 5), (8, 2, 128, 16), (6, 3, 64, 8), (4, 4, 128, 64)])
def test_paged_attention_portions_mixed_with_single_tokens(dtype, window, heads, kv_heads, dim, page):
    ops = cuda_ops(dtype)
    ctx_lens = [40, 1, 130, 2, 16, 17, 300, 64, 33]
    q_lens = [1, 1, 1, 2, 16, 3, 129, 64, 17]
    case = paged_case(dtype, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=4)
    if window is not None:  # pages the window has passed are gone: the kernel must not touch them
        for s, (ctx, q_len) in enumerate(zip(ctx_lens, q_lens)):
            first_needed = max(0, ctx - q_len - window + 1)
            for b in range(first_needed // page):
                pid = int(case["table"][s, b])
                case["keys"][pid] = float("nan")
                case["table"][s, b] = -1
    got, want = run_attention(ops, case, heads, kv_heads, dim, window, q_lens, ctx_lens)
    close(got, want, 2e-5 if dtype == torch.float32 else 2e-2, 0, f"mixed attention window {window}")


def drop_passed_pages(case, page, window, ctx_lens, q_lens):
    """Pages that every query's window has passed are gone: the kernel must not touch them."""
    for s, (ctx, q_len) in enumerate(zip(ctx_lens, q_lens)):
        first_needed = max(0, ctx - q_len - window + 1)
        for b in range(first_needed // page):
            pid = int(case["table"][s, b])
            case["keys"][pid] = float("nan")
            case["values"][pid] = float("nan")
            case["table"][s, b] = -1


# the lengths a serving run brings: a whole 2,048-token prompt, portions of 512 over a long cached
# prefix, a window, and portions beside single tokens; at the head sizes of the tensor-core kernel
SERVED = {
    "prompt_2048": ([2048], [2048], None),
    "512_over_1536": ([2048], [512], None),
    "512_over_3584": ([4096], [512], None),
    "window_1000": ([2048, 1500], [512, 300], 1000),
    "two_portions_beside_eight_single_tokens": (
        [1024, 777, 1, 2048, 513, 64, 1000, 1100, 2048, 1000], [1, 1, 1, 1, 1, 1, 1, 1, 512, 300], None),
    "ragged_edges": ([2047, 129, 1153], [2047, 65, 127], None),
    # a CTA's two chains of 128 rows: a second chain of one row, of none, of all; first rows at positions that
    # are no multiple of the key step, so that the two chains' last keys fall into the same or into different steps
    "chain_edges": ([300, 334, 133, 900, 256, 131], [129, 257, 128, 385, 256, 2], None),
    "chain_edges_window": ([300, 334, 700, 900], [129, 257, 300, 385], 100),
}


@pytest.mark.parametrize("name", list(SERVED))
@pytest.mark.parametrize("splits", [0, 1, 3, 7])
@pytest.mark.parametrize("heads,kv_heads,dim,page", [(28, 4, 128, 16), (14, 2, 64, 16), (12, 2, 128, 32), (5, 1, 64, 8), (6, 2, 128, 64)])
def test_portions_attention_at_served_lengths(name, heads, kv_heads, dim, page, splits):
    """The tensor-core kernel for portions over walks of up to 64 key tiles (its rescaling of the
    running sum, its look-ahead in the block table and its first and last tile only matter on
    long walks), against the plain formula in float64; with the keys of a query tile walked by one
    CTA, shared by as many as the library's rule says (0), or by 3 or 7 (splits that see no key,
    and rows whose keys all lie in other splits, among them)."""
    ctx_lens, q_lens, window = SERVED[name]
    ops = cuda_ops(torch.bfloat16)
    ops.portion_splits = splits
    lib = ops._attention_lib(dim)
    assert lib.shrike_attention_tc_available()
    case = paged_case(torch.bfloat16, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=11)
    if window is not None:
        drop_passed_pages(case, page, window, ctx_lens, q_lens)
    got, want = run_attention(ops, case, heads, kv_heads, dim, window, q_lens, ctx_lens)
    close(got, want, 2e-2, 0, f"{name} heads {heads}/{kv_heads} D {dim} page {page}")
    ops.check_status()


def test_a_portion_beside_decoding_requests_is_split_over_the_gpu():
    """The rule: the query tiles of 492 new tokens of 12 heads over block tables of 2,048 keys would
    occupy a fraction of the GPU; their keys are shared out as far as every CTA still starts at once
    (one per SM), never fewer than two key steps a split.  A whole prompt, whose query tiles of 28
    heads outnumber the SMs, is not split at any length."""
    ops = cuda_ops(torch.bfloat16)
    lib = ops._attention_lib(128)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows, keys = lib.shrike_attention_tc_portions_rows(), 128
    assert rows in (128, 256)
    tiles = -(-492 // rows)
    splits = lib.shrike_attention_tc_portions_splits(512, 12, 128, 16, tiles)
    assert 2 <= splits <= 16 and (2048 // keys) // splits >= 2
    assert 12 * tiles * splits <= sms                                            # one round, one CTA per SM
    for prompt in (2048, 4096, 8192):
        assert lib.shrike_attention_tc_portions_splits(prompt, 28, prompt // 16, 16, prompt // rows) == 1
    assert lib.shrike_attention_tc_portions_splits(64, 2, 8, 16, 1) == 1         # one key step in all
    assert lib.shrike_attention_tc_portions_splits(64, 2, 4096, 16, 1) == 16     # never more than 16
    assert lib.shrike_attention_tc_portions_scratch_floats(512, 12, 4) == 4 * 512 * 12 * 130


def test_portions_attention_finds_a_far_key_among_thousands():
    """One key far back is made to stand out for one query row (its score is large), so the
    output of that row must be that key's value: a tile walked in the wrong order, a page looked up
    a tile too late or a rescale that is skipped would blur it."""
    ops = cuda_ops(torch.bfloat16)
    heads, kv_heads, dim, page = 28, 4, 128, 16
    ctx_lens, q_lens = [4096], [512]
    case = paged_case(torch.bfloat16, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=13)
    q, k, v = case["seqs"][0]
    for far_key, row in ((3, 500), (1031, 17), (3583, 0), (3600, 40), (2050, 511)):
        direction = torch.zeros(dim)
        direction[far_key % dim] = 1.0
        k[far_key] = (14.0 * direction).to(torch.bfloat16)                       # every kv head
        q[4096 - 512 + row] = (14.0 * direction).to(torch.bfloat16)                # every head: score 196 * D^-0.5 = 17.3
        pid, at = int(case["table"][0, far_key // page]), far_key % page
        case["keys"][pid, at] = k[far_key].to(DEV)
    case["q"] = q[4096 - 512:].reshape(512, heads * dim).contiguous().to(DEV)
    got, want = run_attention(ops, case, heads, kv_heads, dim, None, q_lens, ctx_lens)
    close(got, want, 2e-2, 0, "far keys")
    group = heads // kv_heads
    for far_key, row in ((3, 500), (1031, 17), (3583, 0), (3600, 40), (2050, 511)):
        for head in (0, 13, 27):
            # the far key holds all but 3e-4 of the mass (its score leads by 17 over N(0, 1.2) scores)
            close(got[row].view(heads, dim)[head], v[far_key, head // group].double(), 0.05, 0, f"row {row} key {far_key}")


def test_single_token_attention_twice_in_a_row_leaves_its_counters_clean():
    """The split counters must be zero again after a launch: a second launch with other data
    gives that data's result."""
    ops = cuda_ops(torch.bfloat16)
    heads, kv_heads, dim, page = 28, 4, 128, 16
    for seed, ctx_lens in ((1, [700, 64, 65, 1023]), (2, [1, 300, 1024, 129, 17])):
        q_lens = [1] * len(ctx_lens)
        case = paged_case(torch.bfloat16, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=seed)
        got, want = run_attention(ops, case, heads, kv_heads, dim, None, q_lens, ctx_lens)
        close(got, want, 2e-2, 0, f"launch with seed {seed}")
    assert int(ops._arrivals.abs().sum()) == 0


@pytest.mark.parametrize("splits,cluster", [(1, 1), (3, 1), (2, 2), (4, 4), (8, 8), (6, 2), (16, 8), (24, 8), (12, 4)])
@pytest.mark.parametrize("heads,kv_heads,dim,page", [(28, 4, 128, 16), (5, 1, 48, 16), (40, 2, 64, 8)])
def test_single_token_attention_under_every_split_and_cluster_shape(splits, cluster, heads, kv_heads, dim, page, monkeypatch):
    """Clusters add their splits up on chip, more clusters meet in global memory; the result
    is the same attention whichever way the keys are cut, including splits with no keys."""
    ops = cuda_ops(torch.bfloat16)
    monkeypatch.setattr(ops, "single_token_splits", lambda tiles, groups, resident: (splits, cluster))
    ctx_lens = [1, 64, 65, 700, 1500, 130]
    q_lens = [1] * len(ctx_lens)
    for seed in (5, 6):   # twice: the arrival counters are left clean
        case = paged_case(torch.bfloat16, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=seed)
        got, want = run_attention(ops, case, heads, kv_heads, dim, None, q_lens, ctx_lens)
        close(got, want, 2e-2, 0, f"splits {splits} cluster {cluster}")
    assert int(ops._arrivals.abs().sum()) == 0


@pytest.mark.parametrize("window", [None, 40])
@pytest.mark.parametrize("heads,kv_heads,dim,page", [(28, 4, 128, 16), (40, 2, 64, 8), (4, 2, 256, 64), (8, 2, 128, 32), (6, 3, 64, 16)])
def test_single_token_attention_by_pages_and_by_copies(heads, kv_heads, dim, page, window):
    """Head sizes that are multiples of 64 with pages of 8 to 64 tokens load whole pages through
    tensor maps; the same launch can be made to copy row by row.  Both give the attention of the
    plain formula, on a pool whose unwritten slots hold NaN, with a window that has let pages go."""
    ops = cuda_ops(torch.bfloat16)
    lib = ops._attention_lib(dim)
    ctx_lens = [1, 63, 64, 65, 129, 700, 1500, 2100]
    q_lens = [1] * len(ctx_lens)
    case = paged_case(torch.bfloat16, heads, kv_heads, dim, page, ctx_lens, q_lens, seed=9)
    if window is not None:   # pages the window has passed are gone: the kernel must not touch them
        for s, ctx in enumerate(ctx_lens):
            for b in range(max(0, ctx - window) // page):
                case["keys"][int(case["table"][s, b])] = float("nan")
                case["values"][int(case["table"][s, b])] = float("nan")
                case["table"][s, b] = -1
    results = {}
    try:
        for form, enabled in (("pages", 1), ("copies", 0)):
            lib.shrike_attention_single_token_pages(enabled)
            got, want = run_attention(ops, case, heads, kv_heads, dim, window, q_lens, ctx_lens)
            close(got, want, 2e-2, 0, f"single tokens by {form}")
            results[form] = got.clone()
    finally:
        lib.shrike_attention_single_token_pages(1)
    close(results["pages"], results["copies"].double(), 2e-2, 0, "the two forms")
    ops.check_status()


def test_widths_beyond_one_block_are_refused_not_miscomputed():
    from shrike_b200.ops.cuda_ops import KernelError

    ops = cuda_ops(torch.float32)
    width = 32768 + 4
    resid = torch.zeros(2, width, device=DEV)
    with pytest.raises(KernelError, match="add_rmsnorm"):
        ops.add_rmsnorm(resid, None, torch.ones(width, device=DEV), 1e-6, torch.empty(2, width, device=DEV))


def test_head_sizes_outside_the_served_range_are_refused():
    from shrike_b200.ops.cuda_ops import KernelError

    ops = cuda_ops(torch.float32)
    for bad in (8, 24, 272, 100):
        with pytest.raises(KernelError, match="head size"):
            ops.check_head_dim(bad)


def test_sampling_greedy_takes_the_lowest_index_on_ties():
    ops = cuda_ops(torch.float32)
    vocab = 152064 + 5
    logits = rnd(3, vocab, seed=1)
    logits[0, 70000] = 50.0
    logits[0, 9] = 50.0
    logits[1, vocab - 1] = 60.0
    logits[2] = -3.0   # all equal
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(3, device=DEV)
    ops.sample(logits, zeros, torch.ones(3, device=DEV), torch.zeros(3, dtype=torch.int64, device=DEV), out)
    assert out.tolist() == [9, vocab - 1, 0]


def test_sampling_follows_the_distribution_and_top_p():
    ops = cuda_ops(torch.float32)
    vocab, draws = 331, 4000
    g = torch.Generator().manual_seed(3)
    row = torch.randn(vocab, generator=g) * 2.0
    logits = row.to(DEV).repeat(draws, 1).contiguous()
    seeds = torch.arange(draws, dtype=torch.int64, device=DEV) * 7919 + 13
    out = torch.empty(draws, dtype=torch.int32, device=DEV)
    temp = torch.full((draws,), 0.8, device=DEV)
    ops.sample(logits, temp, torch.ones(draws, device=DEV), seeds, out)
    probs = pm.softmax_with_temperature(row, 0.8)
    counts = torch.bincount(out.long().cpu(), minlength=vocab).double()
    top = probs.argsort(descending=True)[:10]
    for token in top.tolist():   # binomial: five standard deviations
        p = float(probs[token])
        assert abs(counts[token] - draws * p) < 5 * math.sqrt(draws * p * (1 - p)) + 1, token
    # same seeds, same tokens, whatever the row or the batch size
    again = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.sample(logits[:5], temp[:5], torch.ones(5, device=DEV), seeds[[9, 3, 3, 0, 1]].contiguous(), again)
    assert again.tolist() == [out[9].item(), out[3].item(), out[3].item(), out[0].item(), out[1].item()]
    # top_p: nothing outside the nucleus is ever drawn, everything inside can be
    for top_p in (0.3, 0.9):
        keep = pm.top_p_keep(probs, top_p)
        ops.sample(logits, temp, torch.full((draws,), top_p, device=DEV), seeds, out)
        drawn = set(out.tolist())
        kept = set(torch.nonzero(keep).flatten().tolist())
        assert drawn <= kept, f"top_p {top_p}: drew {sorted(drawn - kept)} outside the nucleus"
        likely = {t for t in kept if float(probs[t]) * draws > 30}
        assert likely <= drawn
    # a dominant token with a tiny top_p is always taken (shrike tests/test_sampler.py)
    ops.sample(logits[:8], temp[:8], torch.full((8,), 1e-6, device=DEV), seeds[:8].contiguous(), out[:8])
    assert set(out[:8].tolist()) == {int(probs.argmax())}


def test_sampling_a_row_without_a_finite_logit_gives_a_valid_token_and_says_so():
    """NaN compares with nothing, so such a row has no winner: the kernels return token 0 for it
    (a valid id) and leave their code in the status word; rows beside it are not disturbed."""
    from shrike_b200.ops.cuda_ops import KernelError

    ops = cuda_ops(torch.float32)
    vocab = 5000
    logits = rnd(4, vocab, seed=3)
    logits[1] = float("nan")
    logits[3, ::2] = float("nan")   # half NaN: the finite half decides
    temperature = torch.tensor([0.0, 0.0, 0.7, 0.0], device=DEV)
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0], device=DEV)
    seeds = torch.arange(4, dtype=torch.int64, device=DEV)
    out = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    ops.sample(logits, temperature, top_p, seeds, out)
    got = out.tolist()
    assert got[1] == 0 and got[0] == int(logits[0].argmax()) and 0 <= got[2] < vocab
    assert got[3] == int(torch.nan_to_num(logits[3], nan=-1e30).argmax()) and got[3] % 2 == 1
    with pytest.raises(KernelError, match="no finite element"):
        ops.check_status()
    ops.check_status()   # cleared by the raise


def test_sampling_mixes_greedy_and_sampled_rows():
    ops = cuda_ops(torch.float32)
    logits = rnd(4, 1000, seed=5)
    temp = torch.tensor([0.0, 1.0, 0.0, 0.7], device=DEV)
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, torch.ones(4, device=DEV), torch.tensor([1, 2, 3, 4], dtype=torch.int64, device=DEV), out)
    assert out[0].item() == int(logits[0].argmax()) and out[2].item() == int(logits[2].argmax())
    assert 0 <= out[1].item() < 1000 and 0 <= out[3].item() < 1000


@pytest.mark.parametrize("new,ctx_len,window", [(512, 30000, None), (300, 20000, 4096), (2048, 16384, None)])
def test_portions_attention_over_very_long_walks(new, ctx_len, window):
    """Hundreds of key steps per CTA (every barrier of the tensor-core kernel changes its parity
    hundreds of times, the page ids come in dozens of chunks, the rule splits the keys where query
    tiles are few) against the float32 kernel on the same bfloat16 inputs; that kernel is itself
    checked against float64 at the smaller sizes above."""
    heads, kv_heads, dim, page = 28, 4, 128, 16
    g = torch.Generator(device=DEV).manual_seed(new)
    blocks = -(-ctx_len // page)
    pages = blocks + 8
    order = torch.randperm(pages, device=DEV, generator=g)[:blocks].to(torch.int32)
    keys = torch.randn(pages, page, kv_heads, dim, device=DEV, dtype=torch.bfloat16, generator=g)
    values = torch.randn(pages, page, kv_heads, dim, device=DEV, dtype=torch.bfloat16, generator=g)
    q = torch.randn(new, heads * dim, device=DEV, dtype=torch.bfloat16, generator=g)
    table = torch.full((1, blocks + 3), -1, dtype=torch.int32, device=DEV)
    table[0, :blocks] = order
    q_start = torch.tensor([0, new], dtype=torch.int32, device=DEV)
    ctx = torch.tensor([ctx_len], dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(new, dtype=torch.int32, device=DEV)
    ops = cuda_ops(torch.bfloat16)
    assert ops._attention_lib(dim).shrike_attention_tc_available()
    got = torch.empty_like(q)
    ops.paged_attention(q, keys, values, table, q_start, ctx, seq_of, heads, kv_heads, dim, dim ** -0.5, window, got,
                        max_q_len=new, min_q_len=new, q_lens=[new])
    ops.check_status()
    exact = cuda_ops(torch.float32)
    want = torch.empty(new, heads * dim, device=DEV)
    exact.paged_attention(q.float(), keys.float(), values.float(), table, q_start, ctx, seq_of, heads, kv_heads, dim,
                          dim ** -0.5, window, want, max_q_len=new, min_q_len=new)
    close(got, want, 2e-3, 0, f"{new} new tokens over {ctx_len}")
