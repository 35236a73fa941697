"""Inputs made so that a fault shows which random weights would hide: one key far
back among hundreds that must dominate, the edge of a window, and the edge of a page."""

import pytest
import torch

from tests.gpu_common import cuda_ops
from tests.test_gpu_kernels import paged_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def attend(dtype, case, heads, kv_heads, dim, window, q_lens, ctx_lens):
    ops = cuda_ops(dtype)
    out = torch.empty_like(case["q"])
    ops.paged_attention(case["q"], case["keys"], case["values"], case["table"], case["q_start"], case["ctx_len"],
                        case["seq_of"], heads, kv_heads, dim, dim ** -0.5, window, out,
                        max_q_len=max(q_lens), max_ctx_len=max(ctx_lens))
    return out.view(-1, heads, dim).float()


def plant(case, seq, position, page, kv_head, direction, value_mark):
    """Makes key `position` of `seq` point along `direction` (norm 30) and gives its value a mark."""
    pid = int(case["table"][seq, position // page])
    case["keys"][pid, position % page, kv_head] = (direction * 30.0).to(case["keys"].dtype)
    case["values"][pid, position % page, kv_head] = value_mark


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 3, 15, 16, 17, 255, 256, 700, 898])
def test_one_far_key_among_hundreds_dominates(dtype, far):
    heads, kv_heads, dim, page, ctx = 4, 2, 64, 16, 900
    case = paged_case(dtype, heads, kv_heads, dim, page, [ctx, 33], [1, 1], seed=far)
    direction = torch.zeros(dim)
    direction[5] = 1.0
    case["q"].view(-1, heads, dim)[0, :] = (direction * 30.0).to(dtype)   # every head of sequence 0 looks that way
    for kv_head in range(kv_heads):
        plant(case, 0, far, page, kv_head, direction, 7.0)
    out = attend(dtype, case, heads, kv_heads, dim, None, [1, 1], [ctx, 33])
    # score of the planted key is 900 / 8 above the rest: softmax puts all mass there
    assert torch.allclose(out[0], torch.full((heads, dim), 7.0, device=DEV), atol=1e-3), f"key {far} was not found"
    assert not torch.allclose(out[1], torch.full((heads, dim), 7.0, device=DEV), atol=1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 16, 17, 40])
def test_window_edge(dtype, window):
    heads, kv_heads, dim, page, ctx = 2, 1, 32, 16, 100
    direction = torch.zeros(dim)
    direction[0] = 1.0
    for offset, seen in ((window, False), (window - 1, True)):   # just outside / just inside
        case = paged_case(dtype, heads, kv_heads, dim, page, [ctx], [1], seed=window)
        case["q"].view(-1, heads, dim)[0, :] = (direction * 30.0).to(dtype)
        plant(case, 0, ctx - 1 - offset, page, 0, direction, 5.0)
        out = attend(dtype, case, heads, kv_heads, dim, window, [1], [ctx])
        hit = torch.allclose(out[0], torch.full((heads, dim), 5.0, device=DEV), atol=1e-3)
        assert hit == seen, f"window {window}: key at distance {offset} seen={hit}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portion_rows_see_exactly_their_own_past(dtype):
    """In a portion of 20 queries over 52 keys, query t must see key ctx - q_len + t and not the next."""
    heads, kv_heads, dim, page, ctx, q_len = 2, 2, 32, 16, 52, 20
    direction = torch.zeros(dim)
    direction[1] = 1.0
    case = paged_case(dtype, heads, kv_heads, dim, page, [ctx], [q_len], seed=1)
    case["q"].view(-1, heads, dim)[:] = (direction * 30.0).to(dtype)
    planted = ctx - q_len + 7      # the key that the 8th query of the portion brings itself
    for kv_head in range(kv_heads):
        plant(case, 0, planted, page, kv_head, direction, 3.0)
    out = attend(dtype, case, heads, kv_heads, dim, None, [q_len], [ctx])
    mark = torch.full((heads, dim), 3.0, device=DEV)
    for t in range(q_len):
        assert torch.allclose(out[t], mark, atol=1e-3) == (t >= 7), f"query {t}"
