"""`shrike_sample_no_alloc`, the sampling entry point for callers that cannot allocate
device memory when they sample (an engine whose key/value pool already owns all free
memory, a step loop that must never reach cudaMalloc or cudaFree, code living inside
another program's memory manager).  Its scratch is a fixed 256 KiB array inside the
library, so it takes at most 256 rows a call.  The test calls it through its exported C
symbol, twice in a row with different inputs (the array keeps what the first call left),
and checks the tokens against `shrike_sample`, the entry point that is given scratch by
its caller; it also checks that a batch beyond the limit is refused with a clear message
and nothing is written.  The file sorts last on purpose, so that a run that stops at the
first failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from shrike_b200.ops import build

    lib = build.core_library()
    lib.shrike_sample_no_alloc.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.shrike_sample_no_alloc.restype = ctypes.c_int
    lib.shrike_sample_no_alloc_message.argtypes = [ctypes.c_int]
    lib.shrike_sample_no_alloc_message.restype = ctypes.c_char_p
    return lib


def _inputs(rows, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, vocab, generator=g) * 3).cuda()
    temperature = torch.tensor([0.0, 0.8, 1.3, 0.0, 0.6][:rows] + [0.9] * max(0, rows - 5)).cuda()
    top_p = torch.tensor([1.0, 1.0, 0.5, 1.0, 0.9][:rows] + [1.0] * max(0, rows - 5)).cuda()
    seeds = (torch.arange(rows, dtype=torch.int64) * 104729 + seed).cuda()
    return logits, temperature, top_p, seeds


def test_no_alloc_sampling_matches_the_allocating_entry_point():
    from shrike_b200.ops.cuda_ops import CudaOps

    lib = _library()
    ops = CudaOps(torch.float32, "cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # a first call: it looks up the array's address (and whatever the driver sets up on the first use
    # of a kernel happens here), so that the calls below can be held to "the device's free memory
    # does not move", which a cudaMalloc behind torch's back would break
    small = _inputs(2, 64, 0)
    first = torch.empty(2, dtype=torch.int32, device="cuda")
    assert lib.shrike_sample_no_alloc(*(t.data_ptr() for t in small), first.data_ptr(), 2, 64, stream) == 0
    torch.cuda.synchronize()
    for rows, vocab, seed in ((7, 152064, 1), (256, 331, 2)):   # two calls in a row share the array
        logits, temperature, top_p, seeds = _inputs(rows, vocab, seed)
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        ops.sample(logits, temperature, top_p, seeds, want)
        got = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        before = (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0])
        code = lib.shrike_sample_no_alloc(logits.data_ptr(), temperature.data_ptr(), top_p.data_ptr(),
                                          seeds.data_ptr(), got.data_ptr(), rows, vocab, stream)
        assert code == 0, lib.shrike_sample_no_alloc_message(code).decode()
        torch.cuda.synchronize()
        assert (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]) == before, "device memory was allocated"
        assert torch.equal(got, want), f"rows={rows} vocab={vocab}"
        assert int(got.min()) >= 0 and int(got.max()) < vocab


def test_no_alloc_sampling_refuses_more_rows_than_its_array_holds():
    lib = _library()
    rows, vocab = 257, 64
    logits, temperature, top_p, seeds = _inputs(rows, vocab, 3)
    out = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    code = lib.shrike_sample_no_alloc(logits.data_ptr(), temperature.data_ptr(), top_p.data_ptr(),
                                      seeds.data_ptr(), out.data_ptr(), rows, vocab,
                                      torch.cuda.current_stream().cuda_stream)
    assert code == -2
    message = lib.shrike_sample_no_alloc_message(code).decode()
    assert "256 rows" in message and "split the batch" in message
    torch.cuda.synchronize()
    assert bool((out == -7).all()), "a refused call must not write its output"
