"""The kernels, as one object the parts call.

Every method launches hand-written sm_100a code from `csrc/` through the C symbol
of its launcher, on torch's current stream, with raw device pointers.  There is no
CPU path and no library attention or model code: without a CUDA device, or when a
kernel cannot be built, construction fails.  Matrix products in bfloat16 run on this
package's tcgen05 kernel for up to 64 tokens (decoding) and go to cuBLAS through
`torch.mm` above that (Azimml/shrike's own GEMMs are cuBLAS calls through nn.Linear,
shrike/models/qwen.py:111-136); in float32 they run on this package's own FFMA
kernel, so the 32-bit path never touches a reduced-precision matrix mode.
"""

from __future__ import annotations

import ctypes

import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_c = ctypes
_P, _I, _F, _LL = _c.c_void_p, _c.c_int, _c.c_float, _c.c_longlong


class KernelError(RuntimeError):
    pass


class AttentionPlan:
    """What `CudaOps.attention_plan` decides for a batch shape."""

    __slots__ = ("has_single", "has_portions", "tc_portions", "splits", "cluster", "scratch", "arrivals",
                 "portion_splits", "portion_scratch")

    def __init__(self, has_single, has_portions, tc_portions, splits, cluster, scratch, arrivals,
                 portion_splits=1, portion_scratch=None):
        self.has_single, self.has_portions, self.tc_portions = has_single, has_portions, tc_portions
        self.splits, self.cluster, self.scratch, self.arrivals = splits, cluster, scratch, arrivals
        self.portion_splits, self.portion_scratch = portion_splits, portion_scratch   # the tensor-core portions kernel's key splits


def _ptr(tensor):
    return None if tensor is None else tensor.data_ptr()


_LIMITS = {
    "add_rmsnorm": "the row width must be at most 32768 (8192 when it is no multiple of 4)",
    "gather_add_rmsnorm": "the row width must be at most 32768 (8192 when it is no multiple of 4)",
    "gemm_tcgen05": "K must be a multiple of 8 and the operands 16-byte aligned",
    "paged_attention_bf16": "at most 65535 sequences and heads, heads a multiple of kv heads, at most 32 splits",
}


def _check(code: int, what: str):
    if code != 0:
        reason = f"bad argument ({_LIMITS[what]})" if code == -1 and what in _LIMITS else (
            "bad argument" if code == -1 else f"CUDA error {code}")
        raise KernelError(f"{what}: {reason}")


def _dense(tensor, dtype, what):
    if tensor.device.type != "cuda":
        raise KernelError(f"{what} must be on the GPU, is on {tensor.device}")
    if tensor.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, is {tensor.dtype}")
    if not tensor.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


class CudaOps:
    PORTION_SCRATCH_FLOATS = 32 << 20   # at most 128 MiB of partial rows for the split portions kernel

    def __init__(self, dtype: torch.dtype, device="cuda"):
        if dtype not in _DTYPE_CODE:
            raise KernelError(f"no kernels for {dtype}; bfloat16 and float32 are served")
        if not torch.cuda.is_available():
            raise KernelError("shrike_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        self.dtype = dtype
        self.code = _DTYPE_CODE[dtype]
        self.device = torch.device(device)
        self.core = build.core_library()
        self._declare_core()
        self._attention = {}
        self.gemm_tc = None
        self.tensor_core_attention = True   # tcgen05 kernel for portions where the head and page sizes allow
        self.tensor_core_gemm_max_tokens = 64   # above this the library product is used
        self._partials = {}      # data_ptr of an output buffer -> its stack of K-split partial results
        # one host-visible word (of four): the first kernel whose bounded wait ran out, or that met
        # a row without a finite logit, leaves its code here; see `describe_status`
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        if dtype == torch.bfloat16:
            self.gemm_tc = build.tensor_core_gemm_library()
            self.gemm_tc.shrike_gemm_tc.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]
            self.gemm_tc.shrike_gemm_tc.restype = _I
            self.gemm_tc.shrike_gemm_tc_gated.argtypes = [_P, _P, _P, _I, _I, _I, _P, _P]
            self.gemm_tc.shrike_gemm_tc_gated.restype = _I
            self.gemm_tc.shrike_gemm_tc_splits.argtypes = [_I, _I, _I]
            self.gemm_tc.shrike_gemm_tc_splits.restype = _I
        self._scratch = None     # partial results of split single-token attention
        self._sample_scratch = None  # per-slice winners of the sampling kernel
        self._arrivals = None    # per kv head: splits of single-token attention that have finished
        self._portion_scratch = None   # partial rows of the portions kernel when a query tile's keys are split
        self._portion_tiles = None
        self.portion_splits = 0  # 0: the kernel library's rule; n: that many key splits for portions (tests)
        self.generation = 0      # grows when the scratch moves
        self._held_stream = None
        self._layer_program = None   # the native per-layer issue, built on first use
        self.native_layers = True    # whole layers are issued by one native call where the parts allow it
        self.launches = 0        # launches of this package's own kernels
        self.library_calls = 0   # matrix products handed to cuBLAS
        # library matrix products keep float32 accumulation end to end: no TF32 for float32
        # inputs, no bfloat16 partial sums when a bfloat16 product is split along K
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # ---- declarations -------------------------------------------------------
    def _declare_core(self):
        lib = self.core
        lib.shrike_embed.argtypes = [_P, _P, _I, _P, _I, _I, _I, _P, _I, _P]
        lib.shrike_add_rmsnorm.argtypes = [_P, _P, _I, _P, _P, _F, _P, _I, _I, _I, _I, _LL, _P]
        lib.shrike_silu_mul.argtypes = [_P, _P, _I, _I, _I, _I, _P]
        lib.shrike_rope_kv_write.argtypes = [_P] * 10 + [_I] * 5 + [_LL, _I, _LL, _P]
        lib.shrike_kv_write.argtypes = [_P] * 5 + [_I, _I, _I, _LL, _P]
        lib.shrike_gemm_fp32.argtypes = [_P, _P, _P, _P, _I, _I, _I, _P]
        lib.shrike_sample.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _P]
        lib.shrike_sample_slices.argtypes = [_I]
        lib.shrike_sample_slices.restype = _I
        for name in ("shrike_embed", "shrike_add_rmsnorm", "shrike_silu_mul", "shrike_rope_kv_write",
                     "shrike_kv_write", "shrike_gemm_fp32", "shrike_sample"):
            getattr(lib, name).restype = _I

    def _attention_lib(self, head_dim: int):
        lib = self._attention.get(head_dim)
        if lib is None:
            self.check_head_dim(head_dim)
            lib = build.attention_library(head_dim)
            lib.shrike_paged_attention_generic.argtypes = (
                [_P, _P, _P, _P, _I, _P, _P, _P] + [_I] * 6 + [_F, _I, _P, _P]
            )
            lib.shrike_paged_attention_generic.restype = _I
            lib.shrike_paged_attention_bf16.argtypes = (
                [_P, _P, _P, _P, _I, _P, _P] + [_I] * 5 + [_F, _I, _P] + [_I] * 5 + [_P, _P, _P, _P]
            )
            lib.shrike_paged_attention_bf16.restype = _I
            lib.shrike_attention_single_token_pages.argtypes = [_I]
            lib.shrike_attention_single_token_pages.restype = None
            lib.shrike_attention_bf16_resident_ctas.restype = _I
            lib.shrike_attention_tc_available.restype = _I
            lib.shrike_paged_attention_tc_portions.argtypes = (
                [_P, _P, _P, _P, _I, _P, _P] + [_I] * 6 + [_F, _I, _P, _I, _I, _P, _I, _P, _I, _P, _P]
            )
            lib.shrike_paged_attention_tc_portions.restype = _I
            lib.shrike_attention_tc_portions_rows.restype = _I
            lib.shrike_attention_tc_portions_splits.argtypes = [_I, _I, _I, _I, _I]
            lib.shrike_attention_tc_portions_splits.restype = _I
            lib.shrike_attention_tc_portions_scratch_floats.argtypes = [_I, _I, _I]
            lib.shrike_attention_tc_portions_scratch_floats.restype = _LL
            self._attention[head_dim] = lib
        return lib

    def _stream(self):
        return self._held_stream if self._held_stream is not None else torch.cuda.current_stream().cuda_stream

    def hold_stream(self, hold: bool) -> None:
        """Between `hold_stream(True)` and `hold_stream(False)` every launch goes to the stream
        that was current at the first call, looked up once: asking torch for the current stream
        costs more than a launch.  The step function brackets a forward pass with it."""
        self._held_stream = torch.cuda.current_stream().cuda_stream if hold else None

    def check_head_dim(self, head_dim: int):
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(
                f"head size {head_dim} is not served: the attention kernels take multiples of 16 from 16 to 256"
            )

    def layer_program(self):
        """The native per-layer issue (`ops/layer_program.py`), or None when it is switched off."""
        if not self.native_layers or self.dtype != torch.bfloat16:
            return None
        if self._layer_program is None:
            from .layer_program import LayerProgram

            self._layer_program = LayerProgram(self)
        return self._layer_program

    # ---- kernels ------------------------------------------------------------
    def embed(self, ids, table, out, previous=None):
        """Rows of `table` into the float32 residual.  An id of -1 - r is replaced on the device
        by `previous[r]` (int32: the tokens the step before drew)."""
        _dense(ids, torch.int32, "token ids")
        _dense(out, torch.float32, "residual")
        n, width = out.shape
        if previous is not None:
            _dense(previous, torch.int32, "previous tokens")
        self.launches += 1
        _check(self.core.shrike_embed(_ptr(ids), _ptr(table), _DTYPE_CODE[table.dtype], _ptr(out), n, width,
                                      table.shape[0], _ptr(previous), 0 if previous is None else previous.numel(),
                                      self._stream()), "embed")

    @staticmethod
    def _stack(delta):
        """(partials, stride in elements) of a [N, W] array or a [P, N, W] stack of partial sums."""
        if delta is None or delta.dim() == 2:
            return 1, 0
        return delta.shape[0], delta.stride(0)

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        """resid += delta (a [N, W] array, or a [P, N, W] stack added in order); out = norm(resid) * weight."""
        _dense(resid, torch.float32, "residual")
        _dense(weight, torch.float32, "norm weight")
        n, width = resid.shape
        code = -1 if delta is None else _DTYPE_CODE[delta.dtype]
        partials, stride = self._stack(delta)
        self.launches += 1
        _check(self.core.shrike_add_rmsnorm(_ptr(resid), _ptr(delta), code, None, _ptr(weight), eps, _ptr(out),
                                            _DTYPE_CODE[out.dtype], n, width, partials, stride, self._stream()),
               "add_rmsnorm")

    def gather_add_rmsnorm(self, resid, delta, rows, weight, eps, out):
        _dense(resid, torch.float32, "residual")
        _dense(rows, torch.int32, "rows")
        width = resid.shape[1]
        code = -1 if delta is None else _DTYPE_CODE[delta.dtype]
        partials, stride = self._stack(delta)
        self.launches += 1
        _check(self.core.shrike_add_rmsnorm(_ptr(resid), _ptr(delta), code, _ptr(rows), _ptr(weight), eps,
                                            _ptr(out), _DTYPE_CODE[out.dtype], rows.shape[0], width, partials,
                                            stride, self._stream()), "gather_add_rmsnorm")

    def linear(self, x, w, out, bias=None, allow_partials=False):
        """x[N, K] @ w[O, K]^T (+ bias) into `out` [N, O] (float32 or the activation type).

        Returns the array to consume: `out`, or, when `allow_partials` and the product was
        split along K, a float32 stack [P, N, O] whose sum over P is the result (the
        norm and rotary kernels add such stacks themselves)."""
        n, k = x.shape
        o = w.shape[0]
        if w.shape[1] != k or tuple(out.shape) != (n, o):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        if self.dtype == torch.float32:
            self.launches += 1
            _dense(x, torch.float32, "linear input")
            _dense(w, torch.float32, "linear weight")
            _dense(out, torch.float32, "linear output")
            _check(self.core.shrike_gemm_fp32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), n, o, k, self._stream()),
                   "gemm_fp32")
            return out
        _dense(x, torch.bfloat16, "linear input")
        _dense(w, torch.bfloat16, "linear weight")
        if self.gemm_tc is not None and n <= self.tensor_core_gemm_max_tokens and k % 8 == 0:
            _dense(out, out.dtype, "linear output")
            splits, target = 1, out
            if allow_partials and out.dtype == torch.float32:
                splits = self.gemm_tc.shrike_gemm_tc_splits(n, o, k)
                if splits > 1:
                    target = self._partial_stack(out, splits)
            self.launches += 1
            _check(self.gemm_tc.shrike_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), _ptr(target), _DTYPE_CODE[out.dtype],
                                               n, o, k, splits, _ptr(self.status), self._stream()), "gemm_tcgen05")
            return target
        self.library_calls += 1
        if out.dtype == torch.float32:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, w.t(), out=out)
        if bias is not None:
            out.add_(bias)
        return out

    def _partial_stack(self, out, splits):
        """The float32 [splits, N, O] stack that belongs to the output buffer `out`."""
        n, o = out.shape
        key = out.data_ptr()
        held = self._partials.get(key)
        need = splits * n * o
        if held is None or held.numel() < need:
            capacity = max(need, 16 * self.tensor_core_gemm_max_tokens * o)
            held = torch.empty(capacity, dtype=torch.float32, device=self.device)
            self._partials[key] = held
            self.generation += 1
        return held[:need].view(splits, n, o)

    def adopt_status(self, word: torch.Tensor) -> None:
        """Makes `word` (int32 [4] on the device, zeroed) the status word the kernels write, so that
        the step function can bring it to the host in the same copy as a step's drawn tokens.  To be
        called before the first launch: launch sequences that were captured keep the old address."""
        if word.dtype != torch.int32 or word.numel() < 4 or word.device != self.status.device:
            raise KernelError("the status word must be four int32 on the kernels' device")
        word.zero_()
        self.status = word
        self.generation += 1

    @staticmethod
    def describe_status(code: int) -> str:
        """What a nonzero status word means: which kernel gave up, and where."""
        roles = {
            1: "gemm_tcgen05: the TMA producer's wait for a free stage ran out",
            2: "gemm_tcgen05: the MMA issuer's wait for a loaded stage ran out",
            3: "gemm_tcgen05: the epilogue's wait for the accumulator ran out",
            4: "gemm_tcgen05: copies still in flight after an aborted wait",
            11: "attention_tcgen05 (portions): the loader's wait for a free key/value stage ran out",
            12: "attention_tcgen05 (portions): the MMA issuer's wait ran out",
            13: "attention_tcgen05 (portions): a softmax thread's wait ran out",
            14: "attention_tcgen05 (portions): copies still in flight after an aborted wait",
            15: "attention_tcgen05 (portions): shared memory was not aligned as the tiles need",
            21: "attention_bf16 (single tokens, by pages): the wait for a page's tile ran out",
            22: "attention_bf16 (single tokens, by pages): shared memory was not aligned as the tiles need",
            31: "sampling: a row of logits had no finite element (NaN logits); token 0 was returned for it",
        }
        return roles.get(code, f"unknown status code {code}")

    def raise_status(self, code: int):
        """Clears the status word (and the counters an aborted kernel may have left half-way) and
        raises: the results of the step that set `code` are not valid."""
        self.status.zero_()
        if self._arrivals is not None:
            self._arrivals.zero_()
        raise KernelError(f"{self.describe_status(code)}; the results of that step are not valid")

    def check_status(self):
        """Raises when a kernel left a code in the status word (reads one word from the device)."""
        code = int(self.status[0].item())
        if code:
            self.raise_status(code)

    def rope_kv_write(self, qkv, bias, positions, inv_freq, q_out, keys, values, slots,
                      num_heads, num_kv_heads, head_dim, k_out=None, v_out=None):
        """Bias, rotation and cache store of a fused q/k/v projection ([N, W] or a K-split stack).
        `positions`, `slots`, `bias` and `inv_freq` are read while the kernels launched before may
        still run (the angles are formed meanwhile): they must be the step's metadata or
        parameters, not something a kernel of this step computes."""
        _dense(qkv, torch.float32, "qkv")
        _dense(q_out, self.dtype, "q")
        partials, stride = self._stack(qkv)
        n = qkv.shape[-2]
        num_slots = 0
        if keys is not None:
            _dense(keys, self.dtype, "key cache")
            _dense(values, self.dtype, "value cache")
            num_slots = keys.shape[0] * keys.shape[1]
        self.launches += 1
        _check(self.core.shrike_rope_kv_write(
            _ptr(qkv), _ptr(bias), _ptr(positions), _ptr(inv_freq), _ptr(q_out), _ptr(keys), _ptr(values),
            _ptr(slots), _ptr(k_out), _ptr(v_out), self.code, n, num_heads, num_kv_heads, head_dim,
            num_slots, partials, stride, self._stream()), "rope_kv_write")

    def kv_write(self, k_new, v_new, keys, values, slots):
        _dense(keys, self.dtype, "key cache")
        n, kv_width = k_new.shape
        self.launches += 1
        _check(self.core.shrike_kv_write(_ptr(k_new), _ptr(v_new), _ptr(keys), _ptr(values), _ptr(slots),
                                         self.code, n, kv_width, keys.shape[0] * keys.shape[1],
                                         self._stream()), "kv_write")

    def paged_attention(self, q, keys, values, block_table, q_start, ctx_len, seq_of_token,
                        num_heads, num_kv_heads, head_dim, scale, window, out,
                        max_q_len=0, max_ctx_len=0, min_q_len=0, q_lens=None):
        """Attention of the batch's new tokens over the paged cache.  `max_q_len` and
        `min_q_len` are the longest and shortest entry of the batch (0: not known); `q_lens`, every
        entry's length (host list), lets the portions kernel launch exactly the CTAs it needs."""
        _dense(q, self.dtype, "q")
        _dense(keys, self.dtype, "key cache")
        _dense(values, self.dtype, "value cache")
        _dense(block_table, torch.int32, "block table")
        if keys.shape[2] != num_kv_heads or keys.shape[3] != head_dim:
            raise KernelError(f"key cache {tuple(keys.shape)} does not fit {num_kv_heads} heads of {head_dim}")
        lib = self._attention_lib(head_dim)
        num_seqs, max_blocks = block_table.shape
        page_size, num_pages = keys.shape[1], keys.shape[0]
        if self.dtype == torch.float32:
            self.launches += 1
            _check(lib.shrike_paged_attention_generic(
                _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), max_blocks, _ptr(q_start),
                _ptr(ctx_len), _ptr(seq_of_token), self.code, q.shape[0], num_heads, num_kv_heads,
                page_size, num_pages, scale, window or 0, _ptr(out), self._stream()), "paged_attention")
            return
        plan = self.attention_plan(num_heads, num_kv_heads, head_dim, num_seqs, max_blocks, page_size, max_q_len, min_q_len,
                                   q.shape[0], q_lens)
        self.launches += plan.has_single + plan.has_portions + (1 if plan.portion_splits > 1 else 0)
        has_portions = plan.has_portions
        if plan.tc_portions:
            _check(lib.shrike_paged_attention_tc_portions(
                _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), max_blocks, _ptr(q_start), _ptr(ctx_len),
                q.shape[0], num_seqs, num_heads, num_kv_heads, page_size, num_pages, scale, window or 0, _ptr(out),
                plan.has_single, max_q_len, _ptr(self.status), plan.portion_splits, _ptr(plan.portion_scratch),
                self.portion_tiles(q_lens, plan.has_single, lib.shrike_attention_tc_portions_rows()), _ptr(seq_of_token),
                self._stream()), "paged_attention_tc_portions")
            has_portions = 0
            if not plan.has_single:
                return
        _check(lib.shrike_paged_attention_bf16(
            _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), max_blocks, _ptr(q_start), _ptr(ctx_len),
            num_seqs, num_heads, num_kv_heads, page_size, num_pages, scale, window or 0, _ptr(out),
            plan.has_single, has_portions, max_q_len, plan.splits, plan.cluster, _ptr(plan.scratch), _ptr(plan.arrivals),
            _ptr(self.status), self._stream()),
            "paged_attention_bf16")

    def portion_tiles(self, q_lens, skip_single, rows) -> int:
        """Query tiles of `rows` rows that the batch's portions make; 0 when the lengths are not known."""
        if q_lens is None:
            return 0
        held = self._portion_tiles
        if held is not None and held[0] is q_lens and held[1] == (skip_single, rows):
            return held[2]
        tiles = sum(-(-q // rows) for q in q_lens if q > 1 or not skip_single)
        self._portion_tiles = (q_lens, (skip_single, rows), tiles)
        return tiles

    def attention_plan(self, num_heads, num_kv_heads, head_dim, num_seqs, max_blocks, page_size, max_q_len, min_q_len,
                       num_tokens=0, q_lens=None):
        """How a bfloat16 batch's attention is cut: which kernels run (single tokens, portions, the
        tensor-core form of the latter), the key splits and clusters of the single-token kernel, the
        key splits of the portions kernel, and their scratch.  A function of the batch's shape alone."""
        if max_q_len < 1:
            raise KernelError("paged_attention in bfloat16 needs max_q_len, the longest entry of the batch")
        lib = self._attention_lib(head_dim)
        has_single = min_q_len <= 1
        has_portions = max_q_len > 1
        splits, cluster, scratch, arrivals = 1, 1, None, None
        if has_single:
            row_tiles = -(-(num_heads // num_kv_heads) // 16)
            tiles = max(1, -(-(max_blocks * page_size) // 64))
            resident = lib.shrike_attention_bf16_resident_ctas()
            splits, cluster = self.single_token_splits(tiles, num_seqs * num_kv_heads * row_tiles, resident)
            need = num_seqs * num_heads * (splits // cluster) * (head_dim + 2)
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=self.device)
                self.generation += 1
            groups = num_seqs * num_kv_heads * row_tiles
            if self._arrivals is None or self._arrivals.numel() < groups:
                self._arrivals = torch.zeros(max(groups, 4096), dtype=torch.int32, device=self.device)
                self.generation += 1
            scratch, arrivals = self._scratch, self._arrivals
        tc_portions = bool(has_portions and self.tensor_core_attention and lib.shrike_attention_tc_available()
                           and page_size in (8, 16, 32, 64))
        portion_splits, portion_scratch = 1, None
        if tc_portions and num_tokens > 0:
            tiles = self.portion_tiles(q_lens, has_single, lib.shrike_attention_tc_portions_rows())
            portion_splits = self.portion_splits or lib.shrike_attention_tc_portions_splits(
                num_tokens, num_heads, max_blocks, page_size, tiles)
            need = lib.shrike_attention_tc_portions_scratch_floats(num_tokens, num_heads, portion_splits)
            if need > self.PORTION_SCRATCH_FLOATS:   # bound the scratch: fewer splits, never a refusal
                portion_splits = max(1, portion_splits * self.PORTION_SCRATCH_FLOATS // need)
                need = lib.shrike_attention_tc_portions_scratch_floats(num_tokens, num_heads, portion_splits)
            if portion_splits > 1:
                if self._portion_scratch is None or self._portion_scratch.numel() < need:
                    self._portion_scratch = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=self.device)
                    self.generation += 1
                portion_scratch = self._portion_scratch
        return AttentionPlan(int(has_single), int(has_portions), int(tc_portions), splits, cluster, scratch, arrivals,
                             portion_splits, portion_scratch)

    @staticmethod
    def single_token_splits(tiles: int, groups: int, resident: int):
        """(splits, cluster) for single-token attention over `tiles` 64-key tiles of `groups`
        (sequence, kv head) pairs when `resident` CTAs fit the GPU at once.

        Up to eight splits may form a thread-block cluster and add up on chip.  That is the
        quickest way while the clusters fill no more than two thirds of the GPU; a fuller grid
        of clusters starts late (a cluster needs all its places free in one part of the chip
        at once, while the kernel before it is still leaving), and the splits then meet in
        global memory instead, eight partials to a round trip.  Long contexts take several
        clusters per pair, whose partials meet in global memory too."""
        want = max(1, min(tiles, resident // max(1, groups)))
        cluster = 1
        while cluster * 2 <= min(want, 8):
            cluster *= 2
        if cluster == 8 and groups * 8 * 3 > resident * 2:
            return min(want, 32) // 8 * 8, 1
        if tiles <= 4 * cluster or want < 2 * cluster:
            return cluster, cluster
        return min(want // cluster * cluster, 32 * cluster), cluster

    def silu_mul(self, gate_up, out, block=0):
        """out = silu(gate) * up.  `block` 0: a row of gate_up is all gate columns, then all up
        columns; b > 0: runs of b gate columns, each followed by the b up columns of the same features."""
        _dense(gate_up, self.dtype, "gate_up")
        _dense(out, self.dtype, "activation")
        n, inter = out.shape
        self.launches += 1
        _check(self.core.shrike_silu_mul(_ptr(gate_up), _ptr(out), self.code, n, inter, block, self._stream()), "silu_mul")

    @property
    def gated_rows(self) -> int:
        """How a gated feed-forward should interleave the rows of its fused gate/up matrix for
        `linear_gated`: runs of this many gate rows, each followed by the up rows of the same
        features.  0: keep gate rows, then up rows (no fused activation in this mode)."""
        return 16 if self.dtype == torch.bfloat16 and self.gemm_tc is not None else 0

    def linear_gated(self, x, w, out) -> bool:
        """silu(x Wg^T) * (x Wu^T) into `out` [N, I] in one kernel, for `w` [2 I, K] interleaved as
        `gated_rows` says.  Returns False when this shape is not served (many tokens: the caller
        then runs the product and the activation kernel, the latter with block=gated_rows)."""
        n, k = x.shape
        rows = w.shape[0]
        if (self.gated_rows == 0 or n > self.tensor_core_gemm_max_tokens or k % 8 or rows % 32
                or tuple(out.shape) != (n, rows // 2) or w.shape[1] != k):
            return False
        _dense(x, torch.bfloat16, "linear input")
        _dense(w, torch.bfloat16, "linear weight")
        _dense(out, torch.bfloat16, "activation")
        self.launches += 1
        _check(self.gemm_tc.shrike_gemm_tc_gated(_ptr(x), _ptr(w), _ptr(out), n, rows, k, _ptr(self.status),
                                                 self._stream()), "gemm_tcgen05")
        return True

    def sample(self, logits, temperature, top_p, seeds, out):
        _dense(logits, torch.float32, "logits")
        _dense(temperature, torch.float32, "temperature")
        _dense(top_p, torch.float32, "top_p")
        _dense(seeds, torch.int64, "seeds")
        _dense(out, torch.int32, "sampled tokens")
        rows, vocab = logits.shape
        need = max(rows, 64) * self.core.shrike_sample_slices(vocab)
        if self._sample_scratch is None or self._sample_scratch[0].numel() < need:
            self._sample_scratch = (torch.empty(2 * need, dtype=torch.float32, device=self.device),
                                    torch.empty(2 * need, dtype=torch.int32, device=self.device))
            self.generation += 1
        values, indices = self._sample_scratch
        self.launches += 2
        _check(self.core.shrike_sample(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(seeds), _ptr(out),
                                       _ptr(values), _ptr(indices), rows, vocab, _ptr(self.status), self._stream()),
               "sample")
