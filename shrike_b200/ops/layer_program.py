"""One decoder layer issued by one native call (`csrc/layer_program.cu`).

A step that is not replayed from a CUDA graph is issued launch by launch; from Python every
launch costs about ten microseconds of interpreter time, which for a 28-layer model is more
than the GPU needs to run the step.  `LayerProgram` hands a whole pre-norm layer (norm,
q/k/v projection, rotation and cache store, attention, output projection, norm, gated
feed-forward) to one C function that issues the same launchers in the same order with the
same arguments as the part-by-part path, so both paths give the same bits.  What is decided
per step (which product path, how K is split, how attention is cut) is decided here, once per
step, by the same functions the part-by-part path uses; the C side decides nothing.

It serves the package's own attention, gated feed-forward and RMS norm parts in bfloat16.  Any
other part (a toy mixer, a routed feed-forward, a position encoding without a table) keeps the
part-by-part path: `LayerProgram.serves` says which.
"""

from __future__ import annotations

import ctypes
import weakref

import torch

from . import build

_c = ctypes
_P, _I, _F, _LL = _c.c_void_p, _c.c_int, _c.c_float, _c.c_longlong


class LayerFns(_c.Structure):
    _fields_ = [(name, _P) for name in (
        "add_rmsnorm", "gemm_tc", "gemm_tc_gated", "rope_kv_write", "attention_tc_portions", "attention_bf16", "silu_mul",
        "cublas_create", "cublas_set_stream", "cublas_set_workspace", "cublas_set_math_mode", "cublas_gemm_ex")]


class LayerConst(_c.Structure):
    """ShrikeLayerConst: what a layer is for as long as the model and its cache pool live."""

    _fields_ = (
        [(n, _I) for n in ("width", "heads", "kv_heads", "head_dim", "inter", "window")]
        + [(n, _F) for n in ("eps_mixer", "eps_ffn", "scale")]
        + [(n, _I) for n in ("silu_block", "page_size", "num_pages")]
        + [("num_slots", _LL)]
        + [(n, _P) for n in ("norm_mixer_w", "norm_ffn_w", "w_qkv", "b_qkv", "w_o", "b_o", "w_gate_up", "w_down", "inv_freq",
                             "keys", "values", "read_keys", "read_values")]
    )


class LayerStep(_c.Structure):
    """ShrikeLayerStep: what a step brings, the same for every layer of equal sizes."""

    _fields_ = (
        [(n, _I) for n in ("tokens", "seqs", "max_blocks", "max_q_len", "qkv_splits", "o_splits", "down_splits", "use_library",
                           "gated_fused", "has_single", "has_portions", "tc_portions", "attn_splits", "attn_cluster",
                           "portion_splits", "portion_tiles")]
        + [(n, _P) for n in ("positions", "slots", "block_table", "q_start", "ctx_len", "seq_of_token", "resid", "normed", "qkv", "q", "attn_out",
                             "o_out", "gate_up", "act", "down_out", "attn_scratch", "attn_arrivals", "portion_scratch", "status",
                             "workspace")]
        + [("workspace_bytes", _LL)]
    )


def _address(function) -> int:
    return _c.cast(function, _P).value


def _cublas():
    """The copy of cuBLAS the process already holds (torch loads it); opening it by its soname
    returns that copy instead of a second one."""
    for name in ("libcublas.so.12", "libcublas.so.13", "libcublas.so"):
        try:
            return _c.CDLL(name)
        except OSError:
            continue
    return None


class LayerProgram:
    WORKSPACE_BYTES = 32 << 20

    def __init__(self, ops):
        self.ops = weakref.proxy(ops)   # the kernels own this object, not the other way round: no cycle to collect
        self.lib = build.layer_program_library()
        self.lib.shrike_decoder_layer.argtypes = [_P, _P, _P, _P, _I, _I, _LL, _P]
        self.lib.shrike_decoder_layer.restype = _I
        self.lib.shrike_decoder_layer_launches.argtypes = [_P]
        self.lib.shrike_decoder_layer_launches.restype = _I
        self.blas = _cublas()
        self._fns: dict[int, LayerFns] = {}   # head size -> launcher table
        self._fn_refs: dict = {}
        self._workspace = None
        self._warm = False

    # ---- which layers -------------------------------------------------------------
    def serves(self, mixer, mixer_norm, feed_forward, feed_forward_norm) -> bool:
        from ..parts.attention import PagedAttention
        from ..parts.mlp import GatedMLP
        from ..parts.norm import RMSNorm

        if self.blas is None or self.ops.dtype != torch.bfloat16 or self.ops.gemm_tc is None:
            return False
        if type(mixer) is not PagedAttention or type(feed_forward) is not GatedMLP:
            return False
        if type(mixer_norm) is not RMSNorm or type(feed_forward_norm) is not RMSNorm:
            return False
        if mixer.position is not None and mixer.position.rotary_table() is None:
            return False
        if mixer.b_o is not None:
            return False
        if not (mixer.spec.width % 8 == 0 and mixer.q_width % 8 == 0 and feed_forward.spec.intermediate % 8 == 0):
            return False
        self.warm(mixer.spec.head_dim)
        return True

    def warm(self, head_dim: int) -> None:
        """What would otherwise fall into a request's first long step: the library's handle (a tenth
        of a second to make) and its workspace."""
        if self._warm:
            return
        self._warm = True
        self.lib.shrike_layer_program_warm.argtypes = [_P]
        self.lib.shrike_layer_program_warm.restype = _I
        with torch.cuda.device(self.ops.device):
            self.lib.shrike_layer_program_warm(self._fn_ref(head_dim))
        if self._workspace is None:
            self._workspace = torch.empty(self.WORKSPACE_BYTES, dtype=torch.uint8, device=self.ops.device)

    def _launchers(self, head_dim: int) -> LayerFns:
        fns = self._fns.get(head_dim)
        if fns is None:
            ops = self.ops
            attention = ops._attention_lib(head_dim)
            fns = LayerFns(
                add_rmsnorm=_address(ops.core.shrike_add_rmsnorm), gemm_tc=_address(ops.gemm_tc.shrike_gemm_tc),
                gemm_tc_gated=_address(ops.gemm_tc.shrike_gemm_tc_gated), rope_kv_write=_address(ops.core.shrike_rope_kv_write),
                attention_tc_portions=_address(attention.shrike_paged_attention_tc_portions),
                attention_bf16=_address(attention.shrike_paged_attention_bf16), silu_mul=_address(ops.core.shrike_silu_mul),
                cublas_create=_address(self.blas.cublasCreate_v2), cublas_set_stream=_address(self.blas.cublasSetStream_v2),
                cublas_set_workspace=_address(self.blas.cublasSetWorkspace_v2),
                cublas_set_math_mode=_address(self.blas.cublasSetMathMode), cublas_gemm_ex=_address(self.blas.cublasGemmEx))
            self._fns[head_dim] = fns
        return fns

    def _fn_ref(self, head_dim: int):
        ref = self._fn_refs.get(head_dim)
        if ref is None:
            ref = self._fn_refs[head_dim] = _c.byref(self._launchers(head_dim))
        return ref

    # ---- one layer ----------------------------------------------------------------
    def _constants(self, held_by_block: dict, mixer, mixer_norm, feed_forward, feed_forward_norm, ctx, run):
        """The layer's ShrikeLayerConst, built once per (run of the order, cache pool) and kept by the
        block (`held_by_block`): addresses only, valid as long as the block's parts and the pool are."""
        key = (run.cache, run.writes_cache, id(ctx.storage))
        held = held_by_block.get(key)
        if held is None:
            spec, ffn = mixer.spec, feed_forward.spec
            group, keys, values = ctx.storage.keys_values(run.cache)
            table = mixer.position.rotary_table() if mixer.position is not None else None
            const = LayerConst(
                width=spec.width, heads=spec.num_heads, kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                inter=ffn.intermediate, window=spec.window or 0, eps_mixer=mixer_norm.spec.eps,
                eps_ffn=feed_forward_norm.spec.eps, scale=spec.scale, silu_block=feed_forward.run,
                page_size=keys.shape[1], num_pages=keys.shape[0], num_slots=keys.shape[0] * keys.shape[1],
                norm_mixer_w=mixer_norm.weight.data_ptr(), norm_ffn_w=feed_forward_norm.weight.data_ptr(),
                w_qkv=mixer.w_qkv.data_ptr(), b_qkv=None if mixer.b_qkv is None else mixer.b_qkv.data_ptr(),
                w_o=mixer.w_o.data_ptr(), b_o=None, w_gate_up=feed_forward.w_gate_up.data_ptr(),
                w_down=feed_forward.w_down.data_ptr(), inv_freq=None if table is None else table.data_ptr(),
                keys=keys.data_ptr() if run.writes_cache else None, values=values.data_ptr() if run.writes_cache else None,
                read_keys=keys.data_ptr(), read_values=values.data_ptr())
            held = held_by_block[key] = (const, group, keys.shape[1])
        return held

    def _step(self, mixer, feed_forward, ctx, group, page_size):
        """The step's ShrikeLayerStep for layers of these sizes, built once per step and group."""
        spec, inter = mixer.spec, feed_forward.spec.intermediate
        key = (group, spec.width, mixer.qkv_width, mixer.q_width, inter, bool(feed_forward.run))
        cache = getattr(ctx, "_layer_steps", None)
        if cache is None:
            cache = ctx._layer_steps = {}
        held = cache.get(key)
        if held is not None:
            return held
        ops, rt = self.ops, mixer.runtime
        n, width, qkv_width, q_width = ctx.num_tokens, spec.width, mixer.qkv_width, mixer.q_width
        view = ctx.groups[group]
        library = n > ops.tensor_core_gemm_max_tokens
        bf16 = torch.bfloat16
        step = LayerStep(tokens=n, seqs=ctx.num_seqs, max_blocks=view.max_blocks, max_q_len=ctx.max_q_len, use_library=int(library))
        splits_of = ops.gemm_tc.shrike_gemm_tc_splits
        step.qkv_splits = 1 if library else splits_of(n, qkv_width, width)
        step.o_splits = 1 if library else splits_of(n, width, q_width)
        step.down_splits = 1 if library else splits_of(n, width, inter)
        step.gated_fused = int(bool(feed_forward.run) and not library and (2 * inter) % 32 == 0)
        plan = ops.attention_plan(spec.num_heads, spec.num_kv_heads, spec.head_dim, ctx.num_seqs, view.max_blocks, page_size,
                                  ctx.max_q_len, ctx.min_q_len, n, ctx.q_lens)
        step.portion_splits = plan.portion_splits
        step.portion_tiles = ops.portion_tiles(ctx.q_lens, plan.has_single,
                                               ops._attention_lib(spec.head_dim).shrike_attention_tc_portions_rows())
        step.seq_of_token = ctx.seq_of_token.data_ptr()
        step.portion_scratch = None if plan.portion_scratch is None else plan.portion_scratch.data_ptr()
        step.has_single, step.has_portions, step.tc_portions = plan.has_single, plan.has_portions, plan.tc_portions
        step.attn_splits, step.attn_cluster = plan.splits, plan.cluster
        step.attn_scratch = None if plan.scratch is None else plan.scratch.data_ptr()
        step.attn_arrivals = None if plan.arrivals is None else plan.arrivals.data_ptr()
        step.positions, step.slots = ctx.positions.data_ptr(), view.slot_mapping.data_ptr()
        step.block_table, step.q_start, step.ctx_len = view.block_table.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr()
        step.normed = rt.buffer("normed", (n, width), bf16).data_ptr()
        qkv = rt.buffer("qkv", (n, qkv_width), torch.float32)
        step.qkv = (ops._partial_stack(qkv, step.qkv_splits) if step.qkv_splits > 1 else qkv).data_ptr()
        step.q = rt.buffer("q", (n, q_width), bf16).data_ptr()
        step.attn_out = rt.buffer("attn_out", (n, q_width), bf16).data_ptr()
        o_out = rt.buffer("mixer_delta", (n, width), torch.float32)
        step.o_out = (ops._partial_stack(o_out, step.o_splits) if step.o_splits > 1 else o_out).data_ptr()
        if not step.gated_fused:
            step.gate_up = rt.buffer("gate_up", (n, 2 * inter), bf16).data_ptr()
        step.act = rt.buffer("ffn_act", (n, inter), bf16).data_ptr()
        down_out = rt.buffer("ffn_delta", (n, width), torch.float32)
        down_target = ops._partial_stack(down_out, step.down_splits) if step.down_splits > 1 else down_out
        step.down_out = down_target.data_ptr()
        step.status = ops.status.data_ptr()
        if library:
            if self._workspace is None:
                self._workspace = torch.empty(self.WORKSPACE_BYTES, dtype=torch.uint8, device=ops.device)
                ops.generation += 1
            step.workspace, step.workspace_bytes = self._workspace.data_ptr(), self.WORKSPACE_BYTES
        counts = self.lib.shrike_decoder_layer_launches(_c.byref(step))
        held = (step, down_target, counts & 0xFFFF, counts >> 16)
        cache[key] = held
        return held

    def run(self, held_by_block, mixer, mixer_norm, feed_forward, feed_forward_norm, resid, delta, ctx, run):
        """Issues the layer; returns what the next norm has to add to the residual (the
        feed-forward's output: an array [N, W] or a stack of K-split slices).  `held_by_block` is a
        dictionary the calling block keeps for this program's per-layer constants."""
        ops = self.ops
        const, group, page_size = self._constants(held_by_block, mixer, mixer_norm, feed_forward, feed_forward_norm, ctx, run)
        step, down_target, own, library = self._step(mixer, feed_forward, ctx, group, page_size)
        step.resid = resid.data_ptr()
        if delta is None:
            pointer, code, partials, stride = None, -1, 1, 0
        else:
            partials, stride = ops._stack(delta)
            pointer, code = delta.data_ptr(), 0 if delta.dtype == torch.float32 else 1
        rc = self.lib.shrike_decoder_layer(self._fn_ref(const.head_dim), _c.byref(const), _c.byref(step), pointer, code, partials, stride,
                                           ops._stream())
        if rc != 0:
            from .cuda_ops import KernelError

            raise KernelError(f"decoder layer: launcher returned {rc}")
        ops.launches += own
        ops.library_calls += library
        return down_target
