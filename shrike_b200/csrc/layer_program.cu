// One decoder layer issued by one call: norm, q/k/v projection, rotation and cache store,
// attention, output projection, norm, gated feed-forward.  The kernels are the package's own
// launchers, reached through the addresses the caller hands in (they live in the other
// libraries of the package: nothing is compiled twice), and cuBLAS for products of more
// tokens than the tensor-core kernel of the package takes, as everywhere in the engine
// (Azimml/shrike's own products are cuBLAS calls through nn.Linear, shrike/models/qwen.py:111-136).
//
// Why it exists: a step that is not replayed from a CUDA graph (a batch shape seen for the first
// time) is issued launch by launch, and from Python every launch costs about ten microseconds
// of interpreter time, three milliseconds for a 28-layer model, more than the GPU needs to run
// the step.  Issued from here a launch costs what the driver takes.  Every decision (which
// product path, how K is split, how attention is cut) is made by the caller once per step and
// arrives as plain numbers: this file decides nothing.
//
// The sequence is that of a pre-norm block over this package's attention and gated feed-forward
// parts in bfloat16 (shrike/models/qwen.py:147-150 for the arrangement); other arrangements keep
// the part-by-part path.
#include <cublas_v2.h>

#include <mutex>

#include "common.cuh"

extern "C" {
typedef int (*AddRmsnormFn)(float*, const void*, int, const int*, const float*, float, void*, int, int, int, int, long long,
                            cudaStream_t);
typedef int (*GemmTcFn)(const void*, const void*, const float*, void*, int, int, int, int, int, int*, cudaStream_t);
typedef int (*GemmTcGatedFn)(const void*, const void*, void*, int, int, int, int*, cudaStream_t);
typedef int (*RopeKvWriteFn)(const float*, const float*, const int*, const float*, void*, void*, void*, const int*, void*, void*,
                             int, int, int, int, int, long long, int, long long, cudaStream_t);
typedef int (*AttentionTcFn)(const void*, const void*, const void*, const int*, int, const int*, const int*, int, int, int, int,
                             int, int, float, int, void*, int, int, int*, int, float*, int, const int*, cudaStream_t);
typedef int (*AttentionBf16Fn)(const void*, const void*, const void*, const int*, int, const int*, const int*, int, int, int,
                               int, int, float, int, void*, int, int, int, int, int, float*, int*, int*, cudaStream_t);
typedef int (*SiluMulFn)(const void*, void*, int, int, int, int, cudaStream_t);
typedef cublasStatus_t (*CublasCreateFn)(cublasHandle_t*);
typedef cublasStatus_t (*CublasSetStreamFn)(cublasHandle_t, cudaStream_t);
typedef cublasStatus_t (*CublasSetWorkspaceFn)(cublasHandle_t, void*, size_t);
typedef cublasStatus_t (*CublasSetMathModeFn)(cublasHandle_t, cublasMath_t);
typedef cublasStatus_t (*CublasGemmExFn)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                         const void*, cudaDataType, int, const void*, cudaDataType, int, const void*, void*,
                                         cudaDataType, int, cublasComputeType_t, cublasGemmAlgo_t);

// Where the launchers live.  The attention entries belong to the library built for the layer's
// head size; the cuBLAS entries to the copy of cuBLAS the process has already loaded.
struct ShrikeLayerFns {
  AddRmsnormFn add_rmsnorm;
  GemmTcFn gemm_tc;
  GemmTcGatedFn gemm_tc_gated;
  RopeKvWriteFn rope_kv_write;
  AttentionTcFn attention_tc_portions;
  AttentionBf16Fn attention_bf16;
  SiluMulFn silu_mul;
  CublasCreateFn cublas_create;
  CublasSetStreamFn cublas_set_stream;
  CublasSetWorkspaceFn cublas_set_workspace;
  CublasSetMathModeFn cublas_set_math_mode;
  CublasGemmExFn cublas_gemm_ex;
};

// What a layer is, for as long as the model and its cache pool live: sizes, weights, its pages.
struct ShrikeLayerConst {
  int width, heads, kv_heads, head_dim, inter, window;
  float eps_mixer, eps_ffn, scale;
  int silu_block;                            // > 0: gate/up rows interleaved in runs of this many
  int page_size, num_pages;
  long long num_slots;
  const float* norm_mixer_w;
  const float* norm_ffn_w;
  const void* w_qkv;                         // [(heads + 2 kv_heads) head_dim][width]
  const float* b_qkv;
  const void* w_o;                           // [width][heads head_dim]
  const float* b_o;
  const void* w_gate_up;                     // [2 inter][width]
  const void* w_down;                        // [width][inter]
  const float* inv_freq;                     // null: no rotation
  void* keys;                                // this layer's pages; null: store nothing (the layer reads another's cache)
  void* values;
  void* read_keys;                           // the pages attention reads (the same unless the layer reads another's cache)
  void* read_values;
};

// What a step brings, the same for every layer of equal sizes: the batch's shape and metadata, the
// buffers, and how the products and attention are cut.  Buffers are row-major; a product that is
// split along K writes a stack [splits][tokens][columns] of float32 at its output pointer, which
// the next kernel adds up.
struct ShrikeLayerStep {
  int tokens, seqs, max_blocks, max_q_len;
  int qkv_splits, o_splits, down_splits;
  int use_library;                           // 1: the four products go to cuBLAS
  int gated_fused;                           // 1: gate_up and its activation are one tensor-core kernel
  int has_single, has_portions, tc_portions, attn_splits, attn_cluster;
  int portion_splits;                        // key splits of the tensor-core portions kernel
  int portion_tiles;                         // query tiles the batch's portions make (0: not known)
  const int* positions;
  const int* slots;
  const int* block_table;
  const int* q_start;
  const int* ctx_len;
  const int* seq_of_token;
  float* resid;                              // [tokens][width] float32
  void* normed;                              // [tokens][width] bfloat16
  float* qkv;                                // [qkv_splits][tokens][(heads + 2 kv_heads) head_dim]
  void* q;                                   // [tokens][heads head_dim] bfloat16
  void* attn_out;                            // [tokens][heads head_dim] bfloat16
  float* o_out;                              // [o_splits][tokens][width]
  void* gate_up;                             // [tokens][2 inter] bfloat16 (unused when the activation is fused)
  void* act;                                 // [tokens][inter] bfloat16
  float* down_out;                           // [down_splits][tokens][width]
  float* attn_scratch;
  int* attn_arrivals;
  float* portion_scratch;
  int* status;
  void* workspace;                           // for cuBLAS
  long long workspace_bytes;
};
}

namespace {

struct Blas {
  cublasHandle_t handle = nullptr;
  void* workspace = nullptr;
  cudaStream_t stream = nullptr;
  bool stream_set = false;
};
std::mutex blas_mutex;
Blas blas_of_device[64];

// The library's handle of the current device, made on first use (that takes a tenth of a second:
// shrike_layer_program_warm does it when the engine is built, not in a request's first step).
int blas_of_current_device(const ShrikeLayerFns& fn, Blas** out) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return SHRIKE_BAD_ARGUMENT;
  Blas& blas = blas_of_device[device];
  if (blas.handle == nullptr) {
    if (fn.cublas_create(&blas.handle) != CUBLAS_STATUS_SUCCESS) return 2000;
    fn.cublas_set_math_mode(blas.handle, static_cast<cublasMath_t>(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
  }
  *out = &blas;
  return SHRIKE_OK;
}

// out[tokens][columns] = x[tokens][k] * w[columns][k]^T in bfloat16 with float32 accumulation, no
// reduced-precision partial sums.  Row-major operands are column-major ones transposed: C^T = W X^T.
int library_product(const ShrikeLayerFns& fn, const ShrikeLayerStep& c, const void* x, const void* w, void* out, bool out_f32,
                    int columns, int k, cudaStream_t stream) {
  Blas* found = nullptr;
  {
    std::lock_guard<std::mutex> guard(blas_mutex);
    const int rc = blas_of_current_device(fn, &found);
    if (rc != SHRIKE_OK) return rc;
    Blas& blas = *found;
    if (blas.workspace != c.workspace && c.workspace != nullptr) {
      if (fn.cublas_set_workspace(blas.handle, c.workspace, static_cast<size_t>(c.workspace_bytes)) != CUBLAS_STATUS_SUCCESS) return 2001;
      blas.workspace = c.workspace;
    }
    if (!blas.stream_set || blas.stream != stream) {
      if (fn.cublas_set_stream(blas.handle, stream) != CUBLAS_STATUS_SUCCESS) return 2002;
      // setting the stream resets the workspace to the library's own: give ours again
      if (c.workspace != nullptr) fn.cublas_set_workspace(blas.handle, c.workspace, static_cast<size_t>(c.workspace_bytes));
      blas.stream = stream;
      blas.stream_set = true;
    }
  }
  Blas& blas = *found;
  const float one = 1.0f, zero = 0.0f;
  const cublasStatus_t rc = fn.cublas_gemm_ex(blas.handle, CUBLAS_OP_T, CUBLAS_OP_N, columns, c.tokens, k, &one, w, CUDA_R_16BF, k, x,
                                              CUDA_R_16BF, k, &zero, out, out_f32 ? CUDA_R_32F : CUDA_R_16BF, columns,
                                              CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  return rc == CUBLAS_STATUS_SUCCESS ? SHRIKE_OK : 2100 + static_cast<int>(rc);
}

}  // namespace

// Makes the library's handle for the current device now rather than in the first step that needs it.
SHRIKE_API int shrike_layer_program_warm(const ShrikeLayerFns* fns) {
  std::lock_guard<std::mutex> guard(blas_mutex);
  Blas* found = nullptr;
  return blas_of_current_device(*fns, &found);
}

#define SHRIKE_TRY(call)          \
  do {                            \
    const int rc_ = (call);       \
    if (rc_ != SHRIKE_OK) return rc_; \
  } while (0)

// Returns 0, or the first launcher's error code.  `delta` is the branch output still to be added to
// the residual (null: none; else [delta_partials] slices `delta_stride` elements apart).  On return
// the layer's feed-forward output waits at step->down_out (a stack of down_splits slices) to be
// added to the residual by the next norm.
SHRIKE_API int shrike_decoder_layer(const ShrikeLayerFns* fns, const ShrikeLayerConst* layer, const ShrikeLayerStep* step,
                                    const void* delta, int delta_dtype, int delta_partials, long long delta_stride,
                                    cudaStream_t stream) {
  const ShrikeLayerFns& fn = *fns;
  const ShrikeLayerConst& l = *layer;
  const ShrikeLayerStep& c = *step;
  if (c.tokens <= 0) return SHRIKE_OK;
  if (l.b_o != nullptr && c.use_library) return SHRIKE_BAD_ARGUMENT;   // the part-by-part path serves that
  const int q_width = l.heads * l.head_dim;
  const int qkv_width = (l.heads + 2 * l.kv_heads) * l.head_dim;
  const long long slice_qkv = static_cast<long long>(c.tokens) * qkv_width;
  const long long slice_w = static_cast<long long>(c.tokens) * l.width;

  SHRIKE_TRY(fn.add_rmsnorm(c.resid, delta, delta == nullptr ? SHRIKE_NONE : delta_dtype, nullptr, l.norm_mixer_w, l.eps_mixer,
                            c.normed, SHRIKE_BF16, c.tokens, l.width, delta == nullptr ? 1 : delta_partials, delta_stride, stream));
  if (c.use_library) SHRIKE_TRY(library_product(fn, c, c.normed, l.w_qkv, c.qkv, true, qkv_width, l.width, stream));
  else SHRIKE_TRY(fn.gemm_tc(c.normed, l.w_qkv, nullptr, c.qkv, SHRIKE_F32, c.tokens, qkv_width, l.width, c.qkv_splits, c.status, stream));
  SHRIKE_TRY(fn.rope_kv_write(c.qkv, l.b_qkv, c.positions, l.inv_freq, c.q, l.keys, l.values, c.slots, nullptr, nullptr, SHRIKE_BF16,
                              c.tokens, l.heads, l.kv_heads, l.head_dim, l.num_slots, c.use_library ? 1 : c.qkv_splits, slice_qkv, stream));
  bool portions_left = c.has_portions != 0;
  if (portions_left && c.tc_portions) {
    SHRIKE_TRY(fn.attention_tc_portions(c.q, l.read_keys, l.read_values, c.block_table, c.max_blocks, c.q_start, c.ctx_len, c.tokens, c.seqs,
                                        l.heads, l.kv_heads, l.page_size, l.num_pages, l.scale, l.window, c.attn_out, c.has_single,
                                        c.max_q_len, c.status, c.portion_splits, c.portion_scratch, c.portion_tiles, c.seq_of_token, stream));
    portions_left = false;
  }
  if (c.has_single || portions_left)
    SHRIKE_TRY(fn.attention_bf16(c.q, l.read_keys, l.read_values, c.block_table, c.max_blocks, c.q_start, c.ctx_len, c.seqs, l.heads,
                                 l.kv_heads, l.page_size, l.num_pages, l.scale, l.window, c.attn_out, c.has_single, portions_left ? 1 : 0,
                                 c.max_q_len, c.attn_splits, c.attn_cluster, c.attn_scratch, c.attn_arrivals, c.status, stream));
  if (c.use_library) SHRIKE_TRY(library_product(fn, c, c.attn_out, l.w_o, c.o_out, true, l.width, q_width, stream));
  else SHRIKE_TRY(fn.gemm_tc(c.attn_out, l.w_o, l.b_o, c.o_out, SHRIKE_F32, c.tokens, l.width, q_width, c.o_splits, c.status, stream));
  SHRIKE_TRY(fn.add_rmsnorm(c.resid, c.o_out, SHRIKE_F32, nullptr, l.norm_ffn_w, l.eps_ffn, c.normed, SHRIKE_BF16, c.tokens, l.width,
                            c.use_library ? 1 : c.o_splits, slice_w, stream));
  if (c.gated_fused) {
    SHRIKE_TRY(fn.gemm_tc_gated(c.normed, l.w_gate_up, c.act, c.tokens, 2 * l.inter, l.width, c.status, stream));
  } else {
    if (c.use_library) SHRIKE_TRY(library_product(fn, c, c.normed, l.w_gate_up, c.gate_up, false, 2 * l.inter, l.width, stream));
    else SHRIKE_TRY(fn.gemm_tc(c.normed, l.w_gate_up, nullptr, c.gate_up, SHRIKE_BF16, c.tokens, 2 * l.inter, l.width, 1, c.status, stream));
    SHRIKE_TRY(fn.silu_mul(c.gate_up, c.act, SHRIKE_BF16, c.tokens, l.inter, l.silu_block, stream));
  }
  if (c.use_library) SHRIKE_TRY(library_product(fn, c, c.act, l.w_down, c.down_out, true, l.width, l.inter, stream));
  else SHRIKE_TRY(fn.gemm_tc(c.act, l.w_down, nullptr, c.down_out, SHRIKE_F32, c.tokens, l.width, l.inter, c.down_splits, c.status, stream));
  return SHRIKE_OK;
}

// How many kernels of the package and how many library products a layer of this step launches, for
// the caller's counters: launches in the low 16 bits, library products above.
SHRIKE_API int shrike_decoder_layer_launches(const ShrikeLayerStep* step) {
  const ShrikeLayerStep& c = *step;
  const int own = 3 /* two norms, rotary */ + (c.has_portions ? 1 : 0) + (c.has_single ? 1 : 0) + (c.gated_fused ? 0 : 1) +
                  (c.use_library ? 0 : 4) + (c.has_portions && c.tc_portions && c.portion_splits > 1 ? 1 : 0);
  const int library = c.use_library ? 4 : 0;
  return own | (library << 16);
}
