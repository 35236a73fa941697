// Embedding, residual-add + RMSNorm, SiLU-mul, bias + rotary + key/value store.
//
// All statistics, angles and sums are float32; a result is rounded once, when it
// is stored in the activation type.  Formulas: shrike/models/qwen.py:64-74 (norm),
// :77-101 (rotary), :136 (SiLU product), shrike/engine/model_runner.py:69-70 (store).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// A negative id -1 - r stands for "the token the step before drew in its row r": it is read
// from `previous` on the device, so that a step can be launched before the host has seen the
// tokens of the step before it.  Ids outside the vocabulary give a row of zeros.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int width, int vocab,
                             const int* __restrict__ previous, int previous_rows) {
  let_dependents_start();
  wait_for_previous();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 && previous != nullptr && -1 - id < previous_rows) id = previous[-1 - id];
  const bool valid = id >= 0 && id < vocab;
  if (!valid) id = 0;
  const T* src = table + static_cast<size_t>(id) * width;
  float* dst = out + static_cast<size_t>(row) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = valid ? to_float(src[i]) : 0.f;
}

SHRIKE_API int shrike_embed(const int* ids, const void* table, int table_dtype, float* out, int n,
                            int width, int vocab, const int* previous, int previous_rows, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (width <= 0 || vocab <= 0) return SHRIKE_BAD_ARGUMENT;
  const int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == SHRIKE_F32)
    launch_dependent(embed_kernel<float>, n, threads, 0, stream, ids, static_cast<const float*>(table), out, width, vocab,
                     previous, previous_rows);
  else if (table_dtype == SHRIKE_BF16)
    launch_dependent(embed_kernel<__nv_bfloat16>, n, threads, 0, stream, ids, static_cast<const __nv_bfloat16*>(table), out, width,
                     vocab, previous, previous_rows);
  else
    return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

// ------------------------------------------------- residual add + RMSNorm
// One block per output row.  GATHER: the row comes from `rows`, the residual is
// not written back (used for the final norm on the wanted rows only).  Each thread
// keeps its elements in registers between the sum of squares and the scaling, so a
// row is read once; VEC = 4 uses 16-byte accesses (width a multiple of 4).
constexpr int NORM_MAX_PER_THREAD = 8;  // elements (VEC = 1) or float4 groups (VEC = 4) a thread may hold

template <typename TD> __device__ __forceinline__ void load4(const TD* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
template <typename TO> __device__ __forceinline__ void store4(TO* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const unsigned*>(&lo);
  t.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}

// `delta` may be a stack of `partials` arrays (the slices of a K-split matrix product),
// `partial_stride` elements apart; they are added in ascending order.
// PER_THREAD 1 (few rows of up to 1024 groups): a thread holds one group, reads the norm weight
// before the wait and has the residual and up to eight slices in flight together, so the
// row costs one memory round trip.  PER_THREAD 2 (few rows of up to 2048 groups): the same,
// one group after the other.  PER_THREAD 8 (many rows, or wider ones) adds slice by slice.
template <typename TD, typename TO, bool HAS_DELTA, bool GATHER, int VEC, int PER_THREAD>
__global__ void __launch_bounds__(1024, 1) add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ weight,
                                   float eps, TO* __restrict__ out, int width, int partials,
                                   long long partial_stride) {
  __shared__ float scratch[33];
  constexpr int AHEAD = PER_THREAD <= 2 ? 7 : 1;   // the first slice and seven more: a stack of eight in one go
  let_dependents_start();
  const int groups = width / VEC;
  constexpr bool GAIN_AHEAD = PER_THREAD <= 2;   // registers allow it only for the narrow forms
  float gain[GAIN_AHEAD ? PER_THREAD : 1][VEC];   // the norm weight: no kernel writes it, so it is read ahead of the wait
#pragma unroll
  for (int it = 0; it < (GAIN_AHEAD ? PER_THREAD : 0); ++it) {
    const int g = threadIdx.x + it * blockDim.x;
    if (g < groups) {
      if (VEC == 4) {
        float w[4];
        load4<float>(weight + g * 4, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) gain[it][i % VEC] = w[i];
      } else {
        gain[it][0] = weight[g];
      }
    }
  }
  wait_for_previous();
  const int out_row = blockIdx.x;
  const int row = GATHER ? rows[out_row] : out_row;
  float* x = resid + static_cast<size_t>(row) * width;
  const TD* d = HAS_DELTA ? delta + static_cast<size_t>(row) * width : nullptr;
  TO* y = out + static_cast<size_t>(out_row) * width;

  float held[PER_THREAD][VEC];
  float sum_sq = 0.f;
#pragma unroll
  for (int it = 0; it < PER_THREAD; ++it) {
    const int g = threadIdx.x + it * blockDim.x;
    if (g < groups) {
      if (VEC == 4) {
        float v[4], dv[4];
        load4<float>(x + g * 4, v);
        if (HAS_DELTA) {
          load4<TD>(d + g * 4, dv);
          if (partials > 1) {   // AHEAD slices at a time: their loads are issued before the first addition
            for (int first = 1; first < partials; first += AHEAD) {
              float more[AHEAD][4];
#pragma unroll
              for (int q = 0; q < AHEAD; ++q)
                if (first + q < partials) load4<TD>(d + (first + q) * partial_stride + g * 4, more[q]);
#pragma unroll
              for (int q = 0; q < AHEAD; ++q)
                if (first + q < partials) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) dv[i] = __fadd_rn(dv[i], more[q][i]);
                }
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = __fadd_rn(v[i], dv[i]);
          if (!GATHER) store4<float>(x + g * 4, v);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          held[it][i % VEC] = v[i];
          sum_sq = fmaf(v[i], v[i], sum_sq);
        }
      } else {
        float v = x[g];
        if (HAS_DELTA) {
          float dv = to_float(d[g]);
          for (int p = 1; p < partials; ++p) dv = __fadd_rn(dv, to_float(d[p * partial_stride + g]));   // scalar path: widths no multiple of 4
          v = __fadd_rn(v, dv);
          if (!GATHER) x[g] = v;
        }
        held[it][0] = v;
        sum_sq = fmaf(v, v, sum_sq);
      }
    }
  }
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(width) + eps);
#pragma unroll
  for (int it = 0; it < PER_THREAD; ++it) {
    const int g = threadIdx.x + it * blockDim.x;
    if (g < groups) {
      if (VEC == 4) {
        float w[4], r[4];
        if (GAIN_AHEAD) {
#pragma unroll
          for (int i = 0; i < 4; ++i) w[i] = gain[GAIN_AHEAD ? it : 0][i % VEC];
        } else {
          load4<float>(weight + g * 4, w);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = __fmul_rn(__fmul_rn(held[it][i % VEC], inv), w[i]);
        store4<TO>(y + g * 4, r);
      } else {
        const float w = GAIN_AHEAD ? gain[GAIN_AHEAD ? it : 0][0] : weight[g];
        y[g] = from_float<TO>(__fmul_rn(__fmul_rn(held[it][0], inv), w));
      }
    }
  }
}

template <typename TD, typename TO, bool HAS_DELTA>
static int launch_add_rmsnorm(float* resid, const void* delta, const int* rows, const float* weight,
                              float eps, void* out, int n, int width, int partials, long long partial_stride,
                              cudaStream_t stream) {
  const bool vec = width % 4 == 0;
  const int groups = vec ? width / 4 : width;
  // Few rows (decode): latency counts, one group per thread.  Many rows (prompts): bandwidth
  // counts, small blocks whose threads each keep up to eight groups in flight.
  const bool narrow = groups <= 2048 && n <= 256;
  const bool two = narrow && groups > 1024;   // rows of up to 8192: two groups per thread
  int threads = ((two ? (groups + 1) / 2 : groups) + 31) / 32 * 32;
  if (!narrow) {
    threads = ((groups + NORM_MAX_PER_THREAD - 1) / NORM_MAX_PER_THREAD + 31) / 32 * 32;
    threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
  }
  if (static_cast<long long>(threads) * NORM_MAX_PER_THREAD < groups) return SHRIKE_BAD_ARGUMENT;
#define SHRIKE_NORM_LAUNCH_T(G, V, T)                                                              \
  launch_dependent(add_rmsnorm_kernel<TD, TO, HAS_DELTA, G, V, T>, n, threads, 0, stream, resid,   \
                   static_cast<const TD*>(delta), rows, weight, eps, static_cast<TO*>(out), width, partials,  \
                   partial_stride)
#define SHRIKE_NORM_LAUNCH(G, V)                                                                   \
  do { if (two) SHRIKE_NORM_LAUNCH_T(G, V, 2); else if (narrow) SHRIKE_NORM_LAUNCH_T(G, V, 1);   \
       else SHRIKE_NORM_LAUNCH_T(G, V, NORM_MAX_PER_THREAD); } while (0)
  if (rows) { if (vec) SHRIKE_NORM_LAUNCH(true, 4); else SHRIKE_NORM_LAUNCH(true, 1); }
  else { if (vec) SHRIKE_NORM_LAUNCH(false, 4); else SHRIKE_NORM_LAUNCH(false, 1); }
#undef SHRIKE_NORM_LAUNCH
#undef SHRIKE_NORM_LAUNCH_T
  return SHRIKE_OK;
}

// resid [*, width] float32 (updated in place unless rows != null); delta may be null.
SHRIKE_API int shrike_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const int* rows,
                                  const float* weight, float eps, void* out, int out_dtype, int n,
                                  int width, int partials, long long partial_stride, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (width <= 0 || partials < 1) return SHRIKE_BAD_ARGUMENT;
  const bool has_delta = delta != nullptr;
  if (has_delta && delta_dtype != SHRIKE_F32 && delta_dtype != SHRIKE_BF16) return SHRIKE_BAD_ARGUMENT;
  int status = SHRIKE_OK;
#define SHRIKE_NORM_CASE(TD, TO, HD) \
  status = launch_add_rmsnorm<TD, TO, HD>(resid, delta, rows, weight, eps, out, n, width, partials, partial_stride, stream)
  if (out_dtype == SHRIKE_F32) {
    if (!has_delta) SHRIKE_NORM_CASE(float, float, false);
    else if (delta_dtype == SHRIKE_F32) SHRIKE_NORM_CASE(float, float, true);
    else SHRIKE_NORM_CASE(__nv_bfloat16, float, true);
  } else if (out_dtype == SHRIKE_BF16) {
    if (!has_delta) SHRIKE_NORM_CASE(float, __nv_bfloat16, false);
    else if (delta_dtype == SHRIKE_F32) SHRIKE_NORM_CASE(float, __nv_bfloat16, true);
    else SHRIKE_NORM_CASE(__nv_bfloat16, __nv_bfloat16, true);
  } else {
    return SHRIKE_BAD_ARGUMENT;
  }
#undef SHRIKE_NORM_CASE
  if (status != SHRIKE_OK) return status;  // the width exceeds what one block can hold (32768 / 8192 odd)
  return shrike_launch_status();
}

// ------------------------------------------------------------- SiLU * up
// out[r, c] = silu(gate_up[r, c]) * gate_up[r, inter + c], silu(g) = g / (1 + exp(-g)),
// in float32 with one rounding.  VEC elements per thread and access (16 bytes when the
// row length allows, else one).
// `block`: how gate and up columns lie in a row of gate_up.  0: all gate columns, then all up
// columns.  b > 0: runs of b gate columns followed by the b up columns of the same features
// (the order in which a fused gate/up matrix keeps its rows for the tensor-core product's own
// activation epilogue); b is a multiple of VEC.
template <typename T, int VEC>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int rows, int block) {
  let_dependents_start();
  wait_for_previous();
  // blockIdx.y walks the rows, blockIdx.x and the threads a row's groups of VEC columns: no division
  // by the row length anywhere.  Two groups per thread and round, so that four loads are in flight
  // before the arithmetic starts.
  constexpr int ROUND = 2;
  const int groups_per_row = inter / VEC;
  const int stride = gridDim.x * blockDim.x;
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const T* in_row = gate_up + static_cast<size_t>(row) * 2 * inter;
    T* out_row = out + static_cast<size_t>(row) * inter;
    for (int first = blockIdx.x * blockDim.x + threadIdx.x; first < groups_per_row; first += ROUND * stride) {
      Pack g[ROUND], u[ROUND];
#pragma unroll
      for (int k = 0; k < ROUND; ++k) {
        const int group = first + k * stride;
        if (group < groups_per_row) {
          const int col = group * VEC;
          const T* g_ptr = in_row + (block > 0 ? (col / block) * 2 * block + col % block : col);
          g[k] = *reinterpret_cast<const Pack*>(g_ptr);
          u[k] = *reinterpret_cast<const Pack*>(g_ptr + (block > 0 ? block : inter));
        }
      }
#pragma unroll
      for (int k = 0; k < ROUND; ++k) {
        const int group = first + k * stride;
        if (group >= groups_per_row) continue;
        Pack r;
#pragma unroll
        for (int j = 0; j < VEC; ++j) r.v[j] = from_float<T>(silu_times<T>(to_float(g[k].v[j]), to_float(u[k].v[j])));
        *reinterpret_cast<Pack*>(out_row + group * VEC) = r;
      }
    }
  }
}

// Rows whose gate and up columns alternate in runs of 16 bfloat16 (32 bytes each): a thread takes a
// whole run pair, 64 contiguous bytes in and 32 out, so a warp reads 2 KiB in one piece.  (With a
// thread per 16-byte group the gate loads of a warp touch every other 32 bytes, the up loads the
// rest: the same bytes, twice the lines per instruction.)
__global__ void silu_mul_runs16_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter, int rows) {
  let_dependents_start();
  wait_for_previous();
  const int runs_per_row = inter / 16;
  const int stride = gridDim.x * blockDim.x;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const uint4* in_row = reinterpret_cast<const uint4*>(gate_up + static_cast<size_t>(row) * 2 * inter);
    uint4* out_row = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * inter);
    for (int run = blockIdx.x * blockDim.x + threadIdx.x; run < runs_per_row; run += stride) {
      uint4 in[4];   // gate 0..7, gate 8..15, up 0..7, up 8..15
#pragma unroll
      for (int k = 0; k < 4; ++k) in[k] = in_row[run * 4 + k];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&in[half]);
        const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&in[2 + half]);
        uint4 packed;
        __nv_bfloat16* r = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = from_float<__nv_bfloat16>(silu_times<__nv_bfloat16>(to_float(g[j]), to_float(u[j])));
        out_row[run * 2 + half] = packed;
      }
    }
  }
}

template <typename T>
static void launch_silu_mul(const void* gate_up, void* out, int n, int inter, int block, cudaStream_t stream) {
  if (sizeof(T) == 2 && block == 16 && inter % 16 == 0 &&
      (reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
    const int threads = 256, runs_per_row = inter / 16;
    const dim3 grid(max(1, min(64, (runs_per_row + threads - 1) / threads)), max(1, min(n, 65535)));
    launch_dependent(silu_mul_runs16_kernel, grid, threads, 0, stream, static_cast<const __nv_bfloat16*>(gate_up),
                     static_cast<__nv_bfloat16*>(out), inter, n);
    return;
  }
  constexpr int WIDE = 16 / sizeof(T);
  const bool vec = inter % WIDE == 0 && block % WIDE == 0 &&
                   (reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  const int groups_per_row = vec ? inter / WIDE : inter;
  const int threads = 256;
  // a row's groups over as many blocks as give each thread one round of two; one row of blocks per row
  const int across = max(1, min(64, (groups_per_row + 2 * threads - 1) / (2 * threads)));
  const int down = max(1, min(n, 65535));
  const dim3 grid(across, down);
  if (vec)
    launch_dependent(silu_mul_kernel<T, WIDE>, grid, threads, 0, stream, static_cast<const T*>(gate_up),
                     static_cast<T*>(out), inter, n, block);
  else
    launch_dependent(silu_mul_kernel<T, 1>, grid, threads, 0, stream, static_cast<const T*>(gate_up),
                     static_cast<T*>(out), inter, n, block);
}

SHRIKE_API int shrike_silu_mul(const void* gate_up, void* out, int dtype, int n, int inter, int block, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (inter <= 0 || block < 0 || (block > 0 && inter % block)) return SHRIKE_BAD_ARGUMENT;
  if (dtype == SHRIKE_F32) launch_silu_mul<float>(gate_up, out, n, inter, block, stream);
  else if (dtype == SHRIKE_BF16) launch_silu_mul<__nv_bfloat16>(gate_up, out, n, inter, block, stream);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

// --------------------------------------- bias + rotary + key/value store
// One thread per rotation pair; blockIdx.x is the token, blockIdx.y a slice of the
// (head, pair) space over the q, k and v heads (many slices for few tokens, one for many).  qkv is the float32 result of the fused projection,
// [n, (H + 2 Hkv) * D]: q heads, then k heads, then v heads.  The angle of pair j
// is float(position) * inv_freq[j]; pair j rotates elements j and j + D/2.
// Rotated q goes to q_out; rotated k and plain v go to the cache at slots[token]
// (when caches are given) and to k_out / v_out (when given).
template <typename T>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                                     const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     const int* __restrict__ slots, T* __restrict__ k_out, T* __restrict__ v_out,
                                     int num_heads, int num_kv_heads, int head_dim, long long num_slots,
                                     int partials, long long partial_stride, int wide) {
  let_dependents_start();
  // Before the wait: what no kernel writes (the step's positions and slots, the bias, the
  // frequencies) and the angle of this thread's first pair, while the projection still runs.
  const int token = blockIdx.x;
  const int half = head_dim / 2;
  const int q_width = num_heads * head_dim, kv_width = num_kv_heads * head_dim;
  const float* row = qkv + static_cast<size_t>(token) * (q_width + 2 * kv_width);
  long long slot = -1;
  if (k_cache != nullptr) {
    slot = slots[token];
    if (slot < 0 || slot >= num_slots) slot = -1;  // never store outside the pool
  }
  const float pos = static_cast<float>(positions[token]);
  const int pairs = (num_heads + 2 * num_kv_heads) * half;
  const int first = blockIdx.y * blockDim.x + threadIdx.x;
  float first_s = 0.f, first_c = 1.f, first_bias_lo = 0.f, first_bias_hi = 0.f;
  if (gridDim.y > 1 && first < pairs) {
    const int head = first / half, j = first - head * half;
    if (inv_freq != nullptr && head < num_heads + num_kv_heads) sincosf(__fmul_rn(pos, inv_freq[j]), &first_s, &first_c);
    if (bias != nullptr) {
      first_bias_lo = bias[head * head_dim + j];
      first_bias_hi = bias[head * head_dim + j + half];
    }
  }
  wait_for_previous();
  // A block that walks all heads of its token computes the token's angles once, not once per head.
  __shared__ float2 angle[128];
  const bool shared_angles = gridDim.y == 1 && inv_freq != nullptr && half <= 128;
  if (shared_angles) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float s, c;
      sincosf(__fmul_rn(pos, inv_freq[j]), &s, &c);
      angle[j] = make_float2(s, c);
    }
    __syncthreads();
  }
  if (wide && shared_angles) {
    // whole rows (prompts): four pairs per thread with 16-byte loads and packed stores
    for (int idx = threadIdx.x; idx < pairs / 4; idx += blockDim.x) {
      const int head = idx / (half / 4), j = (idx - head * (half / 4)) * 4;
      const bool is_q = head < num_heads, is_k = !is_q && head < num_heads + num_kv_heads;
      const int lo = head * head_dim + j, hi = lo + half;
      float a[4], b[4], ra[4], rb[4];
      load4<float>(row + lo, a);
      load4<float>(row + hi, b);
      if (bias != nullptr) {
        float ba[4], bb[4];
        load4<float>(bias + lo, ba);
        load4<float>(bias + hi, bb);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          a[e] = __fadd_rn(a[e], ba[e]);
          b[e] = __fadd_rn(b[e], bb[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ra[e] = a[e];
        rb[e] = b[e];
        if (is_q || is_k) {
          const float s = angle[j + e].x, c = angle[j + e].y;
          ra[e] = __fsub_rn(__fmul_rn(a[e], c), __fmul_rn(b[e], s));
          rb[e] = __fadd_rn(__fmul_rn(b[e], c), __fmul_rn(a[e], s));
        }
      }
      if (is_q) {
        T* dst = q_out + static_cast<size_t>(token) * q_width;
        store4<T>(dst + lo, ra);
        store4<T>(dst + hi, rb);
      } else {
        const int base = is_k ? q_width : q_width + kv_width;
        const int clo = lo - base, chi = hi - base;
        T* cache = is_k ? k_cache : v_cache;
        T* extra = is_k ? k_out : v_out;
        if (slot >= 0) {
          T* dst = cache + static_cast<size_t>(slot) * kv_width;
          store4<T>(dst + clo, ra);
          store4<T>(dst + chi, rb);
        }
        if (extra != nullptr) {
          T* dst = extra + static_cast<size_t>(token) * kv_width;
          store4<T>(dst + clo, ra);
          store4<T>(dst + chi, rb);
        }
      }
    }
    return;
  }
  for (int idx = first; idx < pairs; idx += gridDim.y * blockDim.x) {
    const int head = idx / half, j = idx - head * half;
    const bool is_q = head < num_heads, is_k = !is_q && head < num_heads + num_kv_heads;
    const int lo = head * head_dim + j, hi = lo + half;  // columns of the row
    const bool ahead = gridDim.y > 1 && idx == first;    // this pair's bias and angle are at hand
    float a = sum_partials(row + lo, partial_stride, partials);   // slices of a K-split projection, added in order
    float b = sum_partials(row + hi, partial_stride, partials);
    if (bias != nullptr) {
      a = __fadd_rn(a, ahead ? first_bias_lo : bias[lo]);
      b = __fadd_rn(b, ahead ? first_bias_hi : bias[hi]);
    }
    float ra = a, rb = b;
    if (inv_freq != nullptr && (is_q || is_k)) {
      float s, c;
      if (ahead) {
        s = first_s;
        c = first_c;
      } else if (shared_angles) {
        s = angle[j].x;
        c = angle[j].y;
      } else {
        sincosf(__fmul_rn(pos, inv_freq[j]), &s, &c);
      }
      ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
      rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
    }
    if (is_q) {
      T* dst = q_out + static_cast<size_t>(token) * q_width;
      dst[lo] = from_float<T>(ra);
      dst[hi] = from_float<T>(rb);
    } else {
      const int base = is_k ? q_width : q_width + kv_width;
      const int clo = lo - base, chi = hi - base;  // columns within the k (or v) heads
      T* cache = is_k ? k_cache : v_cache;
      T* extra = is_k ? k_out : v_out;
      if (slot >= 0) {
        T* dst = cache + static_cast<size_t>(slot) * kv_width;
        dst[clo] = from_float<T>(ra);
        dst[chi] = from_float<T>(rb);
      }
      if (extra != nullptr) {
        T* dst = extra + static_cast<size_t>(token) * kv_width;
        dst[clo] = from_float<T>(ra);
        dst[chi] = from_float<T>(rb);
      }
    }
  }
}

SHRIKE_API int shrike_rope_kv_write(const float* qkv, const float* bias, const int* positions,
                                    const float* inv_freq, void* q_out, void* k_cache, void* v_cache,
                                    const int* slots, void* k_out, void* v_out, int dtype, int n,
                                    int num_heads, int num_kv_heads, int head_dim, long long num_slots,
                                    int partials, long long partial_stride, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (partials < 1) return SHRIKE_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim % 2 || num_heads <= 0 || num_kv_heads <= 0) return SHRIKE_BAD_ARGUMENT;
  if ((k_cache == nullptr) != (v_cache == nullptr)) return SHRIKE_BAD_ARGUMENT;
  if ((k_out == nullptr) != (v_out == nullptr)) return SHRIKE_BAD_ARGUMENT;
  const int pairs = (num_heads + 2 * num_kv_heads) * (head_dim / 2);
  const int threads = n >= 256 ? 256 : 64;
  const int slices = n >= 256 ? 1 : (pairs + threads - 1) / threads;
  if (slices > 65535) return SHRIKE_BAD_ARGUMENT;
  const dim3 grid(n, slices);
  // whole rows with 16-byte accesses: one slice, a single array, pairs in fours, every pointer aligned
  const uintptr_t addresses = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(bias) |
                              reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
                              reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(k_out) |
                              reinterpret_cast<uintptr_t>(v_out);
  const int wide = slices == 1 && partials == 1 && head_dim % 8 == 0 && addresses % 16 == 0 ? 1 : 0;
#define SHRIKE_ROPE_CASE(T)                                                                         \
  launch_dependent(rope_kv_write_kernel<T>, grid, threads, 0, stream,                               \
      qkv, bias, positions, inv_freq, static_cast<T*>(q_out), static_cast<T*>(k_cache),             \
      static_cast<T*>(v_cache), slots, static_cast<T*>(k_out), static_cast<T*>(v_out), num_heads,   \
      num_kv_heads, head_dim, num_slots, partials, partial_stride, wide)
  if (dtype == SHRIKE_F32) SHRIKE_ROPE_CASE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_ROPE_CASE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_ROPE_CASE
  return shrike_launch_status();
}

// ---------------------------------------------------- key/value store only
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new,
                                T* __restrict__ k_cache, T* __restrict__ v_cache,
                                const int* __restrict__ slots, int kv_width, long long num_slots) {
  let_dependents_start();
  wait_for_previous();
  const int token = blockIdx.x;
  const long long slot = slots[token];
  if (slot < 0 || slot >= num_slots) return;
  for (int i = threadIdx.x; i < kv_width; i += blockDim.x) {
    k_cache[static_cast<size_t>(slot) * kv_width + i] = k_new[static_cast<size_t>(token) * kv_width + i];
    v_cache[static_cast<size_t>(slot) * kv_width + i] = v_new[static_cast<size_t>(token) * kv_width + i];
  }
}

SHRIKE_API int shrike_kv_write(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                               const int* slots, int dtype, int n, int kv_width, long long num_slots,
                               cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (kv_width <= 0) return SHRIKE_BAD_ARGUMENT;
  if (dtype == SHRIKE_F32)
    kv_write_kernel<float><<<n, 128, 0, stream>>>(static_cast<const float*>(k_new), static_cast<const float*>(v_new),
                                                  static_cast<float*>(k_cache), static_cast<float*>(v_cache), slots, kv_width, num_slots);
  else if (dtype == SHRIKE_BF16)
    kv_write_kernel<__nv_bfloat16><<<n, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new),
        static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), slots, kv_width, num_slots);
  else
    return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}
