// Paged grouped-query attention, any query length, all float32 arithmetic.
//
// One warp per (token, query head).  A query at sequence position p sees the keys
// [max(0, p - window + 1), p]; p = ctx_len - q_len + t for the t-th new token of
// its sequence (the end-aligned causal mask of shrike/engine/model_runner.py:146-148
// and shrike/models/qwen.py:243-248).  Scores, scale, softmax and PV follow
// model_runner.py:129-136 in float32; keys are walked 32 at a time with a running
// maximum and sum.  Key j of a sequence lives in page table[j / page_size], row
// j % page_size.  The work for one (token, head) does not depend on what else is
// in the batch, so results are the same however requests are cut or mixed.
//
// Built once per head size: -DSHRIKE_HEAD_DIM=<multiple of 16, at most 256>.
#include "common.cuh"

#ifndef SHRIKE_HEAD_DIM
#error "compile with -DSHRIKE_HEAD_DIM=<head size>"
#endif
static_assert(SHRIKE_HEAD_DIM % 16 == 0 && SHRIKE_HEAD_DIM >= 16 && SHRIKE_HEAD_DIM <= 256,
              "head size must be a multiple of 16 in [16, 256]");

constexpr int D = SHRIKE_HEAD_DIM;
constexpr int WARPS = 4;
constexpr int DPL = (D + 31) / 32;  // output elements per lane

template <typename T> struct Vec16;  // 16 consecutive elements
template <> struct Vec16<float> {
  float4 v[4];
  __device__ __forceinline__ void load(const float* p) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __ldg(q + i);
  }
  __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(v)[i]; }
};
template <> struct Vec16<__nv_bfloat16> {
  uint4 v[2];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    v[0] = __ldg(q);
    v[1] = __ldg(q + 1);
  }
  __device__ __forceinline__ float get(int i) const {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(v)[i]);
  }
};

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ block_table,
                               int max_blocks, const int* __restrict__ q_start,
                               const int* __restrict__ ctx_len, const int* __restrict__ seq_of_token,
                               int num_heads, int num_kv_heads, int page_size, int num_pages,
                               float scale, int window, T* __restrict__ out, int num_tokens) {
  __shared__ float q_shared[WARPS][D];
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long work = static_cast<long long>(blockIdx.x) * WARPS + warp;
  if (work >= static_cast<long long>(num_tokens) * num_heads) return;
  const int token = static_cast<int>(work / num_heads);
  const int head = static_cast<int>(work - static_cast<long long>(token) * num_heads);
  const int kv_head = head / (num_heads / num_kv_heads);
  const int seq = seq_of_token[token];
  const int start = q_start[seq];
  const int q_len = q_start[seq + 1] - start;
  const int last = ctx_len[seq] - q_len + (token - start);
  const int first = window > 0 ? max(0, last - window + 1) : 0;
  const int* table = block_table + static_cast<size_t>(seq) * max_blocks;

  const T* q_row = q + (static_cast<size_t>(token) * num_heads + head) * D;
  for (int d = lane; d < D; d += 32) q_shared[warp][d] = to_float(q_row[d]);
  __syncwarp();

  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  float running_max = -INFINITY, running_sum = 0.f;
  const size_t row_stride = static_cast<size_t>(num_kv_heads) * D;

  for (int base = first; base <= last; base += 32) {
    const int key = base + lane;
    const bool valid = key <= last;
    long long row = -1;
    if (valid) {
      const int block = key / page_size;
      const int page = block < max_blocks ? table[block] : -1;
      if (page >= 0 && page < num_pages) row = static_cast<long long>(page) * page_size + (key - block * page_size);
    }
    float score = -INFINITY;
    if (row >= 0) {
      const T* k_row = k_cache + static_cast<size_t>(row) * row_stride + static_cast<size_t>(kv_head) * D;
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        Vec16<T> chunk;
        chunk.load(k_row + c * 16);
#pragma unroll
        for (int i = 0; i < 16; ++i) dot = fmaf(q_shared[warp][c * 16 + i], chunk.get(i), dot);
      }
      score = dot * scale;
    }
    const float tile_max = warp_max(score);
    const float new_max = fmaxf(running_max, tile_max);
    // new_max is finite: the query's own key is always present and valid
    const float correction = expf(running_max - new_max);
    const float p = row >= 0 ? expf(score - new_max) : 0.f;
    running_sum = running_sum * correction + warp_sum(p);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] *= correction;
    const int count = min(32, last - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long row_j = __shfl_sync(0xffffffffu, row, j);
      if (row_j < 0) continue;
      const T* v_row = v_cache + static_cast<size_t>(row_j) * row_stride + static_cast<size_t>(kv_head) * D;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pj, to_float(v_row[d]), acc[i]);
      }
    }
  }
  T* out_row = out + (static_cast<size_t>(token) * num_heads + head) * D;
  const float inv = running_sum > 0.f ? 1.0f / running_sum : 0.f;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out_row[d] = from_float<T>(acc[i] * inv);
  }
}

SHRIKE_API int shrike_attention_head_dim() { return D; }

SHRIKE_API int shrike_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                              const int* block_table, int max_blocks, const int* q_start,
                                              const int* ctx_len, const int* seq_of_token, int dtype,
                                              int num_tokens, int num_heads, int num_kv_heads,
                                              int page_size, int num_pages, float scale, int window,
                                              void* out, cudaStream_t stream) {
  if (num_tokens <= 0) return SHRIKE_OK;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || page_size <= 0 || max_blocks <= 0)
    return SHRIKE_BAD_ARGUMENT;
  const long long work = static_cast<long long>(num_tokens) * num_heads;
  const long long blocks = (work + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return SHRIKE_BAD_ARGUMENT;
#define SHRIKE_ATTN_CASE(T)                                                                        \
  paged_attention_generic_kernel<T><<<static_cast<int>(blocks), WARPS * 32, 0, stream>>>(           \
      static_cast<const T*>(q), static_cast<const T*>(k_cache), static_cast<const T*>(v_cache),     \
      block_table, max_blocks, q_start, ctx_len, seq_of_token, num_heads, num_kv_heads, page_size,  \
      num_pages, scale, window, static_cast<T*>(out), num_tokens)
  if (dtype == SHRIKE_F32) SHRIKE_ATTN_CASE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_ATTN_CASE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_ATTN_CASE
  return shrike_launch_status();
}
