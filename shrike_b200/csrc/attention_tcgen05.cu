// Paged causal attention for portions (q_len > 1) in bfloat16 on the fifth-generation
// tensor cores.  One CTA owns 128 queries of one head of one sequence and walks the keys
// 64 at a time:
//   S = Q K^T      tcgen05.mma, M 128 x N 64 x K head size, accumulator in tensor memory
//   softmax        four warps, ONE THREAD PER QUERY ROW: the row of S comes out of tensor
//                  memory with tcgen05.ld, scale, mask, running maximum and sum in float32,
//                  probabilities go to shared memory as bfloat16 in the MMA's swizzled layout
//   O += P V       tcgen05.mma, M 128 x N head size x K 64; O stays in tensor memory across
//                  tiles and is rescaled there (tcgen05.ld / st) when a row's maximum moved
// Keys and values arrive by TMA, one box per page and 64-element half of the head (the
// block table is read by the producer thread), double-buffered; the query tile by TMA once.
// Roles: warp 0 TMA producer, warp 1 MMA issuer (one elected lane each), warps 2..5 softmax
// and epilogue.  tcgen05.commit arrives on mbarriers: s_full after S, kv_free after PV;
// MMAs execute in issue order, so "S of tile i+1 is ready" also says "PV of tile i is done".
// Mask and window as everywhere: a query at position p sees keys [max(0, p - window + 1), p].
// Rows of a page beyond the context may hold anything (a page is reused without clearing):
// scores are masked by selection, and the value rows beyond the context are zeroed in shared
// memory before PV, because 0 * NaN would not be 0.
// Every wait is bounded (status word, CTA-wide abort flag); no TMA load uses multicast.
// Tensor memory is allocated BEFORE dependents are allowed to start, so that a dependent
// kernel that also wants tensor memory cannot starve a CTA of this one it is waiting for.
//
// Built once per head size; serves head sizes 64 and 128 and page sizes 8, 16, 32, 64.
#include "blackwell.cuh"

#ifndef SHRIKE_HEAD_DIM
#error "compile with -DSHRIKE_HEAD_DIM=<head size>"
#endif

#if SHRIKE_HEAD_DIM == 64 || SHRIKE_HEAD_DIM == 128
#define SHRIKE_TC_ATTENTION 1

namespace tcattn {
using namespace bw;

constexpr int D = SHRIKE_HEAD_DIM;
constexpr int BM = 128, BN = 64;
constexpr int HALVES = D / 64;                 // 64-element groups of the head size
constexpr int THREADS = 192;
constexpr int STAGES = 2;
constexpr int Q_HALF = BM * 128, KV_HALF = BN * 128;          // bytes of one 64-element-wide sub-tile
constexpr int Q_BYTES = HALVES * Q_HALF, KV_BYTES = HALVES * KV_HALF, P_BYTES = BM * BN * 2;
constexpr unsigned TMEM_COLS = D == 128 ? 256 : 128;           // S: 64 columns, O: D columns
constexpr float LOG2E = 1.4426950408889634f;

enum : int { ERR_PRODUCER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_DRAIN = 14, ERR_ALIGNMENT = 15 };

struct Shared {
  unsigned long long q_full, s_full, p_full, o_done;
  unsigned long long kv_full[STAGES], kv_free[STAGES];
  unsigned tmem_base;
  volatile int abort;
};
// two CTAs must fit an SM (233,472 bytes, 1 KiB reserved per CTA): no slack for alignment is added; the
// dynamic window starts 1 KiB-aligned (declared so below), and the kernel checks that it does.
constexpr size_t SMEM_BYTES = Q_BYTES + STAGES * 2 * KV_BYTES + P_BYTES + sizeof(Shared);

struct Args {
  const int* block_table;
  const int* q_start;
  const int* ctx_len;
  __nv_bfloat16* out;
  int* status;
  int max_blocks, num_heads, num_kv_heads, page_size, num_pages, window, skip_single;
  float scale_log2;
};

__global__ void __launch_bounds__(THREADS, 2)
portions_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const Args args) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int seq = blockIdx.z, head = blockIdx.y;
  const int tile_start = (gridDim.x - 1 - blockIdx.x) * BM;    // long tiles are scheduled first
  const int start = args.q_start[seq];                          // metadata: written before the step's kernels
  const int q_len = args.q_start[seq + 1] - start;
  if (tile_start >= q_len || (q_len == 1 && args.skip_single)) {
    let_dependents_start();
    wait_for_previous();
    return;
  }
  if (smem_u32(smem_raw) & 1023u) {   // the swizzled tiles need 1 KiB alignment
    if (threadIdx.x == 0 && args.status != nullptr) *args.status = ERR_ALIGNMENT;
    let_dependents_start();
    wait_for_previous();
    return;
  }
  unsigned char* q_tile = smem_raw;
  unsigned char* kv_tiles = q_tile + Q_BYTES;                   // [STAGES][K | V]
  unsigned char* p_tile = kv_tiles + STAGES * 2 * KV_BYTES;
  Shared* sh = reinterpret_cast<Shared*>(p_tile + P_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->s_full, 1);
    mbar_init(&sh->p_full, 128);
    mbar_init(&sh->o_done, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->kv_free[s], 1);
    }
    sh->abort = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&sh->tmem_base, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  let_dependents_start();
  wait_for_previous();   // the query and the newest keys come from the kernel before this one

  const unsigned tmem_s = sh->tmem_base, tmem_o = sh->tmem_base + BN;
  const int pos0 = args.ctx_len[seq] - q_len;                   // position of the first new token
  const int kv_head = head / (args.num_heads / args.num_kv_heads);
  const int rows_here = min(BM, q_len - tile_start);
  const int lo = args.window > 0 ? max(0, pos0 + tile_start - args.window + 1) : 0;
  const int hi = pos0 + tile_start + rows_here - 1;             // last key any row of this tile sees
  const int tile_lo = lo / BN, tile_hi = hi / BN;
  const int num_tiles = tile_hi - tile_lo + 1;

  if (warp == 0) {
    if (lane == 0) {
      const int* table = args.block_table + static_cast<size_t>(seq) * args.max_blocks;
      const int pages_per_tile = BN / args.page_size;
      const int nowhere = args.num_pages * args.page_size;      // a row coordinate outside the cache: reads zeros
      mbar_expect_tx(&sh->q_full, Q_BYTES);
      for (int h = 0; h < HALVES; ++h) tma_load_2d(q_tile + h * Q_HALF, &map_q, &sh->q_full, head * D + h * 64, start + tile_start);
      int issued = 0;
      for (int i = 0; i < num_tiles; ++i) {
        const int s = i % STAGES;
        const unsigned phase = (i / STAGES) & 1;
        if (!mbar_wait(&sh->kv_free[s], phase ^ 1, &sh->abort, args.status, ERR_PRODUCER)) break;
        mbar_expect_tx(&sh->kv_full[s], 2 * KV_BYTES);
        unsigned char* k_tile = kv_tiles + s * 2 * KV_BYTES;
        unsigned char* v_tile = k_tile + KV_BYTES;
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int key0 = (tile_lo + i) * BN + pg * args.page_size;
          const int block = key0 / args.page_size;
          int page = (key0 <= hi && block < args.max_blocks) ? table[block] : -1;
          if (page < 0 || page >= args.num_pages) page = -1;
          const int y = page < 0 ? nowhere : page * args.page_size;
          const int at = pg * args.page_size * 128;
          for (int h = 0; h < HALVES; ++h) {
            tma_load_2d(k_tile + h * KV_HALF + at, &map_k, &sh->kv_full[s], kv_head * D + h * 64, y);
            tma_load_2d(v_tile + h * KV_HALF + at, &map_v, &sh->kv_full[s], kv_head * D + h * 64, y);
          }
        }
        issued = i + 1;
      }
      if (sh->abort) {   // copies may still be in flight: wait for the stages armed last
        for (int i = max(0, issued - STAGES); i < issued; ++i) {
          bool landed = false;
          for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries)
            landed = mbar_try_wait(&sh->kv_full[i % STAGES], (i / STAGES) & 1);
          if (!landed && args.status != nullptr) *args.status = ERR_DRAIN;
        }
        bool landed = false;
        for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries) landed = mbar_try_wait(&sh->q_full, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc_s = instruction_descriptor(BM, BN, false);
      const unsigned idesc_o = instruction_descriptor(BM, D, true);
      const unsigned q_addr = smem_u32(q_tile), p_addr = smem_u32(p_tile);
      bool ok = mbar_wait(&sh->q_full, 0, &sh->abort, args.status, ERR_MMA);
      for (int i = 0; i < num_tiles && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&sh->kv_full[s], (i / STAGES) & 1, &sh->abort, args.status, ERR_MMA);
        if (!ok) break;
        fence_after_sync();
        const unsigned k_addr = smem_u32(kv_tiles + s * 2 * KV_BYTES), v_addr = k_addr + KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const unsigned off = (kk / 4) * Q_HALF + (kk % 4) * 32, koff = (kk / 4) * KV_HALF + (kk % 4) * 32;
          umma(tmem_s, smem_descriptor(q_addr + off), smem_descriptor(k_addr + koff), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sh->s_full);
        ok = mbar_wait(&sh->p_full, i & 1, &sh->abort, args.status, ERR_MMA);
        if (!ok) break;
        fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)   // 16 keys a step: P advances 32 bytes in its rows, V 16 rows
          umma(tmem_o, smem_descriptor(p_addr + kk * 32), smem_descriptor(v_addr + kk * 16 * 128, KV_HALF, 1024), idesc_o,
               (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh->kv_free[s]);
      }
      if (ok) umma_commit(&sh->o_done);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int t = tile_start + row;
    const int last = t < q_len ? pos0 + t : -1;
    const int first = args.window > 0 ? max(0, last - args.window + 1) : 0;
    const unsigned lane_base = static_cast<unsigned>(quarter * 32) << 16;
    float row_max = -INFINITY, row_sum = 0.f;
    bool ok = true;
    for (int i = 0; i < num_tiles && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(&sh->s_full, i & 1, &sh->abort, args.status, ERR_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);   // the warp stays together: the tensor-memory accesses below are warp-wide
      if (!ok) break;
      fence_after_sync();
      unsigned v0[32], v1[32];
      tmem_load32(tmem_s + lane_base, v0);
      tmem_load32(tmem_s + lane_base + 32, v1);
      tmem_wait_load();
      const int key_base = (tile_lo + i) * BN;
      float tile_max = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int k0 = key_base + j, k1 = key_base + 32 + j;
        const float a = (k0 >= first && k0 <= last) ? __uint_as_float(v0[j]) * args.scale_log2 : -INFINITY;
        const float b = (k1 >= first && k1 <= last) ? __uint_as_float(v1[j]) * args.scale_log2 : -INFINITY;
        v0[j] = __float_as_uint(a);
        v1[j] = __float_as_uint(b);
        tile_max = fmaxf(tile_max, fmaxf(a, b));
      }
      const float new_max = fmaxf(row_max, tile_max);
      const float base = new_max == -INFINITY ? 0.f : new_max;   // a row that has seen no key yet
      const float correction = exp2f(row_max - base);           // exp2(-inf) = 0
      row_max = new_max;
      float sum = 0.f;
      unsigned char* p_row = p_tile + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {   // eight 16-byte chunks of the row, chunk c at (c xor row mod 8)
        unsigned packed[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = c * 8 + e * 2;
          const float x0 = exp2f(__uint_as_float(j < 32 ? v0[j] : v1[j - 32]) - base);
          const float x1 = exp2f(__uint_as_float(j + 1 < 32 ? v0[j + 1] : v1[j + 1 - 32]) - base);
          sum += x0 + x1;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(x0, x1);
          packed[e] = *reinterpret_cast<const unsigned*>(&pair);
        }
        *reinterpret_cast<uint4*>(p_row + ((c ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      row_sum = row_sum * correction + sum;
      // value rows beyond the context: zero them (only the tile that holds the last key has any)
      if (tile_lo + i == tile_hi && (hi + 1) % BN != 0) {
        unsigned char* v_tile = kv_tiles + s * 2 * KV_BYTES + KV_BYTES;
        const int first_bad = hi + 1 - key_base;
        for (int idx = threadIdx.x - 64; idx < (BN - first_bad) * HALVES * 8; idx += 128) {
          const int r = first_bad + idx / (HALVES * 8), rest = idx % (HALVES * 8);
          *reinterpret_cast<uint4*>(v_tile + (rest / 8) * KV_HALF + r * 128 + (rest % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // O of the tiles before is scaled by `correction`; skipped when no row of the warp moved
      if (i > 0 && __any_sync(0xffffffffu, correction != 1.0f)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          unsigned o[32];
          tmem_load32(tmem_o + lane_base + c * 32, o);
          tmem_wait_load();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * correction);
          tmem_store32(tmem_o + lane_base + c * 32, o);
        }
        tmem_wait_store();
      }
      fence_before_sync();
      fence_async_shared();
      mbar_arrive(&sh->p_full);
    }
    if (ok) ok = mbar_wait(&sh->o_done, 0, &sh->abort, args.status, ERR_SOFTMAX);
    ok = __all_sync(0xffffffffu, ok);
    fence_after_sync();
    if (ok) {
      const float inv = row_sum > 0.f ? 1.0f / row_sum : 0.f;
      __nv_bfloat16* dst = args.out + (static_cast<size_t>(start + t) * args.num_heads + head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        unsigned o[32];
        tmem_load32(tmem_o + lane_base + c * 32, o);
        tmem_wait_load();
        if (t < q_len) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            unsigned packed[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(o[j + 2 * e]) * inv, __uint_as_float(o[j + 2 * e + 1]) * inv);
              packed[e] = *reinterpret_cast<const unsigned*>(&pair);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_free(sh->tmem_base, TMEM_COLS);
  }
}

}  // namespace tcattn

SHRIKE_API int shrike_attention_tc_available() { return 1; }

// Portions (q_len > 1) of a batch; entries with q_len == 1 are skipped when skip_single.
// q [tokens, heads * D] and out alike; caches [pages, page_size, kv heads, D]; page_size one of
// 8, 16, 32, 64.
SHRIKE_API int shrike_paged_attention_tc_portions(const void* q, const void* k_cache, const void* v_cache,
                                                  const int* block_table, int max_blocks, const int* q_start,
                                                  const int* ctx_len, int num_tokens, int num_seqs, int num_heads,
                                                  int num_kv_heads, int page_size, int num_pages, float scale,
                                                  int window, void* out, int skip_single, int max_q_len, int* status,
                                                  cudaStream_t stream) {
  using namespace tcattn;
  if (num_seqs <= 0 || num_tokens <= 0) return SHRIKE_OK;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || max_blocks <= 0 || max_q_len < 1 ||
      num_seqs > 65535 || num_heads > 65535 || !(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64))
    return SHRIKE_BAD_ARGUMENT;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(portions_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
    if (err != cudaSuccess) return static_cast<int>(err);
    configured = true;
  }
  CUtensorMap map_q, map_k, map_v;
  int rc = bw::tensor_map_bf16(q, num_tokens, num_heads * D, BM, &map_q);
  if (rc != SHRIKE_OK) return rc;
  rc = bw::tensor_map_bf16(k_cache, static_cast<long long>(num_pages) * page_size, num_kv_heads * D, page_size, &map_k);
  if (rc != SHRIKE_OK) return rc;
  rc = bw::tensor_map_bf16(v_cache, static_cast<long long>(num_pages) * page_size, num_kv_heads * D, page_size, &map_v);
  if (rc != SHRIKE_OK) return rc;
  Args args;
  args.block_table = block_table;
  args.q_start = q_start;
  args.ctx_len = ctx_len;
  args.out = static_cast<__nv_bfloat16*>(out);
  args.status = status;
  args.max_blocks = max_blocks;
  args.num_heads = num_heads;
  args.num_kv_heads = num_kv_heads;
  args.page_size = page_size;
  args.num_pages = num_pages;
  args.window = window;
  args.skip_single = skip_single;
  args.scale_log2 = scale * LOG2E;
  const dim3 grid((max_q_len + BM - 1) / BM, num_heads, num_seqs);
  const cudaError_t err = launch_dependent(portions_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, map_q, map_k, map_v, args);
  if (err != cudaSuccess) return static_cast<int>(err);
  return shrike_launch_status();
}

#else  // other head sizes: the mma.sync kernel serves them

SHRIKE_API int shrike_attention_tc_available() { return 0; }
SHRIKE_API int shrike_paged_attention_tc_portions(const void*, const void*, const void*, const int*, int, const int*,
                                                  const int*, int, int, int, int, int, int, float, int, void*, int, int,
                                                  int*, cudaStream_t) {
  return SHRIKE_BAD_ARGUMENT;
}

#endif
