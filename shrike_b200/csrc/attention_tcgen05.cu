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
// Roles: warp 0 TMA producer, warp 1 MMA issuer (one elected lane), warps 2..5 softmax and
// epilogue.  S has two buffers in tensor memory: the scores of tile i + 1 are computed while
// the softmax warps work on tile i, and their exponentials while PV of tile i still runs;
// only writing P (one buffer) and rescaling O wait for that PV (barrier pv_done).
// Keys and values have stages and barriers of their own: a key stage is free again as soon
// as its S is computed, long before the value stage of the same tile, so the keys of the tile
// after next are already on their way while this tile's softmax runs.
// tcgen05.commit arrives on mbarriers: s_full[b] and k_free after S into buffer b, v_free and
// pv_done after PV.
// Mask and window as everywhere: a query at position p sees keys [max(0, p - window + 1), p].
// Rows of a page beyond the context may hold anything (a page is reused without clearing):
// scores are masked by selection, and the value rows beyond the context are zeroed in shared
// memory before PV, because 0 * NaN would not be 0.
// Few query tiles and many keys (a portion of a long prompt beside decoding requests) would leave
// most of the GPU idle: the keys of a query tile are then split across `splits` CTAs, each of which
// leaves its unnormalised output rows with their (base, sum) in scratch, and a second small kernel
// adds the splits up (combine_portions_kernel).
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
constexpr unsigned TMEM_COLS = 256;                            // S: 2 x 64 columns, O: D columns from column 128
constexpr float LOG2E = 1.4426950408889634f;

enum : int { ERR_PRODUCER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_DRAIN = 14, ERR_ALIGNMENT = 15 };

struct Shared {
  unsigned long long q_full, s_full[2], p_full, pv_done;
  unsigned long long k_full[STAGES], k_free[STAGES], v_full[STAGES], v_free[STAGES];
  unsigned tmem_base;
  volatile int abort;
};
// two CTAs must fit an SM (233,472 bytes, 1 KiB reserved per CTA): no slack for alignment is added; the
// dynamic window starts 1 KiB-aligned (declared so below), and the kernel checks that it does.
constexpr size_t SMEM_BYTES = Q_BYTES + STAGES * 2 * KV_BYTES + P_BYTES + sizeof(Shared);

// 2^x on the special-function unit; -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Args {
  const int* block_table;
  const int* q_start;
  const int* ctx_len;
  __nv_bfloat16* out;
  int* status;
  int max_blocks, num_heads, num_kv_heads, page_size, num_pages, window, skip_single;
  float scale_log2;
  int splits;          // CTAs that share a query tile's keys; > 1: results go to the scratch below
  float* partial_o;    // [splits][tokens][heads][D] unnormalised output rows
  float* partial_ml;   // [splits][tokens][heads][2] their base (log2 domain) and sum
  int num_tokens;
  int num_seqs;
  const int* seq_of_token;   // [tokens], for the combine
};

// Which (sequence, query tile) a CTA with work index `work` owns: sequences in order, each with its
// query tiles of BM rows, the last (longest to walk) first; sequences of one token own none when
// skip_single.  Every lane of the calling warp gets the answer; tile_start < 0: no such work.
__device__ __forceinline__ void find_work(const Args& args, int work, int& seq_out, int& tile_start_out) {
  const int lane = threadIdx.x & 31;
  int before = 0;
  seq_out = -1;
  tile_start_out = -1;
  for (int base = 0; base < args.num_seqs; base += 32) {
    const int s = base + lane;
    int tiles = 0;
    if (s < args.num_seqs) {
      const int q_len = args.q_start[s + 1] - args.q_start[s];
      tiles = (q_len == 1 && args.skip_single) ? 0 : (q_len + BM - 1) / BM;
    }
    int inclusive = tiles;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if (lane >= offset) inclusive += other;
    }
    const int first = before + inclusive - tiles;            // work index of this sequence's first tile
    const bool mine = tiles > 0 && work >= first && work < first + tiles;
    const unsigned owner = __ballot_sync(0xffffffffu, mine);
    if (owner != 0) {
      const int src = __ffs(owner) - 1;
      const int first_of_owner = __shfl_sync(0xffffffffu, first, src);
      const int tiles_of_owner = __shfl_sync(0xffffffffu, tiles, src);
      seq_out = base + src;
      tile_start_out = (tiles_of_owner - 1 - (work - first_of_owner)) * BM;
      return;
    }
    before += __shfl_sync(0xffffffffu, inclusive, 31);
  }
}

__global__ void __launch_bounds__(THREADS, 2)
portions_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const Args args) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // CTAs are handed out x first: the heads of a group, which read the same keys and values, run
  // side by side; within a sequence the longest query tiles go first (a causal tile's work grows
  // with its position).
  // CTAs are numbered (head, work, split): `work` counts the query tiles of the batch's portions
  // (find_work), so no CTA is spent on a sequence of one token or on rows a sequence does not have.
  const int head = blockIdx.x, split = blockIdx.z;
  int seq, tile_start;
  find_work(args, blockIdx.y, seq, tile_start);                 // metadata: written before the step's kernels
  if (tile_start < 0) {
    let_dependents_start();
    wait_for_previous();
    return;
  }
  const int start = args.q_start[seq];
  const int q_len = args.q_start[seq + 1] - start;
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
    mbar_init(&sh->s_full[0], 1);
    mbar_init(&sh->s_full[1], 1);
    mbar_init(&sh->p_full, 128);
    mbar_init(&sh->pv_done, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_free[s], 1);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->v_free[s], 1);
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

  const unsigned tmem_s = sh->tmem_base, tmem_o = sh->tmem_base + 2 * BN;   // S buffer b at columns b * 64
  const int pos0 = args.ctx_len[seq] - q_len;                   // position of the first new token
  const int kv_head = head / (args.num_heads / args.num_kv_heads);
  const int rows_here = min(BM, q_len - tile_start);
  const int lo = args.window > 0 ? max(0, pos0 + tile_start - args.window + 1) : 0;
  const int hi = pos0 + tile_start + rows_here - 1;             // last key any row of this tile sees
  const int tile_hi = hi / BN;
  // this CTA's share of the key tiles [lo / BN, tile_hi]: `per` tiles from tile_lo on (none: an empty split)
  const int all_tiles = tile_hi - lo / BN + 1;
  const int per = (all_tiles + args.splits - 1) / args.splits;
  const int tile_lo = lo / BN + split * per;
  const int num_tiles = max(0, min(tile_hi, tile_lo + per - 1) - tile_lo + 1);

  if (warp == 0) {
    // The whole warp runs the loop: lane 0 waits for the stage and arms its barrier, then lane
    // pg looks up page pg of the tile and issues that page's four boxes (K and V, both halves).
    const int* table = args.block_table + static_cast<size_t>(seq) * args.max_blocks;
    const int pages_per_tile = BN / args.page_size;
    const int nowhere = args.num_pages * args.page_size;      // a row coordinate outside the cache: reads zeros
    if (lane == 0 && num_tiles > 0) {
      mbar_expect_tx(&sh->q_full, Q_BYTES);
      for (int h = 0; h < HALVES; ++h) tma_load_2d(q_tile + h * Q_HALF, &map_q, &sh->q_full, head * D + h * 64, start + tile_start);
    }
    // page ids are looked up three tiles ahead of their use, so that the table's latency never
    // sits between a stage becoming free and its copy being issued
    auto look_up = [&](int i) -> int {
      if (lane >= pages_per_tile || i >= num_tiles) return -1;
      const int key0 = (tile_lo + i) * BN + lane * args.page_size;
      const int block = key0 / args.page_size;
      const int page = (key0 <= hi && block < args.max_blocks) ? table[block] : -1;
      return page >= args.num_pages ? -1 : page;
    };
    int page = look_up(0), page_1 = look_up(1), page_2 = look_up(2);
    int issued = 0;
    for (int i = 0; i < num_tiles; ++i) {
      const int s = i % STAGES;
      const unsigned phase = (i / STAGES) & 1;
      const int page_3 = look_up(i + 3);
      unsigned char* k_tile = kv_tiles + s * 2 * KV_BYTES;
      unsigned char* v_tile = k_tile + KV_BYTES;
      const int y = page < 0 ? nowhere : page * args.page_size;
      const int at = lane * args.page_size * 128;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(&sh->k_free[s], phase ^ 1, &sh->abort, args.status, ERR_PRODUCER) ? 1 : 0;
        if (ok) mbar_expect_tx(&sh->k_full[s], KV_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile)
        for (int h = 0; h < HALVES; ++h) tma_load_2d(k_tile + h * KV_HALF + at, &map_k, &sh->k_full[s], kv_head * D + h * 64, y);
      if (lane == 0) {
        ok = mbar_wait(&sh->v_free[s], phase ^ 1, &sh->abort, args.status, ERR_PRODUCER) ? 1 : 0;
        if (ok) mbar_expect_tx(&sh->v_full[s], KV_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile)
        for (int h = 0; h < HALVES; ++h) tma_load_2d(v_tile + h * KV_HALF + at, &map_v, &sh->v_full[s], kv_head * D + h * 64, y);
      issued = i + 1;
      page = page_1;
      page_1 = page_2;
      page_2 = page_3;
    }
    if (lane == 0 && sh->abort) {   // copies may still be in flight: wait for the stages armed last
      for (int i = max(0, issued - STAGES); i < issued; ++i) {
        bool landed = false;
        for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries)
          landed = mbar_try_wait(&sh->k_full[i % STAGES], (i / STAGES) & 1) && mbar_try_wait(&sh->v_full[i % STAGES], (i / STAGES) & 1);
        if (!landed && args.status != nullptr) *args.status = ERR_DRAIN;
      }
      bool landed = num_tiles <= 0;
      for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries) landed = mbar_try_wait(&sh->q_full, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc_s = instruction_descriptor(BM, BN, false);
      const unsigned idesc_o = instruction_descriptor(BM, D, true);
      const unsigned q_addr = smem_u32(q_tile), p_addr = smem_u32(p_tile);
      // S of tile i into buffer i mod 2; issued one tile ahead of the softmax
      auto issue_scores = [&](int i) -> bool {
        const int st = i % STAGES;
        if (!mbar_wait(&sh->k_full[st], (i / STAGES) & 1, &sh->abort, args.status, ERR_MMA)) return false;
        fence_after_sync();
        const unsigned k_addr = smem_u32(kv_tiles + st * 2 * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const unsigned off = (kk / 4) * Q_HALF + (kk % 4) * 32, koff = (kk / 4) * KV_HALF + (kk % 4) * 32;
          umma(tmem_s + (i & 1) * BN, smem_descriptor(q_addr + off), smem_descriptor(k_addr + koff), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sh->s_full[i & 1]);
        umma_commit(&sh->k_free[st]);
        return true;
      };
      bool ok = num_tiles > 0 && mbar_wait(&sh->q_full, 0, &sh->abort, args.status, ERR_MMA);
      if (ok) ok = issue_scores(0);
      for (int i = 0; i < num_tiles && ok; ++i) {
        // buffer (i + 1) mod 2 was last read for tile i - 1, whose P has arrived: it is free
        if (i + 1 < num_tiles) ok = issue_scores(i + 1);
        if (!ok) break;
        ok = mbar_wait(&sh->v_full[i % STAGES], (i / STAGES) & 1, &sh->abort, args.status, ERR_MMA) &&
             mbar_wait(&sh->p_full, i & 1, &sh->abort, args.status, ERR_MMA);
        if (!ok) break;
        fence_after_sync();
        const unsigned v_addr = smem_u32(kv_tiles + (i % STAGES) * 2 * KV_BYTES) + KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)   // 16 keys a step: P advances 32 bytes in its rows, V 16 rows
          umma(tmem_o, smem_descriptor(p_addr + kk * 32), smem_descriptor(v_addr + kk * 16 * 128, KV_HALF, 1024), idesc_o,
               (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh->v_free[i % STAGES]);
        umma_commit(&sh->pv_done);
      }
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
      ok = mbar_wait(&sh->s_full[i & 1], (i >> 1) & 1, &sh->abort, args.status, ERR_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);   // the warp stays together: the tensor-memory accesses below are warp-wide
      if (!ok) break;
      fence_after_sync();
      unsigned v0[32], v1[32];
      tmem_load32(tmem_s + (i & 1) * BN + lane_base, v0);
      tmem_load32(tmem_s + (i & 1) * BN + lane_base + 32, v1);
      tmem_wait_load();
      const int key_base = (tile_lo + i) * BN;
      // most tiles lie wholly inside the row's visible range: only the others pay for masking
      if (key_base < first || key_base + BN - 1 > last) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int k0 = key_base + j, k1 = key_base + 32 + j;
          if (k0 < first || k0 > last) v0[j] = 0xff800000u;   // -inf
          if (k1 < first || k1 > last) v1[j] = 0xff800000u;
        }
      }
      float tile_max = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) tile_max = fmaxf(tile_max, fmaxf(__uint_as_float(v0[j]), __uint_as_float(v1[j])));
      tile_max *= args.scale_log2;   // the scale is positive: the maximum of the raw scores is the one to scale
      // The base of the exponentials follows the running maximum lazily: it moves (and O is
      // rescaled) only when the maximum has grown by more than 2^8; until then probabilities
      // are at most 2^8, which float32 sums and bfloat16 products hold without loss.
      float correction = 1.0f;
      if (tile_max > row_max + 8.0f || row_max == -INFINITY) {
        const float new_max = fmaxf(row_max, tile_max);
        const float base = new_max == -INFINITY ? 0.f : new_max;   // a row that has seen no key yet
        correction = row_max == -INFINITY ? 0.f : fast_exp2(row_max - base);
        row_max = new_max;
      }
      const float base = row_max == -INFINITY ? 0.f : row_max;
      float sum = 0.f;
      unsigned packed[32];   // the row's 64 probabilities as bfloat16 pairs
#pragma unroll
      for (int j = 0; j < 64; j += 2) {
        const float x0 = fast_exp2(fmaf(__uint_as_float(j < 32 ? v0[j] : v1[j - 32]), args.scale_log2, -base));
        const float x1 = fast_exp2(fmaf(__uint_as_float(j + 1 < 32 ? v0[j + 1] : v1[j + 1 - 32]), args.scale_log2, -base));
        sum += x0 + x1;
        const __nv_bfloat162 pair = __floats2bfloat162_rn(x0, x1);
        packed[j / 2] = *reinterpret_cast<const unsigned*>(&pair);
      }
      row_sum = row_sum * correction + sum;
      // P has one buffer and O one accumulator: both belong to PV of the tile before until it is done
      if (i > 0) {
        ok = mbar_wait(&sh->pv_done, (i - 1) & 1, &sh->abort, args.status, ERR_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after_sync();
      }
      unsigned char* p_row = p_tile + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)   // eight 16-byte chunks of the row, chunk c at (c xor row mod 8)
        *reinterpret_cast<uint4*>(p_row + ((c ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      // value rows beyond the context: zero them (only the tile that holds the last key has any)
      if (tile_lo + i == tile_hi && (hi + 1) % BN != 0) {
        ok = mbar_wait(&sh->v_full[s], (i / STAGES) & 1, &sh->abort, args.status, ERR_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
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
    if (ok && num_tiles > 0) ok = mbar_wait(&sh->pv_done, (num_tiles - 1) & 1, &sh->abort, args.status, ERR_SOFTMAX);
    ok = __all_sync(0xffffffffu, ok);
    fence_after_sync();
    if (ok && args.splits > 1) {
      // a split's share: the unnormalised row as it stands in tensor memory, its base and its sum
      const size_t at = (static_cast<size_t>(split) * args.num_tokens + start + t) * args.num_heads + head;
      if (t < q_len) {
        args.partial_ml[2 * at] = num_tiles > 0 ? row_max : -INFINITY;
        args.partial_ml[2 * at + 1] = num_tiles > 0 ? row_sum : 0.f;
      }
      if (num_tiles > 0) {
        float* dst = args.partial_o + at * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          unsigned o[32];
          tmem_load32(tmem_o + lane_base + c * 32, o);
          tmem_wait_load();
          if (t < q_len) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(o[j], o[j + 1], o[j + 2], o[j + 3]);
          }
        }
      }
    } else if (ok) {
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

// Adds up the splits of every query row of the portions: out = sum_s O_s 2^(base_s - M) / sum_s l_s 2^(base_s - M)
// with M the largest base.  One warp per (token, head), lanes over the splits first (bases and sums),
// then over the head size.  Tokens of one-token sequences belong to the other kernel and are left alone.
__global__ void __launch_bounds__(256)
combine_portions_kernel(const Args args) {
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.y * 8 + warp, head = blockIdx.x;
  if (token >= args.num_tokens) return;
  const int seq = args.seq_of_token[token];
  if (args.skip_single && args.q_start[seq + 1] - args.q_start[seq] == 1) return;
  const size_t token_head = static_cast<size_t>(token) * args.num_heads + head;
  const size_t slice = static_cast<size_t>(args.num_tokens) * args.num_heads;
  float m = -INFINITY, l = 0.f;                       // lane s holds split s (at most 32 splits)
  if (lane < args.splits) {
    m = args.partial_ml[2 * (lane * slice + token_head)];
    l = args.partial_ml[2 * (lane * slice + token_head) + 1];
    if (!(l > 0.f)) m = -INFINITY;                    // a split that saw no key of this row
  }
  float base = m;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) base = fmaxf(base, __shfl_xor_sync(0xffffffffu, base, offset));
  const float weight = m == -INFINITY ? 0.f : fast_exp2(m - base);
  float total = l * weight;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
  float acc[D / 32];
#pragma unroll
  for (int c = 0; c < D / 32; ++c) acc[c] = 0.f;
  for (int s = 0; s < args.splits; ++s) {
    const float w = __shfl_sync(0xffffffffu, weight, s);
    if (w == 0.f) continue;                           // its output row was never written
    const float* src = args.partial_o + (s * slice + token_head) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) acc[c] += src[c * 32 + lane] * w;
  }
  const float inv = total > 0.f ? 1.0f / total : 0.f;
  __nv_bfloat16* dst = args.out + token_head * D;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) dst[c * 32 + lane] = __float2bfloat16_rn(acc[c] * inv);
}

}  // namespace tcattn

SHRIKE_API int shrike_attention_tc_available() { return 1; }

// How many CTAs should share the keys of a query tile, for a batch of `num_tokens` new tokens whose
// block tables are `max_blocks` pages wide: as many as fill the GPU twice, each with at least four
// key tiles, at most 16; 1 when the query tiles alone fill it.  The scratch for splits > 1 is
// splits * num_tokens * num_heads * (D + 2) floats.
SHRIKE_API int shrike_attention_tc_portions_splits(int num_tokens, int num_heads, int max_blocks, int page_size) {
  const int ctas = num_heads * ((num_tokens + tcattn::BM - 1) / tcattn::BM + 1);
  const int key_tiles = (max_blocks * page_size + tcattn::BN - 1) / tcattn::BN;
  int splits = (2 * shrike_device().sm_count) / (ctas < 1 ? 1 : ctas);
  if (splits > key_tiles / 4) splits = key_tiles / 4;
  if (splits > 16) splits = 16;
  return splits < 1 ? 1 : splits;   // the kernels take up to 32
}
SHRIKE_API long long shrike_attention_tc_portions_scratch_floats(int num_tokens, int num_heads, int splits) {
  return splits <= 1 ? 0 : static_cast<long long>(splits) * num_tokens * num_heads * (tcattn::D + 2);
}

// Portions (q_len > 1) of a batch; entries with q_len == 1 are skipped when skip_single.
// q [tokens, heads * D] and out alike; caches [pages, page_size, kv heads, D]; page_size one of
// 8, 16, 32, 64.
SHRIKE_API int shrike_paged_attention_tc_portions(const void* q, const void* k_cache, const void* v_cache,
                                                  const int* block_table, int max_blocks, const int* q_start,
                                                  const int* ctx_len, int num_tokens, int num_seqs, int num_heads,
                                                  int num_kv_heads, int page_size, int num_pages, float scale,
                                                  int window, void* out, int skip_single, int max_q_len, int* status,
                                                  int splits, float* scratch, int portion_tiles, const int* seq_of_token,
                                                  cudaStream_t stream) {
  using namespace tcattn;
  if (num_seqs <= 0 || num_tokens <= 0) return SHRIKE_OK;
  if (splits < 1 || splits > 32 || (splits > 1 && (scratch == nullptr || seq_of_token == nullptr))) return SHRIKE_BAD_ARGUMENT;
  // query tiles of the batch's portions: the caller's count, or what `num_tokens` tokens in
  // `num_seqs` sequences can make at most
  const int most_tiles = (num_tokens + BM - 1) / BM + num_seqs;
  const int work = portion_tiles > 0 && portion_tiles < most_tiles ? portion_tiles : most_tiles;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || max_blocks <= 0 || max_q_len < 1 ||
      num_seqs > 65535 || (num_tokens + BM - 1) / BM + num_seqs > 65535 || !(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64))
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
  args.splits = splits;
  args.num_tokens = num_tokens;
  args.num_seqs = num_seqs;
  args.seq_of_token = seq_of_token;
  args.partial_o = splits > 1 ? scratch : nullptr;   // rows first (16-byte stores), then the (base, sum) pairs
  args.partial_ml = splits > 1 ? scratch + static_cast<long long>(splits) * num_tokens * num_heads * D : nullptr;
  cudaError_t err = launch_dependent(portions_tc_kernel, dim3(num_heads, work, splits), dim3(THREADS), SMEM_BYTES, stream,
                                     map_q, map_k, map_v, args);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (splits > 1) {
    err = launch_dependent(combine_portions_kernel, dim3(num_heads, (num_tokens + 7) / 8), dim3(256), 0, stream, args);
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  return shrike_launch_status();
}

#else  // other head sizes: the mma.sync kernel serves them

SHRIKE_API int shrike_attention_tc_available() { return 0; }
SHRIKE_API int shrike_attention_tc_portions_splits(int, int, int, int) { return 1; }
SHRIKE_API long long shrike_attention_tc_portions_scratch_floats(int, int, int) { return 0; }
SHRIKE_API int shrike_paged_attention_tc_portions(const void*, const void*, const void*, const int*, int, const int*,
                                                  const int*, int, int, int, int, int, int, float, int, void*, int, int,
                                                  int*, int, float*, int, const int*, cudaStream_t) {
  return SHRIKE_BAD_ARGUMENT;
}

#endif
