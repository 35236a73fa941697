// Paged causal attention for portions (q_len > 1) in bfloat16 on the fifth-generation
// tensor cores.  One CTA owns 256 query rows of one head of one sequence, as two chains of
// 128 rows; a chain walks the keys 64 at a time:
//   S = Q K^T       tcgen05.mma, M 128 x N 64 x K head size, into the chain's 64 score columns
//   softmax         four warps per chain, ONE THREAD PER QUERY ROW: the row of S comes out of
//                   tensor memory with tcgen05.ld, scale, mask, running maximum and sum in
//                   float32; the probabilities go back INTO tensor memory as packed bfloat16
//                   (tcgen05.st), into one of the chain's two probability buffers of 32 columns
//   O += P V        tcgen05.mma with its A operand in tensor memory, M 128 x N head size x K 64;
//                   O stays in tensor memory across steps and is rescaled there when a row's
//                   maximum moved by more than 2^8
// A chain's tensor memory is 64 (S) + 2 x 32 (P) + head size (O) columns; two chains fill the
// 512.  The scores of step h + 1 need only the keys and the score columns, and those are free
// as soon as the softmax threads hold step h in registers (s_read): they are computed while the
// softmax of step h runs, so a softmax thread finds its next scores waiting.  P(h) is written to
// the buffer P(h - 2) was in once PV(h - 2) has read it (pv_done), and O is rescaled only after
// PV(h - 1) (the same barrier, the other buffer).
// Both chains read the same key and value stages (two each, 128 keys a stage), so a tile is
// loaded once for 256 rows.  The later chain sees up to one key tile more than the earlier one;
// a chain without rows (a sequence's last 128 or fewer) has no steps.
// Keys and values arrive by TMA, one box per page and 64-element half of the head, the two
// query tiles by TMA once.  Handing a box to the copy engine costs the issuing warp about
// 50 ns, and a tile of 16-token pages is 16 boxes of keys and 16 of values: warp 0 brings the
// keys and warp 3 the values, each with the page ids of the next tiles fetched 32 at a time (a
// lookup per tile would stall the warp for a trip to L2 in every iteration).
// Roles: warp 0 keys (and the query tiles), warp 3 values (and the tensor-memory allocation),
// warp 1 / warp 2 one issuing thread for chain 0 / chain 1 (a single thread for both chains was
// the CTA's bottleneck), warps 4..7 softmax and epilogue of chain 0, warps 8..11 of chain 1.
// tcgen05.commit arrives on mbarriers: s_full[c] after S of chain c, pv_done[c][buffer] after a
// PV, k_free / v_free after a chain's last use of a stage (a stage is free when every chain that
// reads it has arrived), pv_last[c] after a chain's last PV.  A wait on pv_done cannot stand in
// for pv_last: a thread that has skipped phases cannot tell them apart by parity.
// Mask and window as everywhere: a query at position p sees keys [max(0, p - window + 1), p].
// Rows of a page beyond the context may hold anything (a page is reused without clearing):
// scores are masked by selection, and the value rows beyond the context are zeroed in shared
// memory before PV, because 0 * NaN would not be 0.
// The grid holds exactly the query tiles the batch's portions make (find_work).  Few query tiles
// and many keys (a portion of a long prompt beside decoding requests) would leave most of the GPU
// idle: the keys of a query tile are then split across `splits` CTAs, each of which leaves its
// unnormalised output rows with their (base, sum) in scratch, and a second small kernel adds the
// splits up (combine_portions_kernel).
// Earlier forms, each slower: one query tile per CTA with probabilities through shared memory; two
// chains with 128-key steps whose probabilities lay over the scores (the next scores could only be
// issued after PV, so the softmax threads waited for the tensor pipe and it for them); one chain of
// 128 rows with two threads per row (twice the key traffic and CTAs, and the two warps of a
// sub-partition in step with each other).
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
constexpr int BM = 128;                         // query rows of one chain
constexpr int HALVES = D / 64;                 // 64-element groups of the head size
constexpr int Q_HALF = BM * 128;               // bytes of one 64-element-wide sub-tile of a query tile
constexpr int Q_BYTES = HALVES * Q_HALF;
constexpr float LOG2E = 1.4426950408889634f;

enum : int { ERR_PRODUCER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_DRAIN = 14, ERR_ALIGNMENT = 15 };

// 2^x on the special-function unit; -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The softmax threads are short of issue slots, not of arithmetic: the maximum of three in one
// instruction, and multiply-add and add on pairs of floats (one instruction for two elements).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ unsigned long long pair_of(float lo, float hi) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void halves_of(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_pair(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_pair(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
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
// query tiles of `rows` rows, the last (longest to walk) first; sequences of one token own none when
// skip_single.  Every lane of the calling warp gets the answer; tile_start < 0: no such work.
__device__ __forceinline__ void find_work(const Args& args, int work, int rows, int& seq_out, int& tile_start_out) {
  const int lane = threadIdx.x & 31;
  int before = 0;
  seq_out = -1;
  tile_start_out = -1;
  for (int base = 0; base < args.num_seqs; base += 32) {
    const int s = base + lane;
    int tiles = 0;
    if (s < args.num_seqs) {
      const int q_len = args.q_start[s + 1] - args.q_start[s];
      tiles = (q_len == 1 && args.skip_single) ? 0 : (q_len + rows - 1) / rows;
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
      tile_start_out = (tiles_of_owner - 1 - (work - first_of_owner)) * rows;
      return;
    }
    before += __shfl_sync(0xffffffffu, inclusive, 31);
  }
}

namespace pair {
constexpr int ROWS = 2 * BM;                  // query rows per CTA
constexpr int KEYS = 128;                     // keys per step
constexpr int PSTAGES = 2;
constexpr int PTHREADS = 128 + 2 * 128;   // producer, two issuers, tensor-memory owner; four softmax warps per chain
constexpr int KV_TILE_HALF = KEYS * 128;      // bytes of one 64-element-wide sub-tile of a key (or value) tile
constexpr int KV_TILE = HALVES * KV_TILE_HALF;
constexpr int HALF_KEYS = KEYS / 2;           // keys per softmax step
constexpr unsigned CHAIN_COLS = 256;          // a chain's tensor memory: scores of one step (64 columns),
constexpr unsigned P_COL = 64;                // two probability buffers of 32 columns (bfloat16 pairs),
constexpr unsigned O_COL = 128;               // the output accumulator (head size columns)
constexpr unsigned PAIR_TMEM_COLS = 512;

struct PairShared {
  unsigned long long q_full, s_full[2], s_read[2], p_full[2][2], pv_done[2][2], pv_last[2], stagger;   // [chain]([P buffer])
  unsigned long long k_full[PSTAGES], k_free[PSTAGES], v_full[PSTAGES], v_free[PSTAGES];
  unsigned tmem_base;
  volatile int abort;
};
constexpr size_t PAIR_SMEM = 2 * Q_BYTES + PSTAGES * 2 * KV_TILE + sizeof(PairShared);

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (probabilities, bfloat16 packed two to a column, one
// row per lane) comes from tensor memory.
__device__ __forceinline__ void umma_a_in_tmem(unsigned tmem_d, unsigned tmem_a, unsigned long long b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}

// Rarely run parts of the softmax loop, kept out of line: the loop's body should stay small (its
// instructions are fetched again in every step).
__device__ __noinline__ void rescale_output_row(unsigned tmem_o, float correction) {
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    unsigned o[32];
    tmem_load32(tmem_o + c * 32, o);
    tmem_wait_load();
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * correction);
    tmem_store32(tmem_o + c * 32, o);
  }
}
// Zeroes the rows first_bad .. 127 of a value tile (128 threads share the work).
__device__ __noinline__ void zero_value_rows(unsigned char* v_tile, int first_bad, int row) {
  for (int idx = row; idx < (KEYS - first_bad) * HALVES * 8; idx += 128) {
    const int r = first_bad + idx / (HALVES * 8), rest = idx % (HALVES * 8);
    *reinterpret_cast<uint4*>(v_tile + (rest / 8) * KV_TILE_HALF + r * 128 + (rest % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_async_shared();
}

__global__ void __launch_bounds__(PTHREADS, 1)
portions_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const Args args) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int head = blockIdx.x, split = blockIdx.z;
  int seq, tile_start;
  find_work(args, blockIdx.y, ROWS, seq, tile_start);           // metadata: written before the step's kernels
  if (tile_start < 0 || (smem_u32(smem_raw) & 1023u)) {
    if (tile_start >= 0 && threadIdx.x == 0 && args.status != nullptr) *args.status = ERR_ALIGNMENT;
    let_dependents_start();
    wait_for_previous();
    return;
  }
  const int start = args.q_start[seq];
  const int q_len = args.q_start[seq + 1] - start;
  unsigned char* q_tiles = smem_raw;                             // [2 chains][Q_BYTES]
  unsigned char* k_tiles = q_tiles + 2 * Q_BYTES;                // [PSTAGES][KV_TILE]
  unsigned char* v_tiles = k_tiles + PSTAGES * KV_TILE;          // [PSTAGES][KV_TILE]
  PairShared* sh = reinterpret_cast<PairShared*>(v_tiles + PSTAGES * KV_TILE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // (lengths and positions are step metadata, written before the step's kernels: readable before the wait below)
  const int pos0 = args.ctx_len[seq] - q_len;                   // position of the first new token
  const int kv_head = head / (args.num_heads / args.num_kv_heads);
  // chain c owns rows tile_start + 128 c ...; rows_c <= 0: the chain has none
  const int rows_0 = min(BM, q_len - tile_start), rows_1 = min(BM, q_len - tile_start - BM);
  const int lo = args.window > 0 ? max(0, pos0 + tile_start - args.window + 1) : 0;   // first key any row sees
  const int hi_0 = pos0 + tile_start + rows_0 - 1;              // last key chain 0 sees
  const int hi_1 = rows_1 > 0 ? hi_0 + rows_1 : -1;
  const int hi = max(hi_0, hi_1);
  const int tile_hi = hi / KEYS;
  const int all_tiles = tile_hi - lo / KEYS + 1;
  const int per = (all_tiles + args.splits - 1) / args.splits;
  const int tile_lo = lo / KEYS + split * per;                  // this CTA's share: tiles tile_lo ... (none: an empty split)
  const int last_tile = min(tile_hi, tile_lo + per - 1);
  const int count_0 = max(0, min(last_tile, hi_0 / KEYS) - tile_lo + 1);
  const int count_1 = rows_1 > 0 ? max(0, min(last_tile, hi_1 / KEYS) - tile_lo + 1) : 0;
  const int num_tiles = max(count_0, count_1);
  // the same in steps of 64 keys: a chain's last tile may need its first half only
  const int steps_0 = count_0 > 0 ? min(2 * count_0, hi_0 / HALF_KEYS - 2 * tile_lo + 1) : 0;
  const int steps_1 = count_1 > 0 ? min(2 * count_1, hi_1 / HALF_KEYS - 2 * tile_lo + 1) : 0;

  const unsigned users = (steps_0 > 0 ? 1u : 0u) + (steps_1 > 0 ? 1u : 0u);   // chains that read the key and value stages
  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    for (int c = 0; c < 2; ++c) {
      mbar_init(&sh->s_full[c], 1);
      mbar_init(&sh->s_read[c], 128);
      for (int b = 0; b < 2; ++b) {
        mbar_init(&sh->p_full[c][b], 128);
        mbar_init(&sh->pv_done[c][b], 1);
      }
      mbar_init(&sh->pv_last[c], 1);
    }
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_free[s], users > 0 ? users : 1u);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->v_free[s], users > 0 ? users : 1u);
    }
    mbar_init(&sh->stagger, 1);
    sh->abort = 0;
    mbar_init_fence();
  }
  if (warp == 3) tmem_alloc(&sh->tmem_base, PAIR_TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  let_dependents_start();
  wait_for_previous();   // the query and the newest keys come from the kernel before this one

  if (warp == 0 || warp == 3) {
    // Warp 0 brings the query tiles and the keys, warp 3 the values: lane 0 waits for the stage and arms
    // its barrier, then lane pg issues the boxes of page pg of the tile (every 64-element half).  Handing
    // a box to the copy engine costs the issuing warp about 50 ns, and a tile of 16-token pages is 16
    // boxes of keys and 16 of values: one warp for both would need longer per tile than the tensor
    // pipe does.
    const bool for_keys = warp == 0;
    const int* table = args.block_table + static_cast<size_t>(seq) * args.max_blocks;
    const int pages_per_tile = KEYS / args.page_size;
    const int nowhere = args.num_pages * args.page_size;      // a row coordinate outside the cache: reads zeros
    if (for_keys && lane == 0 && num_tiles > 0) {
      mbar_expect_tx(&sh->q_full, 2 * Q_BYTES);
      for (int c = 0; c < 2; ++c)
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(q_tiles + c * Q_BYTES + h * Q_HALF, &map_q, &sh->q_full, head * D + h * 64, start + tile_start + c * BM);
    }
    // Page ids come a chunk of 32 at a time (lane l: page l of the chunk, several tiles' worth), the
    // next chunk while this one is used: a lookup per tile would stall the warp for a trip to L2 in
    // every iteration.
    const int tiles_per_chunk = 32 / pages_per_tile;
    auto load_chunk = [&](int chunk) -> int {
      const int key0 = tile_lo * KEYS + (chunk * 32 + lane) * args.page_size;
      const int block = key0 / args.page_size;
      return (chunk * tiles_per_chunk < num_tiles && key0 <= hi && block < args.max_blocks) ? table[block] : -1;
    };
    unsigned char* const tiles = for_keys ? k_tiles : v_tiles;
    unsigned long long* const full = for_keys ? sh->k_full : sh->v_full;
    unsigned long long* const free_again = for_keys ? sh->k_free : sh->v_free;
    const CUtensorMap* const map = for_keys ? &map_k : &map_v;
    int chunk_pages = load_chunk(0), next_pages = load_chunk(1);
    int issued = 0;
    for (int i = 0; i < num_tiles; ++i) {
      const int s = i % PSTAGES;
      const unsigned phase = (i / PSTAGES) & 1;
      const int within = i % tiles_per_chunk;
      if (within == 0 && i > 0) {
        chunk_pages = next_pages;
        next_pages = load_chunk(i / tiles_per_chunk + 1);
      }
      int page = __shfl_sync(0xffffffffu, chunk_pages, within * pages_per_tile + (lane % pages_per_tile));
      if (page >= args.num_pages) page = -1;
      unsigned char* tile = tiles + s * KV_TILE;
      const int y = page < 0 ? nowhere : page * args.page_size;
      const int at = lane * args.page_size * 128;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(&free_again[s], phase ^ 1, &sh->abort, args.status, ERR_PRODUCER) ? 1 : 0;
        if (ok) mbar_expect_tx(&full[s], KV_TILE);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile)
        for (int h = 0; h < HALVES; ++h) tma_load_2d(tile + h * KV_TILE_HALF + at, map, &full[s], kv_head * D + h * 64, y);
      issued = i + 1;
    }
    if (lane == 0 && sh->abort) {   // copies may still be in flight: wait for the stages armed last
      for (int i = max(0, issued - PSTAGES); i < issued; ++i) {
        bool landed = false;
        for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries) landed = mbar_try_wait(&full[i % PSTAGES], (i / PSTAGES) & 1);
        if (!landed && args.status != nullptr) *args.status = ERR_DRAIN;
      }
      bool landed = !for_keys || num_tiles <= 0;
      for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries) landed = mbar_try_wait(&sh->q_full, 0);
    }
  } else if (warp == 1 || warp == 2) {
    // One issuing thread per chain.  The scores of step h + 1 need nothing but the keys and the
    // chain's score columns, which are free as soon as the softmax threads hold step h in registers
    // (s_read); the probabilities have columns of their own, two buffers of them.  So the thread
    // follows the chain's events in the order they come: s_read(h) -> S(h + 1), p_full(h) -> PV(h).
    const int c = warp - 1;
    const int steps = c == 0 ? steps_0 : steps_1;
    if (lane == 0 && steps > 0) {
      const unsigned idesc_s = instruction_descriptor(BM, HALF_KEYS, false);
      const unsigned idesc_o = instruction_descriptor(BM, D, true);
      const unsigned tmem_chain = sh->tmem_base + c * CHAIN_COLS, tmem_o = tmem_chain + O_COL;
      // operand descriptors are formed once (a descriptor's low bits are the address in 16-byte
      // units, so a tile further on is an addition), not per instruction
      const unsigned long long q_base = smem_descriptor(smem_u32(q_tiles + c * Q_BYTES));
      const unsigned long long k_desc0 = smem_descriptor(smem_u32(k_tiles));
      const unsigned long long v_desc0 = smem_descriptor(smem_u32(v_tiles), KV_TILE_HALF, 1024);
      bool ok = mbar_wait(&sh->q_full, 0, &sh->abort, args.status, ERR_MMA);
      int keys_ready = -1, values_ready = -1;   // the newest tile whose keys (values) are known to have landed
      // S for step h (keys 64 h ... of this CTA's share); the chain's last use of a stage hands it back
      // (the stage is free when every chain that uses it has)
      auto issue_scores = [&](int h) {
        const int i = h >> 1, st = i % PSTAGES;
        if (keys_ready < i) {
          ok = mbar_wait(&sh->k_full[st], (i / PSTAGES) & 1, &sh->abort, args.status, ERR_MMA);
          if (!ok) return;
          keys_ready = i;
        }
        fence_after_sync();
        const unsigned long long k_base = k_desc0 + static_cast<unsigned>((st * KV_TILE + (h & 1) * HALF_KEYS * 128) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem_chain, q_base + (((kk / 4) * Q_HALF + (kk % 4) * 32) >> 4), k_base + (((kk / 4) * KV_TILE_HALF + (kk % 4) * 32) >> 4), idesc_s,
               kk > 0 ? 1u : 0u);
        umma_commit(&sh->s_full[c]);
        if ((h & 1) || h + 1 == steps) umma_commit(&sh->k_free[st]);
      };
      // The two chains' softmax warps share the sub-partitions; started together they stay in step and
      // do their arithmetic at the same time and their waiting at the same time.  The later chain
      // starts when the earlier one has written its first probabilities: most of a step behind.
      if (ok && c == 1 && steps_0 > 0) ok = mbar_wait(&sh->stagger, 0, &sh->abort, args.status, ERR_MMA);
      if (ok) issue_scores(0);
      for (int h = 0; h < steps && ok; ++h) {
        if (h + 1 < steps) {
          ok = mbar_wait(&sh->s_read[c], h & 1, &sh->abort, args.status, ERR_MMA);
          if (!ok) break;
          issue_scores(h + 1);
          if (!ok) break;
        }
        const int i = h >> 1, st = i % PSTAGES;
        if (values_ready < i) {
          ok = mbar_wait(&sh->v_full[st], (i / PSTAGES) & 1, &sh->abort, args.status, ERR_MMA);
          values_ready = i;
        }
        if (ok) ok = mbar_wait(&sh->p_full[c][h & 1], (h >> 1) & 1, &sh->abort, args.status, ERR_MMA);
        if (!ok) break;
        if (c == 0 && h == 0) mbar_arrive(&sh->stagger);   // on every path: the other issuer waits for it
        fence_after_sync();
        const unsigned long long v_base = v_desc0 + static_cast<unsigned>((st * KV_TILE + (h & 1) * HALF_KEYS * 128) >> 4);
        const unsigned tmem_p = tmem_chain + P_COL + (h & 1) * 32;
#pragma unroll
        for (int kk = 0; kk < HALF_KEYS / 16; ++kk)   // 16 keys an instruction: 8 packed columns of P, 16 rows of V
          umma_a_in_tmem(tmem_o, tmem_p + kk * 8, v_base + ((kk * 16 * 128) >> 4), idesc_o, (h > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh->pv_done[c][h & 1]);
        if (h + 1 == steps) umma_commit(&sh->pv_last[c]);
        if ((h & 1) || h + 1 == steps) umma_commit(&sh->v_free[st]);
      }
    }
  } else if (warp >= 4) {
    const int chain = (warp - 4) >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int t = tile_start + chain * BM + row;
    const int my_steps = chain == 0 ? steps_0 : steps_1;
    const int last = t < q_len ? pos0 + t : -1;
    const int first = args.window > 0 ? max(0, last - args.window + 1) : 0;
    const unsigned lane_base = static_cast<unsigned>(quarter * 32) << 16;
    const unsigned tmem_chain = sh->tmem_base + chain * CHAIN_COLS + lane_base, tmem_o = tmem_chain + O_COL;
    float row_max = -INFINITY, row_sum = 0.f;
    bool ok = true;
    for (int h = 0; h < my_steps && ok; ++h) {
      ok = mbar_wait(&sh->s_full[chain], h & 1, &sh->abort, args.status, ERR_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);   // the warp stays together: the tensor-memory accesses below are warp-wide
      if (!ok) break;
      fence_after_sync();
      unsigned v[2][32];
      tmem_load32(tmem_chain, v[0]);
      tmem_load32(tmem_chain + 32, v[1]);
      tmem_wait_load();
      fence_before_sync();
      mbar_arrive(&sh->s_read[chain]);    // the scores are in registers: their columns may take the next step
      const int key_base = tile_lo * KEYS + h * HALF_KEYS;
      if (key_base < first || key_base + HALF_KEYS - 1 > last) {   // only steps at the edge of the row's range pay for masking
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key_base + g * 32 + j;
            if (key < first || key > last) v[g][j] = 0xff800000u;   // -inf
          }
      }
      float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains of dependent instructions, not one
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int j = 0; j < 32; j += 8)
#pragma unroll
          for (int a = 0; a < 4; ++a) part_max[a] = max3(part_max[a], __uint_as_float(v[g][j + 2 * a]), __uint_as_float(v[g][j + 2 * a + 1]));
      float step_max = fmaxf(max3(part_max[0], part_max[1], part_max[2]), part_max[3]);
      step_max *= args.scale_log2;
      // The base of the exponentials follows the running maximum lazily: it moves (and O is
      // rescaled) only when the maximum has grown by more than 2^8; until then probabilities
      // are at most 2^8, which float32 sums and bfloat16 products hold without loss.
      float correction = 1.0f;
      if (step_max > row_max + 8.0f || row_max == -INFINITY) {
        const float new_max = fmaxf(row_max, step_max);
        const float base = new_max == -INFINITY ? 0.f : new_max;
        // a row that has seen no key yet has O = 0 and a sum of 0: nothing to rescale
        correction = row_max == -INFINITY ? 1.0f : fast_exp2(row_max - base);
        row_max = new_max;
      }
      const float base = row_max == -INFINITY ? 0.f : row_max;
      const unsigned long long scale_pair = pair_of(args.scale_log2, args.scale_log2), base_pair = pair_of(-base, -base);
      unsigned long long sum_pair[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
#pragma unroll
      for (int g = 0; g < 2; ++g) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float x0, x1;
          halves_of(fma_pair(pair_of(__uint_as_float(v[g][j]), __uint_as_float(v[g][j + 1])), scale_pair, base_pair), x0, x1);
          x0 = fast_exp2(x0);
          x1 = fast_exp2(x1);
          sum_pair[(j >> 1) & 1] = add_pair(sum_pair[(j >> 1) & 1], pair_of(x0, x1));
          const __nv_bfloat162 two = __floats2bfloat162_rn(x0, x1);
          v[0][g * 16 + j / 2] = *reinterpret_cast<const unsigned*>(&two);   // packed over the scores already used
        }
      }
      float sum_lo, sum_hi;
      halves_of(add_pair(sum_pair[0], sum_pair[1]), sum_lo, sum_hi);
      row_sum = row_sum * correction + (sum_lo + sum_hi);
      // P(h) goes where P(h - 2) was: the PV of step h - 2 must have read it (it has, long ago)
      if (h >= 2) {
        ok = mbar_wait(&sh->pv_done[chain][h & 1], ((h >> 1) & 1) ^ 1, &sh->abort, args.status, ERR_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after_sync();
      }
      tmem_store32(tmem_chain + P_COL + (h & 1) * 32, v[0]);   // keys 2 j and 2 j + 1 of the step in column j
      // value rows beyond the context: zero them (only the tile that holds the sequence's last key has
      // any), at the tile's first step, before either of its PV
      if ((h & 1) == 0 && tile_lo + (h >> 1) == tile_hi && (hi + 1) % KEYS != 0) {
        const int s = (h >> 1) % PSTAGES;
        ok = mbar_wait(&sh->v_full[s], ((h >> 1) / PSTAGES) & 1, &sh->abort, args.status, ERR_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        zero_value_rows(v_tiles + s * KV_TILE, hi + 1 - key_base, row);
      }
      if (h > 0 && __any_sync(0xffffffffu, correction != 1.0f)) {
        // O still takes the step before: wait for its PV, then rescale
        ok = mbar_wait(&sh->pv_done[chain][(h - 1) & 1], ((h - 1) >> 1) & 1, &sh->abort, args.status, ERR_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after_sync();
        rescale_output_row(tmem_o, correction);
      }
      tmem_wait_store();
      fence_before_sync();
      mbar_arrive(&sh->p_full[chain][h & 1]);
    }
    const int my_count = my_steps;
    if (ok && my_steps > 0) ok = mbar_wait(&sh->pv_last[chain], 0, &sh->abort, args.status, ERR_SOFTMAX);
    ok = __all_sync(0xffffffffu, ok);
    fence_after_sync();
    if (ok && args.splits > 1) {
      const size_t at = (static_cast<size_t>(split) * args.num_tokens + start + t) * args.num_heads + head;
      if (t < q_len) {
        args.partial_ml[2 * at] = my_count > 0 ? row_max : -INFINITY;
        args.partial_ml[2 * at + 1] = my_count > 0 ? row_sum : 0.f;
      }
      if (my_count > 0) {
        float* dst = args.partial_o + at * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          unsigned o[32];
          tmem_load32(tmem_o + c * 32, o);
          tmem_wait_load();
          if (t < q_len) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(o[j], o[j + 1], o[j + 2], o[j + 3]);
          }
        }
      }
    } else if (ok && my_count > 0) {
      const float inv = row_sum > 0.f ? 1.0f / row_sum : 0.f;
      __nv_bfloat16* dst = args.out + (static_cast<size_t>(start + t) * args.num_heads + head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        unsigned o[32];
        tmem_load32(tmem_o + c * 32, o);
        tmem_wait_load();
        if (t < q_len) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            unsigned packed[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(o[j + 2 * e]) * inv, __uint_as_float(o[j + 2 * e + 1]) * inv);
              packed[e] = *reinterpret_cast<const unsigned*>(&two);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 3) {
    fence_after_sync();
    tmem_free(sh->tmem_base, PAIR_TMEM_COLS);
  }
}

}  // namespace pair

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

// Query rows a CTA owns: what the caller counts the portions' query tiles in.
SHRIKE_API int shrike_attention_tc_portions_rows() { return tcattn::pair::ROWS; }

// How many CTAs should share the keys of a query tile, for a batch of `num_tokens` new tokens whose
// portions make `portion_tiles` query tiles (0: not known; the most they can make is assumed) and whose
// block tables are `max_blocks` pages wide.  The GPU holds one CTA per SM.  Splitting pays only while
// every CTA still starts at once (measured: 512 new tokens of 28 heads over 7,680 cached take 156 us
// unsplit, 97 with two splits, which make 112 CTAs, and 124 with three, which need a second round; a
// whole prompt, whose query tiles outnumber the SMs, is best left alone at every length).  Among the
// split counts that keep the launch to one round, with at least two key steps per split and at most
// 16, the one with the fewest steps per CTA, counting three steps' worth for a CTA's start and three
// more for the second kernel that adds the splits up.  The scratch for s > 1 is
// s * num_tokens * num_heads * (D + 2) floats.
SHRIKE_API int shrike_attention_tc_portions_splits(int num_tokens, int num_heads, int max_blocks, int page_size, int portion_tiles) {
  const int rows = shrike_attention_tc_portions_rows();
  const int most = (num_tokens + rows - 1) / rows + 1;
  const int tiles = portion_tiles > 0 && portion_tiles < most ? portion_tiles : most;
  const long long ctas = static_cast<long long>(num_heads) * tiles;
  const int keys = tcattn::pair::KEYS;
  const int key_steps = (max_blocks * page_size + keys - 1) / keys;
  const long long capacity = shrike_device().sm_count;   // one CTA per SM
  int best = 1;
  long long best_cost = -1;
  for (int s = 1; s <= 16 && (s == 1 || (key_steps / s >= 2 && ctas * s <= capacity)); ++s) {
    const long long cost = (key_steps + s - 1) / s + 3 + (s > 1 ? 3 : 0);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;   // the kernels take up to 32
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
  const int rows = shrike_attention_tc_portions_rows();
  const int most_tiles = (num_tokens + rows - 1) / rows + num_seqs;
  const int work = portion_tiles > 0 && portion_tiles < most_tiles ? portion_tiles : most_tiles;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || max_blocks <= 0 || max_q_len < 1 ||
      num_seqs > 65535 || (num_tokens + BM - 1) / BM + num_seqs > 65535 || !(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64))
    return SHRIKE_BAD_ARGUMENT;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(pair::portions_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(pair::PAIR_SMEM));
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
  cudaError_t err = launch_dependent(pair::portions_pair_kernel, dim3(num_heads, work, splits), dim3(pair::PTHREADS), pair::PAIR_SMEM,
                                     stream, map_q, map_k, map_v, args);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (splits > 1) {
    err = launch_dependent(combine_portions_kernel, dim3(num_heads, (num_tokens + 7) / 8), dim3(256), 0, stream, args);
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  return shrike_launch_status();
}

#else  // other head sizes: the mma.sync kernel serves them

SHRIKE_API int shrike_attention_tc_available() { return 0; }
SHRIKE_API int shrike_attention_tc_portions_rows() { return 128; }
SHRIKE_API int shrike_attention_tc_portions_splits(int, int, int, int, int) { return 1; }
SHRIKE_API long long shrike_attention_tc_portions_scratch_floats(int, int, int) { return 0; }
SHRIKE_API int shrike_paged_attention_tc_portions(const void*, const void*, const void*, const int*, int, const int*,
                                                  const int*, int, int, int, int, int, int, float, int, void*, int, int,
                                                  int*, int, float*, int, const int*, cudaStream_t) {
  return SHRIKE_BAD_ARGUMENT;
}

#endif
