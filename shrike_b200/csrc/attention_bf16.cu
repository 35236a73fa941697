// Paged grouped-query attention in bfloat16 on the tensor cores (mma.sync m16n8k16,
// float32 accumulation), for the serving path.
//
// Two kernels share the tile code:
//   * portions (q_len > 1): one CTA per (64 queries, query head, sequence); four warps
//     own 16 query rows each and walk the keys 64 at a time (FlashAttention-2 order).
//   * single tokens (q_len == 1): one CTA per (key split, kv head, sequence).  The G
//     query heads that share a kv head are the rows of one 16-row tile, so keys and
//     values are read once per kv head, not once per query head; eight warps take 8 keys
//     each of every 64-key tile for Q K^T and every eighth 16-column block of the output for
//     P V (the probabilities pass through shared memory), tiles arrive through a three-deep
//     cp.async pipeline;
//     the splits of one kv head form thread-block clusters of up to eight CTAs, which add
//     their partial results up through distributed shared memory; where one cluster covers
//     all splits the result goes straight out, otherwise each cluster writes one partial
//     and the CTA that finishes last (an atomic counter per kv head, which it resets)
//     combines them.  Split and cluster counts are launch parameters, the key ranges come
//     from ctx_len on the device, so a captured launch sequence stays valid as contexts grow.
// Keys and values are fetched through the block table with 16-byte cp.async copies into
// padded shared-memory rows (double-buffered) and read with ldmatrix.  Scores, running
// maximum, sum and the output accumulate in float32; probabilities are rounded to
// bfloat16 for the PV product, as the values are.  Mask: a query at position p sees keys
// [max(0, p - window + 1), p] (shrike/engine/model_runner.py:129-150).
//
// Built once per head size: -DSHRIKE_HEAD_DIM=<multiple of 16, at most 256>.
#include <cooperative_groups.h>

#include "blackwell.cuh"
#include "common.cuh"

#ifndef SHRIKE_HEAD_DIM
#error "compile with -DSHRIKE_HEAD_DIM=<head size>"
#endif

namespace bf16attn {

constexpr int D = SHRIKE_HEAD_DIM;
constexpr int BN = 64;              // keys per tile, single tokens
constexpr int PBN = 32;             // keys per tile, portions: small tiles and few registers, so that four CTAs fit an SM
constexpr int BM = 64;              // query rows per CTA (portions)
constexpr int THREADS = 128;
constexpr int ROW = D + 8;          // padded row, in elements: 16 bytes of padding keep ldmatrix conflict-free
constexpr int CHUNKS = D / 8;       // 16-byte chunks per row
constexpr int KSTEPS = D / 16;
constexpr int DTILES = D / 8;
constexpr bool Q_IN_REGS = D <= 128;   // single tokens keep the query fragments in registers
constexpr float LOG2E = 1.4426950408889634f;
using bf16 = __nv_bfloat16;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void* smem) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

struct Params {
  const bf16* q;
  const bf16* k_cache;
  const bf16* v_cache;
  const int* block_table;
  const int* q_start;
  const int* ctx_len;
  bf16* out;
  float* partial_out;   // [seq, head, splits / cluster, D], single tokens only
  float* partial_ml;    // [seq, head, splits / cluster, 2]
  int* arrivals;        // [seq, kv head * row tiles]: CTAs that have stored their share; zero between launches
  int max_blocks, num_heads, num_kv_heads, page_size, num_pages, window, splits;
  int page_shift;       // log2(page_size) when that is a power of two, else -1: shifts instead of divisions
  int cluster;          // single tokens: consecutive splits that form one thread-block cluster
  int* status;          // host-visible; a wait that ran out leaves ERR_TILE_WAIT here
  int skip_single;      // portions kernel: leave q_len == 1 to the single-token kernel
  float scale_log2;     // scale * log2(e)
};

// Where the keys [tile_base, tile_base + BN) of one kv head start in the cache, in
// elements; -1 for keys outside [lo, hi] or on a page the sequence does not hold.  One
// table lookup and one division per key, done by the first BN threads.
// `leave_out` (or -1): a key whose row is marked -2, which copy_tile does not touch at all.
// In two steps, so that a caller can issue the table lookup one round before it needs the
// row: the page of key j (-1: none, -2: leave the row untouched), then the row's offset.
__device__ __forceinline__ int lookup_page(const Params& p, const int* table, int j, int lo, int hi, int leave_out) {
  if (j == leave_out) return -2;
  if (j < lo || j > hi) return -1;
  const int block = p.page_shift >= 0 ? j >> p.page_shift : j / p.page_size;
  return block < p.max_blocks ? table[block] : -1;
}
__device__ __forceinline__ long long row_of(const Params& p, int kv_head, int j, int page) {
  if (page == -2) return -2;
  if (page < 0 || page >= p.num_pages) return -1;
  const int within = p.page_shift >= 0 ? j & (p.page_size - 1) : j % p.page_size;
  return (static_cast<long long>(page) * p.page_size + within) * p.num_kv_heads * D + static_cast<long long>(kv_head) * D;
}
template <int KEYS>
__device__ __forceinline__ void locate_tile(long long* rows, const Params& p, const int* table, int kv_head,
                                            int tile_base, int lo, int hi, int leave_out = -1) {
  if (threadIdx.x < KEYS) {
    const int j = tile_base + threadIdx.x;
    rows[threadIdx.x] = row_of(p, kv_head, j, lookup_page(p, table, j, lo, hi, leave_out));
  }
}

// Copies the located keys and values into k_tile / v_tile; consecutive threads take
// consecutive 16-byte chunks of a row, so a warp's copies cover whole 128-byte lines.
// Keys without a row become zeros.
template <int KEYS, int NTHREADS>
__device__ __forceinline__ void copy_tile(bf16* k_tile, bf16* v_tile, const Params& p, const long long* rows) {
  constexpr int ROUNDS = (KEYS * CHUNKS + NTHREADS - 1) / NTHREADS;
  long long row[ROUNDS];
#pragma unroll
  for (int i = 0; i < ROUNDS; ++i) {   // every row offset first: the copies then go out back to back
    const int c = threadIdx.x + i * NTHREADS;
    row[i] = c < KEYS * CHUNKS ? rows[c / CHUNKS] : -2;
  }
#pragma unroll
  for (int i = 0; i < ROUNDS; ++i) {
    const int c = threadIdx.x + i * NTHREADS;
    const int key = c / CHUNKS, chunk = c - key * CHUNKS;
    if (row[i] == -2) continue;
    const bool valid = row[i] >= 0;
    const size_t offset = valid ? static_cast<size_t>(row[i]) + chunk * 8 : 0;
    cp_async16(k_tile + key * ROW + chunk * 8, p.k_cache + offset, valid);
    cp_async16(v_tile + key * ROW + chunk * 8, p.v_cache + offset, valid);
  }
}

// Both steps at once, with a barrier between them (for code that loads one tile ahead).
template <int KEYS>
__device__ __forceinline__ void load_kv_tile(bf16* k_tile, bf16* v_tile, long long* rows, const Params& p,
                                             const int* table, int kv_head, int tile_base, int lo, int hi) {
  locate_tile<KEYS>(rows, p, table, kv_head, tile_base, lo, hi);
  __syncthreads();
  copy_tile<KEYS, THREADS>(k_tile, v_tile, p, rows);
}

// S[16 x (8 * NT)] += Q[16 x D] * K^T for keys [key0, key0 + 8 * NT) of the tile.
template <int NT, bool IN_REGS>
__device__ __forceinline__ void scores(float (&s)[NT][4], const unsigned (&q_frag)[IN_REGS ? KSTEPS : 1][4],
                                       const bf16* q_rows, const bf16* k_tile, int key0, int lane) {
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    unsigned a[4];
    if (IN_REGS) {
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = q_frag[IN_REGS ? kk : 0][i];
    } else {
      ldmatrix_x4(a, q_rows + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + kk * 16 + 8 * (lane >> 4));
    }
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      unsigned b[4];
      const int key = key0 + np * 16 + (lane & 7) + 8 * (lane >> 4);
      ldmatrix_x4(b, k_tile + key * ROW + kk * 16 + 8 * ((lane >> 3) & 1));
      mma_bf16(s[2 * np], a, b[0], b[1]);
      mma_bf16(s[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x (8 * NT)] * V for keys [key0, key0 + 8 * NT) of the tile.
template <int NT>
__device__ __forceinline__ void accumulate(float (&o)[DTILES][4], const float (&s)[NT][4], const bf16* v_tile,
                                           int key0, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < DTILES / 2; ++dp) {
      unsigned b[4];
      const int key = key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
      ldmatrix_x4_trans(b, v_tile + key * ROW + dp * 16 + 8 * (lane >> 4));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Masks, scales and folds one block of scores into the running softmax state of the two
// rows this thread holds (row lane/4 and that + 8); leaves probabilities in s.
template <int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&o)[DTILES][4], float (&row_max)[2],
                                               float (&row_sum)[2], const int (&first)[2], const int (&last)[2],
                                               int key_base, float scale_log2, int lane) {
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key_base + j * 8 + (lane & 3) * 2 + (e & 1);
      const int r = e >> 1;
      const bool seen = key >= first[r] && key <= last[r];
      s[j][e] = seen ? s[j][e] * scale_log2 : -INFINITY;
      tile_max[r] = fmaxf(tile_max[r], s[j][e]);
    }
  float correction[2], base[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
    const float new_max = fmaxf(row_max[r], tile_max[r]);
    base[r] = new_max == -INFINITY ? 0.f : new_max;   // a row that has seen no key yet
    correction[r] = exp2f(row_max[r] - base[r]);      // exp2(-inf) = 0
    row_max[r] = new_max;
    row_sum[r] *= correction[r];
  }
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float prob = exp2f(s[j][e] - base[e >> 1]);
      s[j][e] = prob;
      row_sum[e >> 1] += prob;
    }
#pragma unroll
  for (int j = 0; j < DTILES; ++j) {
    o[j][0] *= correction[0];
    o[j][1] *= correction[0];
    o[j][2] *= correction[1];
    o[j][3] *= correction[1];
  }
}

// ------------------------------------------------------------------ portions
__global__ void __launch_bounds__(THREADS, D <= 128 ? 4 : 2) portions_kernel(const Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);           // [BM][ROW]
  bf16* k_tiles = q_tile + BM * ROW;                          // [2][PBN][ROW]
  bf16* v_tiles = k_tiles + 2 * PBN * ROW;                    // [2][PBN][ROW]
  __shared__ long long tile_rows[2][PBN];
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int tile_start = (gridDim.x - 1 - blockIdx.x) * BM;   // long tiles are scheduled first
  const int start = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - start;
  if (tile_start >= q_len || (q_len == 1 && p.skip_single)) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos0 = p.ctx_len[seq] - q_len;                    // position of the first new token
  const int kv_head = head / (p.num_heads / p.num_kv_heads);
  const int* table = p.block_table + static_cast<size_t>(seq) * p.max_blocks;
  const int rows_here = min(BM, q_len - tile_start);
  const int lo = p.window > 0 ? max(0, pos0 + tile_start - p.window + 1) : 0;
  const int hi = pos0 + tile_start + rows_here - 1;
  const int tile_lo = lo / PBN, tile_hi = hi / PBN;

  for (int c = threadIdx.x; c < BM * CHUNKS; c += THREADS) {
    const int row = c / CHUNKS, chunk = c - row * CHUNKS;
    const bool valid = row < rows_here;
    const bf16* src = p.q + (static_cast<size_t>(start + tile_start + (valid ? row : 0)) * p.num_heads + head) * D + chunk * 8;
    cp_async16(q_tile + row * ROW + chunk * 8, src, valid);
  }
  load_kv_tile<PBN>(k_tiles, v_tiles, tile_rows[0], p, table, kv_head, tile_lo * PBN, lo, hi);
  cp_async_commit();

  int first[2], last[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = tile_start + warp * 16 + (lane >> 2) + 8 * r;
    last[r] = t < q_len ? pos0 + t : -1;
    first[r] = p.window > 0 ? max(0, last[r] - p.window + 1) : 0;
  }
  float o[DTILES][4];
#pragma unroll
  for (int j = 0; j < DTILES; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  unsigned q_frag[1][4];   // query fragments are re-read from shared memory: registers are the scarcer resource here
  const bf16* q_rows = q_tile + warp * 16 * ROW;

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int buffer = (tile - tile_lo) & 1;
    if (tile < tile_hi) {
      load_kv_tile<PBN>(k_tiles + (buffer ^ 1) * PBN * ROW, v_tiles + (buffer ^ 1) * PBN * ROW, tile_rows[buffer ^ 1], p,
                        table, kv_head, (tile + 1) * PBN, lo, hi);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // a warp whose rows all end before this tile has nothing to add
    const int warp_last = pos0 + min(q_len, tile_start + warp * 16 + 16) - 1;
    const bool warp_active = tile_start + warp * 16 < q_len && tile * PBN <= warp_last;
    if (warp_active) {
      float s[PBN / 8][4];
#pragma unroll
      for (int j = 0; j < PBN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
      const bf16* k_tile = k_tiles + buffer * PBN * ROW;
      const bf16* v_tile = v_tiles + buffer * PBN * ROW;
      scores<PBN / 8, false>(s, q_frag, q_rows, k_tile, 0, lane);
      softmax_update<PBN / 8>(s, o, row_max, row_sum, first, last, tile * PBN, p.scale_log2, lane);
      accumulate<PBN / 8>(o, s, v_tile, 0, lane);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = tile_start + warp * 16 + (lane >> 2) + 8 * r;
    if (t >= q_len) continue;
    const float inv = row_sum[r] > 0.f ? 1.0f / row_sum[r] : 0.f;
    bf16* dst = p.out + (static_cast<size_t>(start + t) * p.num_heads + head) * D + (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < DTILES; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
  }
}

// ------------------------------------------------------------- single tokens
constexpr int ST = 3;  // pipeline depth of the single-token kernel, in 64-key tiles
constexpr int MAX_SPLITS = 32;
constexpr int SW = 8;                      // warps: each takes BN / SW keys of a tile for the scores ...
constexpr int STHREADS = SW * 32;
constexpr int WARP_KEYS = BN / SW;         // ... (8: one MMA column block)
constexpr int DPAIRS = D / 16;             // ... and every SW-th 16-column block of the output for PV
constexpr int MY_PAIRS = (DPAIRS + SW - 1) / SW;
constexpr int PROW = BN + 8;               // padded row of the probability tile, in elements
constexpr size_t SINGLE_EXCHANGE_SMEM = sizeof(bf16) * 16 * PROW + sizeof(float) * 2 * SW * 16;
// The probabilities and the warps' maxima and sums take the query tile's space once the query
// sits in registers, where that space suffices (two CTAs of head size 128 fill an SM's shared
// memory to the last kilobyte); otherwise they lie behind the key and value tiles.
constexpr bool EXCHANGE_OVER_QUERY = Q_IN_REGS && SINGLE_EXCHANGE_SMEM <= sizeof(bf16) * 16 * ROW;
// Two ways to bring a tile of keys and values in.  COPIES: sixteen-byte cp.async copies row by
// row through the block table, into padded rows; any head size, any page size.  PAGES: one
// tensor-map (TMA) load per page and 64-column half into dense, 128-byte-swizzled tiles, issued
// by one thread: the other warps spend no instruction on moving data, which is what bounds the
// COPIES form when a CTA walks many tiles (each tile is 2,048 copies through the load-store
// unit).  PAGES wants head sizes that are multiples of 64 and pages of 8, 16, 32 or 64 tokens.
constexpr bool CAN_PAGES = D % 64 == 0;
constexpr int HALVES = D / 64;
constexpr int ERR_TILE_WAIT = 21, ERR_TILE_ALIGNMENT = 22;

// The 8-element chunk that holds element d (a multiple of 8) of key `key` in a tile.
template <bool PAGES>
__device__ __forceinline__ bf16* tile_chunk(bf16* tile, int key, int d) {
  if (PAGES) return tile + ((d >> 6) * BN + key) * 64 + ((((d & 63) >> 3) ^ (key & 7)) << 3);
  return tile + key * ROW + d;
}

// The warps split a tile's keys for Q K^T and the head dimension for P V; the probabilities
// pass through shared memory in between.  So each warp keeps only its columns of the output
// (a few registers), twice as many warps fit as with a whole output row per warp, and nothing
// is merged across warps when the keys run out.
// PAGES adds a ninth warp that does nothing but hand a tile's loads to the copy engine (each
// takes the issuing warp a few hundred cycles), so the eight others never wait on that.
constexpr int PAGES_THREADS = STHREADS + 32;
__device__ __forceinline__ void math_warps_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(STHREADS) : "memory"); }

template <bool PAGES>
__global__ void __launch_bounds__(PAGES ? PAGES_THREADS : STHREADS, D <= 128 ? 2 : 1)
single_token_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int is_last;
  __shared__ int give_up;
  __shared__ long long tile_rows[PAGES ? 1 : ST + 1][PAGES ? 1 : BN];
  __shared__ unsigned long long tile_full[ST];   // PAGES: a stage's pages have all arrived
  constexpr int TILE = PAGES ? BN * D : BN * ROW;   // elements of one key (or value) tile
  constexpr int NT = PAGES ? PAGES_THREADS : STHREADS;
  // COPIES: query tile, then the key and value stages.  PAGES: the stages first (the swizzle
  // wants them on 1 KiB boundaries), then the query tile and the exchange space.
  bf16* k_tiles = reinterpret_cast<bf16*>(smem_raw) + (PAGES ? 0 : 16 * ROW);   // [ST][TILE]
  bf16* v_tiles = k_tiles + ST * TILE;
  bf16* q_tile = PAGES ? v_tiles + ST * TILE : reinterpret_cast<bf16*>(smem_raw);   // [16][ROW]
  unsigned char* exchange = PAGES ? reinterpret_cast<unsigned char*>(q_tile + 16 * ROW)
                                  : (EXCHANGE_OVER_QUERY ? smem_raw : reinterpret_cast<unsigned char*>(v_tiles + ST * TILE));
  bf16* probs = reinterpret_cast<bf16*>(exchange);                                 // [16][PROW]
  float* warp_max = reinterpret_cast<float*>(exchange + sizeof(bf16) * 16 * PROW); // [SW][16]
  float* warp_sum = warp_max + SW * 16;                                            // [SW][16]
  let_dependents_start();
  // Before wait_for_previous() only what no kernel of this step writes is read: the batch's
  // metadata and the keys and values of earlier positions.  The newest key (position
  // ctx_len - 1) and the query are written by the kernel just before this one.
  const int seq = blockIdx.z, split = blockIdx.x;
  const int group = p.num_heads / p.num_kv_heads;
  const int row_tiles = (group + 15) / 16;
  const int kv_head = blockIdx.y / row_tiles, row_tile = blockIdx.y - kv_head * row_tiles;
  const int start = p.q_start[seq];
  if (p.q_start[seq + 1] - start != 1) {
    wait_for_previous();
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int last_key = p.ctx_len[seq] - 1;
  const int first_key = p.window > 0 ? max(0, last_key - p.window + 1) : 0;
  const int* table = p.block_table + static_cast<size_t>(seq) * p.max_blocks;
  const int head0 = kv_head * group + row_tile * 16;
  const int rows_here = min(16, group - row_tile * 16);
  const int tile_lo = first_key / BN, tile_hi = last_key / BN;
  // the tiles are dealt out as evenly as they go: no two splits differ by more than one
  const int tiles = tile_hi - tile_lo + 1;
  const int my_lo = tile_lo + static_cast<int>(static_cast<long long>(split) * tiles / p.splits);
  const int my_hi = tile_lo + static_cast<int>(static_cast<long long>(split + 1) * tiles / p.splits) - 1;

  float o[MY_PAIRS][2][4];   // rows lane/4 and lane/4 + 8 of this warp's 16-column blocks
#pragma unroll
  for (int i = 0; i < MY_PAIRS; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][j][e] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY};   // the same in every warp
  float row_sum[2] = {0.f, 0.f};               // this thread's share: its keys only

  // PAGES: the ninth warp brings the tiles in.  Its lane j looks up page j of a tile in the block
  // table (-1: no key of [first_key, last_key] lies there, or the sequence holds no such page);
  // then each lane issues one of the tile's loads (page x 64-column half x key-or-value).  The
  // copy engine takes them in one after the other (about 50 ns apiece), which holds the issuing
  // warp for most of a microsecond per tile: hence a warp of its own.
  const int pages_per_tile = PAGES ? BN >> p.page_shift : 1;
  auto lookup_page_of_lane = [&](int tile) -> int {
    if (lane >= pages_per_tile) return -1;
    const int block = tile * pages_per_tile + lane;
    const int lo = block << p.page_shift, hi = lo + p.page_size - 1;
    if (hi < first_key || lo > last_key || block >= p.max_blocks) return -1;
    return table[block];   // used (and checked) a round later: nothing here waits for the load
  };
  auto issue_pages = [&](int stage, int page_of_lane, bool after_stores) {   // the loading warp, all lanes
    if (page_of_lane >= p.num_pages) page_of_lane = -1;
    const unsigned holders = __ballot_sync(0xffffffffu, page_of_lane >= 0);
    // the copy engine is about to write where ordinary stores have been (value rows cleared in a
    // sequence's first tile): those must be out of its way.  Reads alone need no such fence.
    if (after_stores) bw::fence_async_shared();
    if (lane == 0) {   // the one arrival of the phase
      if (holders == 0) bw::mbar_arrive(&tile_full[stage]);
      else bw::mbar_expect_tx(&tile_full[stage], static_cast<unsigned>(__popc(holders)) * p.page_size * D * 2u * sizeof(bf16));
    }
    __syncwarp();
    const int loads = pages_per_tile * HALVES * 2;
    for (int base = 0; base < loads; base += 32) {
      const int index = base + lane;
      const int j = min(index / (HALVES * 2), pages_per_tile - 1), rest = index % (HALVES * 2);
      const int page = __shfl_sync(0xffffffffu, page_of_lane, j);
      if (index < loads && page >= 0) {
        const int h = rest >> 1;
        const int at = stage * TILE + (h * BN + j * p.page_size) * 64;
        if (rest & 1) bw::tma_load_2d(v_tiles + at, &map_v, &tile_full[stage], kv_head * D + h * 64, page * p.page_size);
        else bw::tma_load_2d(k_tiles + at, &map_k, &tile_full[stage], kv_head * D + h * 64, page * p.page_size);
      }
    }
  };
  if (PAGES) {
    if (threadIdx.x == 0) {
      for (int stage = 0; stage < ST; ++stage) bw::mbar_init(&tile_full[stage], 1);
      give_up = 0;
      bw::mbar_init_fence();
      if ((bw::smem_u32(smem_raw) & 1023u) && p.status != nullptr) *p.status = ERR_TILE_ALIGNMENT;
    }
    __syncthreads();
    // the first ST - 1 tiles ahead of the wait; the row of the newest key in them is stale and
    // is copied again after the wait
    if (warp == SW) {
#pragma unroll
      for (int ahead = 0; ahead < ST - 1; ++ahead)
        if (my_lo + ahead <= my_hi) issue_pages(ahead, lookup_page_of_lane(my_lo + ahead), false);
    }
  } else if (my_lo <= my_hi) {
    // rows of the first ST - 1 tiles without the newest key, and their copies, ahead of the wait
#pragma unroll
    for (int ahead = 0; ahead < ST - 1; ++ahead)
      if (my_lo + ahead <= my_hi)
        locate_tile<BN>(tile_rows[ahead], p, table, kv_head, (my_lo + ahead) * BN, first_key, last_key, last_key);
    __syncthreads();
    // one commit group per tile, also when there is no tile left, so that the count is uniform
#pragma unroll
    for (int ahead = 0; ahead < ST - 1; ++ahead) {
      if (my_lo + ahead <= my_hi) copy_tile<BN, STHREADS>(k_tiles + ahead * TILE, v_tiles + ahead * TILE, p, tile_rows[ahead]);
      cp_async_commit();
    }
  }
  wait_for_previous();
  if (my_lo <= my_hi) {
    for (int c = threadIdx.x; c < 16 * CHUNKS; c += NT) {
      const int row = c / CHUNKS, chunk = c - row * CHUNKS;
      const bool valid = row < rows_here;
      const bf16* src = p.q + (static_cast<size_t>(start) * p.num_heads + head0 + (valid ? row : 0)) * D + chunk * 8;
      cp_async16(q_tile + row * ROW + chunk * 8, src, valid);
    }
    // the newest key, when its tile is one of those copied above
    const int newest_tile = last_key / BN;
    const bool newest_copied = newest_tile >= my_lo && newest_tile <= my_hi && newest_tile - my_lo < ST - 1;
    if (PAGES && newest_copied)   // its page must have landed before the row is replaced
      bw::mbar_wait(&tile_full[newest_tile - my_lo], 0, &give_up, p.status, ERR_TILE_WAIT);
    if (newest_copied && threadIdx.x < CHUNKS) {
      const int block = last_key / p.page_size;
      const int page = block < p.max_blocks ? table[block] : -1;
      const bool valid = page >= 0 && page < p.num_pages;
      const size_t offset = valid ? (static_cast<size_t>(page) * p.page_size + (last_key - block * p.page_size)) * p.num_kv_heads * D +
                                        static_cast<size_t>(kv_head) * D + threadIdx.x * 8 : 0;
      const int stage = newest_tile - my_lo, key = last_key - newest_tile * BN;
      cp_async16(tile_chunk<PAGES>(k_tiles + stage * TILE, key, threadIdx.x * 8), p.k_cache + offset, valid);
      cp_async16(tile_chunk<PAGES>(v_tiles + stage * TILE, key, threadIdx.x * 8), p.v_cache + offset, valid);
    }
    cp_async_commit();
    if (!PAGES && my_lo + ST - 1 <= my_hi)   // copied by the first round of the loop
      locate_tile<BN>(tile_rows[ST - 1], p, table, kv_head, (my_lo + ST - 1) * BN, first_key, last_key);
    // The table lookup for a tile is issued one round before its rows are stored, which is
    // one more round before they are copied: no round waits for a lookup of its own.
    int pending_page = -1;
    if (!PAGES && my_lo + ST <= my_hi && threadIdx.x < BN)
      pending_page = lookup_page(p, table, (my_lo + ST) * BN + threadIdx.x, first_key, last_key, -1);
    int page_ahead = -1;   // PAGES, loading warp: lane j's page of the tile that the next round loads
    if (PAGES && warp == SW && my_lo + ST - 1 <= my_hi) page_ahead = lookup_page_of_lane(my_lo + ST - 1);
    cp_async_wait<0>();
    __syncthreads();
    unsigned q_frag[Q_IN_REGS ? KSTEPS : 1][4];
    if (Q_IN_REGS && warp < SW) {
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk)
        ldmatrix_x4(q_frag[Q_IN_REGS ? kk : 0], q_tile + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + kk * 16 + 8 * (lane >> 4));
    }
    for (int tile = my_lo; tile <= my_hi; ++tile) {
      const int buffer = (tile - my_lo) % ST;
      const int ahead = tile + ST - 1;
      // this tile has arrived; every warp is done with the tile before (its buffer is loaded into
      // next), and, in the first round, with reading the query out of the space the probabilities take
      if (PAGES) bw::mbar_wait(&tile_full[buffer], ((tile - my_lo) / ST) & 1, &give_up, p.status, ERR_TILE_WAIT);
      else cp_async_wait<ST - 2>();
      __syncthreads();
      if (PAGES && give_up) break;   // a load that never landed is reported, not waited for; all leave together
      if (PAGES) {
        // Pages come whole: rows of keys outside [first_key, last_key] hold whatever the pool holds
        // (or nothing was loaded for them).  Their probabilities are zero, but zero times a stray
        // NaN is NaN, so those value rows are cleared.  Only a sequence's first and last tiles have any.
        if (tile * BN < first_key || tile * BN + BN - 1 > last_key) {
          for (int c = threadIdx.x; c < BN * CHUNKS; c += NT) {
            const int key = c / CHUNKS, chunk = c - key * CHUNKS;
            const int position = tile * BN + key;
            if (position < first_key || position > last_key)
              *reinterpret_cast<uint4*>(tile_chunk<PAGES>(v_tiles + buffer * TILE, key, chunk * 8)) = make_uint4(0u, 0u, 0u, 0u);
          }
          __syncthreads();
        }
        if (warp == SW) {   // the loading warp: the next tile's loads, then on to the next round's barrier
          if (ahead <= my_hi) {
            issue_pages((ahead - my_lo) % ST, page_ahead, (ahead - ST) * BN < first_key);
            page_ahead = ahead + 1 <= my_hi ? lookup_page_of_lane(ahead + 1) : -1;   // used one round from now
          }
          continue;
        }
      } else if (ahead <= my_hi) {
        const int into = (ahead - my_lo) % ST;
        copy_tile<BN, STHREADS>(k_tiles + into * TILE, v_tiles + into * TILE, p, tile_rows[(ahead - my_lo) % (ST + 1)]);
      }
      if (!PAGES) cp_async_commit();
      if (!PAGES && threadIdx.x < BN) {
        if (ahead + 1 <= my_hi)   // read in the next round, after its opening barrier
          tile_rows[(ahead + 1 - my_lo) % (ST + 1)][threadIdx.x] = row_of(p, kv_head, (ahead + 1) * BN + threadIdx.x, pending_page);
        if (ahead + 2 <= my_hi)
          pending_page = lookup_page(p, table, (ahead + 2) * BN + threadIdx.x, first_key, last_key, -1);
      }
      bf16* k_tile = k_tiles + buffer * TILE;
      bf16* v_tile = v_tiles + buffer * TILE;
      // scores of this warp's keys: S[16 x 8] = Q[16 x D] K^T
      const int key0 = warp * WARP_KEYS;
      float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc_odd[4] = {0.f, 0.f, 0.f, 0.f};   // two chains of dependent MMAs, not one
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        unsigned a[4], b[2];
        if (Q_IN_REGS) {
#pragma unroll
          for (int i = 0; i < 4; ++i) a[i] = q_frag[Q_IN_REGS ? kk : 0][i];
        } else {
          ldmatrix_x4(a, q_tile + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + kk * 16 + 8 * (lane >> 4));
        }
        ldmatrix_x2(b, tile_chunk<PAGES>(k_tile, key0 + (lane & 7), kk * 16 + 8 * ((lane >> 3) & 1)));
        if (kk & 1) mma_bf16(sc_odd, a, b[0], b[1]);
        else mma_bf16(sc, a, b[0], b[1]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[e] += sc_odd[e];
      // mask, scale, and this warp's maximum per row
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = tile * BN + key0 + (lane & 3) * 2 + (e & 1);
        const bool seen = key >= first_key && key <= last_key;
        sc[e] = seen ? sc[e] * p.scale_log2 : -INFINITY;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], sc[e]);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        if ((lane & 3) == 0) warp_max[warp * 16 + (lane >> 2) + 8 * r] = tile_max[r];
      }
      if (PAGES) math_warps_barrier();
      else __syncthreads();
      // the tile's maximum over all warps, the same sum order everywhere: every warp arrives
      // at the same running maximum and the same correction
      float correction[2], base[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float m = row_max[r];
#pragma unroll
        for (int w = 0; w < SW; ++w) m = fmaxf(m, warp_max[w * 16 + (lane >> 2) + 8 * r]);
        base[r] = m == -INFINITY ? 0.f : m;              // a row that has seen no key yet
        correction[r] = exp2f(row_max[r] - base[r]);     // exp2(-inf) = 0
        row_max[r] = m;
        row_sum[r] *= correction[r];
      }
      float prob[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        prob[e] = exp2f(sc[e] - base[e >> 1]);
        row_sum[e >> 1] += prob[e];
      }
      // probabilities as bfloat16 (as the values are) into the shared tile
      *reinterpret_cast<unsigned*>(probs + (lane >> 2) * PROW + key0 + (lane & 3) * 2) = pack_bf16(prob[0], prob[1]);
      *reinterpret_cast<unsigned*>(probs + ((lane >> 2) + 8) * PROW + key0 + (lane & 3) * 2) = pack_bf16(prob[2], prob[3]);
#pragma unroll
      for (int i = 0; i < MY_PAIRS; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          o[i][j][0] *= correction[0];
          o[i][j][1] *= correction[0];
          o[i][j][2] *= correction[1];
          o[i][j][3] *= correction[1];
        }
      if (PAGES) math_warps_barrier();
      else __syncthreads();
      // O[16 x 16 columns] += P[16 x 64] V[64 x 16 columns] for each of this warp's column blocks
#pragma unroll
      for (int i = 0; i < MY_PAIRS; ++i) {
        const int pair = warp + i * SW;
        if (pair < DPAIRS) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            unsigned a[4], b[4];
            ldmatrix_x4(a, probs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * PROW + kk * 16 + 8 * (lane >> 4));
            ldmatrix_x4_trans(b, tile_chunk<PAGES>(v_tile, kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), pair * 16 + 8 * (lane >> 4)));
            mma_bf16(o[i][0], a, b[0], b[1]);
            mma_bf16(o[i][1], a, b[2], b[3]);
          }
        }
      }
    }
    if (!PAGES) cp_async_wait<0>();
  }
  // every row's sum: the threads' shares over the quad, then over the warps
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
  if ((lane & 3) == 0 && warp < SW) {   // a space of its own: no barrier needed before it is written
    warp_sum[warp * 16 + (lane >> 2)] = row_sum[0];
    warp_sum[warp * 16 + (lane >> 2) + 8] = row_sum[1];
  }
  __syncthreads();
  float total_sum[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int w = 0; w < SW; ++w) total_sum[r] += warp_sum[w * 16 + (lane >> 2) + 8 * r];
  __syncthreads();   // the tiles and the exchange space are free from here on
  // this CTA's result, unnormalised, with its maximum and sum: to the output, to the cluster
  // (shared memory) or to global memory, straight from the registers
  float* cta_o = reinterpret_cast<float*>(smem_raw);          // [16][D], read by the cluster
  float* cta_ml = cta_o + 16 * D;                             // [16][2]
  const bool direct = p.splits == 1;   // nothing to combine: the result goes straight out
  const int partials = p.splits / p.cluster;   // what the clusters leave in global memory
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    if (row >= rows_here || warp >= SW) continue;
    const float inv = total_sum[r] > 0.f ? 1.0f / total_sum[r] : 0.f;
    const size_t slot = (static_cast<size_t>(seq) * p.num_heads + head0 + row) * p.splits + split;
#pragma unroll
    for (int i = 0; i < MY_PAIRS; ++i) {
      const int pair = warp + i * SW;
      if (pair >= DPAIRS) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int d = pair * 16 + j * 8 + (lane & 3) * 2;
        const float x = o[i][j][2 * r], y = o[i][j][2 * r + 1];
        if (p.cluster > 1) {
          *reinterpret_cast<float2*>(cta_o + row * D + d) = make_float2(x, y);
        } else if (direct) {
          *reinterpret_cast<__nv_bfloat162*>(p.out + (static_cast<size_t>(start) * p.num_heads + head0 + row) * D + d) =
              __floats2bfloat162_rn(x * inv, y * inv);
        } else {
          *reinterpret_cast<float2*>(p.partial_out + slot * D + d) = make_float2(x, y);
        }
      }
    }
    if (warp == 0 && (lane & 3) == 0) {
      if (p.cluster > 1) {
        cta_ml[row * 2] = row_max[r];
        cta_ml[row * 2 + 1] = total_sum[r];
      } else if (!direct) {
        p.partial_ml[slot * 2] = row_max[r];
        p.partial_ml[slot * 2 + 1] = total_sum[r];
      }
    }
  }
  if (p.cluster > 1) {
    // The cluster's CTAs add their results up through distributed shared memory: each takes
    // a slice of the (row, column) space and reads that slice from every CTA of the cluster,
    // in rank order.  Nothing passes through global memory unless there are more clusters.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int rank = static_cast<int>(cluster.block_rank());
    const int outputs = rows_here * D;
    const int share = (outputs + p.cluster - 1) / p.cluster;
    const int stop = min(outputs, (rank + 1) * share);
    for (int idx = rank * share + threadIdx.x; idx < stop; idx += NT) {
      const int row = idx / D, d = idx - row * D;
      float peer_max[8], peer_sum[8], peer_o[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < p.cluster) {
          const float* ml = cluster.map_shared_rank(cta_ml, r);
          peer_max[r] = ml[row * 2];
          peer_sum[r] = ml[row * 2 + 1];
          peer_o[r] = cluster.map_shared_rank(cta_o, r)[idx];
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.cluster) m = fmaxf(m, peer_max[r]);
      float sum = 0.f, total = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < p.cluster) {
          const float weight = peer_max[r] == -INFINITY ? 0.f : exp2f(peer_max[r] - m);
          sum += weight * peer_sum[r];
          total += weight * peer_o[r];
        }
      }
      if (partials == 1) {
        p.out[(static_cast<size_t>(start) * p.num_heads + head0 + row) * D + d] =
            __float2bfloat16_rn(sum > 0.f ? total / sum : 0.f);
      } else {
        const size_t slot = (static_cast<size_t>(seq) * p.num_heads + head0 + row) * partials + split / p.cluster;
        p.partial_out[slot * D + d] = total;
        if (d == 0) {
          p.partial_ml[slot * 2] = m;
          p.partial_ml[slot * 2 + 1] = sum;
        }
      }
    }
    cluster.sync();   // no CTA leaves while its shared memory may still be read
  }
  if (direct || partials == 1) return;
  // the CTA that arrives last combines all partials; the order of the sum is by partial
  // index, whoever does it
  // One thread speaks for the CTA: the barrier orders every thread's stores before its fence, the
  // fence before its count; on the other side its count, then its fence, then the barrier come
  // before every thread's loads (which bypass L1).  A fence in every thread would say no more.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    int* counter = p.arrivals + static_cast<size_t>(seq) * gridDim.y + blockIdx.y;
    const int before = atomicAdd(counter, 1);
    is_last = before == p.splits - 1;   // every CTA counts, whatever the cluster size
    if (is_last) *counter = 0;   // ready for the next launch
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  // Each thread takes four columns of one row and reads the (max, sum) pairs and the four
  // columns of up to eight partials in one go: the combine costs one memory round trip per
  // eight partials, not one per partial.  Chunks of eight are merged like attention tiles, in
  // partial order.
  constexpr int QUADS = D / 4;
  const int items = rows_here * QUADS;
  for (int item = threadIdx.x; item < items; item += NT) {
    const int row = item / QUADS, quad = item - row * QUADS;
    float run_max = -INFINITY, run_sum = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int base = 0; base < partials; base += 8) {
      float2 ml[8];
      float4 part[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (base + j < partials) {
          const size_t slot = (static_cast<size_t>(seq) * p.num_heads + head0 + row) * partials + base + j;
          ml[j] = __ldcg(reinterpret_cast<const float2*>(p.partial_ml + slot * 2));
          part[j] = __ldcg(reinterpret_cast<const float4*>(p.partial_out + slot * D + quad * 4));
        }
      }
      float m = run_max;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (base + j < partials) m = fmaxf(m, ml[j].x);
      const float rescale = run_max == -INFINITY ? 0.f : exp2f(run_max - m);
      float sum = run_sum * rescale;
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] *= rescale;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (base + j < partials) {
          const float weight = ml[j].x == -INFINITY ? 0.f : exp2f(ml[j].x - m);
          sum += weight * ml[j].y;
          acc[0] += weight * part[j].x;
          acc[1] += weight * part[j].y;
          acc[2] += weight * part[j].z;
          acc[3] += weight * part[j].w;
        }
      }
      run_max = m;
      run_sum = sum;
    }
    const float inv = run_sum > 0.f ? 1.0f / run_sum : 0.f;
    uint2 packed;
    packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(start) * p.num_heads + head0 + row) * D + quad * 4) = packed;
  }
}

constexpr size_t PORTIONS_SMEM = sizeof(bf16) * (BM * ROW + 4 * PBN * ROW);
constexpr size_t SINGLE_TILES_SMEM = sizeof(bf16) * (16 * ROW + 2 * ST * BN * ROW) + (EXCHANGE_OVER_QUERY ? 0 : SINGLE_EXCHANGE_SMEM);
constexpr size_t SINGLE_MERGE_SMEM = sizeof(float) * (16 * D + 32);
constexpr size_t SINGLE_SMEM = SINGLE_TILES_SMEM > SINGLE_MERGE_SMEM ? SINGLE_TILES_SMEM : SINGLE_MERGE_SMEM;
constexpr size_t SINGLE_PAGES_TILES_SMEM = sizeof(bf16) * (2 * ST * BN * D + 16 * ROW) + SINGLE_EXCHANGE_SMEM;
constexpr size_t SINGLE_PAGES_SMEM = SINGLE_PAGES_TILES_SMEM > SINGLE_MERGE_SMEM ? SINGLE_PAGES_TILES_SMEM : SINGLE_MERGE_SMEM;

}  // namespace bf16attn

// Whether single tokens may take the PAGES form (tensor-map loads); off: always COPIES.
static int g_single_token_pages = 1;
SHRIKE_API void shrike_attention_single_token_pages(int enabled) { g_single_token_pages = enabled ? 1 : 0; }

// Scratch the single-token path needs, in floats: partial outputs and (max, sum) pairs,
// one per cluster of splits.
SHRIKE_API long long shrike_attention_bf16_scratch_floats(int num_seqs, int num_heads, int splits, int cluster) {
  return static_cast<long long>(num_seqs) * num_heads * (splits / (cluster < 1 ? 1 : cluster)) * (bf16attn::D + 2);
}
// How many single-token CTAs the GPU holds at once; the host picks
// splits = min(tiles, this / (seqs * kv heads * row tiles)).
SHRIKE_API int shrike_attention_bf16_resident_ctas() {
  const size_t smem = bf16attn::SINGLE_SMEM + 1024;
  const ShrikeDevice& device = shrike_device();
  const int per_sm = static_cast<int>(static_cast<size_t>(device.max_smem) / smem);
  return device.sm_count * (per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm));
}

// has_single / has_portions: whether the batch holds rows with q_len == 1 / q_len > 1
// (known on the host); max_q_len bounds the portions grid.  `cluster` (1, 2, 4 or 8, a
// divisor of splits) consecutive splits add up on chip.  scratch holds
// shrike_attention_bf16_scratch_floats(num_seqs, num_heads, splits, cluster) floats when has_single, and
// arrivals num_seqs * num_kv_heads * ceil(group / 16) ints that are zero before the first launch
// (every launch leaves them zero again).
SHRIKE_API int shrike_paged_attention_bf16(const void* q, const void* k_cache, const void* v_cache,
                                           const int* block_table, int max_blocks, const int* q_start,
                                           const int* ctx_len, int num_seqs, int num_heads, int num_kv_heads,
                                           int page_size, int num_pages, float scale, int window, void* out,
                                           int has_single, int has_portions, int max_q_len, int splits,
                                           int cluster, float* scratch, int* arrivals, int* status, cudaStream_t stream) {
  using namespace bf16attn;
  if (num_seqs <= 0) return SHRIKE_OK;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || page_size <= 0 || max_blocks <= 0 ||
      num_seqs > 65535 || num_heads > 65535)
    return SHRIKE_BAD_ARGUMENT;
  if (has_single) {
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return SHRIKE_BAD_ARGUMENT;
    if (splits < 1 || splits % cluster || splits / cluster > MAX_SPLITS || arrivals == nullptr) return SHRIKE_BAD_ARGUMENT;
    if (splits > cluster && scratch == nullptr) return SHRIKE_BAD_ARGUMENT;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e1 = cudaFuncSetAttribute(portions_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(PORTIONS_SMEM));
    cudaError_t e2 = cudaFuncSetAttribute(single_token_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SINGLE_SMEM));
    if (e1 != cudaSuccess || e2 != cudaSuccess) return static_cast<int>(e1 != cudaSuccess ? e1 : e2);
    if (CAN_PAGES) {
      cudaError_t e3 = cudaFuncSetAttribute(single_token_kernel<CAN_PAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SINGLE_PAGES_SMEM));
      if (e3 != cudaSuccess) return static_cast<int>(e3);
    }
    configured = true;
  }
  Params p;
  p.q = static_cast<const bf16*>(q);
  p.k_cache = static_cast<const bf16*>(k_cache);
  p.v_cache = static_cast<const bf16*>(v_cache);
  p.block_table = block_table;
  p.q_start = q_start;
  p.ctx_len = ctx_len;
  p.out = static_cast<bf16*>(out);
  p.max_blocks = max_blocks;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.page_shift = -1;
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) p.page_shift = shift;
  p.num_pages = num_pages;
  p.window = window;
  p.splits = has_single ? splits : 1;
  p.cluster = has_single ? cluster : 1;
  p.skip_single = has_single ? 1 : 0;
  p.scale_log2 = scale * LOG2E;
  p.partial_out = scratch;
  p.partial_ml = scratch ? scratch + static_cast<size_t>(num_seqs) * num_heads * (p.splits / p.cluster) * D : nullptr;
  p.arrivals = arrivals;
  p.status = status;
  if (has_single) {
    const int group = num_heads / num_kv_heads;
    const dim3 grid(p.splits, num_kv_heads * ((group + 15) / 16), num_seqs);
    CUtensorMap map_k = {}, map_v = {};
    bool pages = CAN_PAGES && g_single_token_pages && p.page_shift >= 3 && p.page_shift <= 6;
    if (pages) {   // one row of the map per cache slot, all kv heads side by side
      const long long slots = static_cast<long long>(num_pages) * page_size;
      pages = bw::tensor_map_bf16(k_cache, slots, num_kv_heads * D, page_size, &map_k) == SHRIKE_OK &&
              bw::tensor_map_bf16(v_cache, slots, num_kv_heads * D, page_size, &map_v) == SHRIKE_OK;
    }
    if (pages) launch_dependent_clusters(single_token_kernel<CAN_PAGES>, grid, PAGES_THREADS, SINGLE_PAGES_SMEM, stream, p.cluster, map_k, map_v, p);
    else launch_dependent_clusters(single_token_kernel<false>, grid, STHREADS, SINGLE_SMEM, stream, p.cluster, map_k, map_v, p);
  }
  if (has_portions) {
    const dim3 grid((max_q_len + BM - 1) / BM, num_heads, num_seqs);
    launch_dependent(portions_kernel, grid, THREADS, PORTIONS_SMEM, stream, p);
  }
  return shrike_launch_status();
}
