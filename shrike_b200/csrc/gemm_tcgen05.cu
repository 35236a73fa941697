// out[T, N] = x[T, K] * w[N, K]^T (+ bias) in bfloat16 with float32 accumulation, on the
// fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory,
// operands brought to shared memory by TMA.  Written for few tokens against a large
// weight (decoding): the step is bound by reading w once from HBM, so the kernel is laid
// out to keep every SM streaming weights.
//
// Orientation ("swap A and B"): the 128-row MMA dimension runs over WEIGHT rows, the
// narrow dimension (16..256) over tokens.  One CTA owns 128 weight rows and, when K is
// split, one slice of K; the accumulator D[weight row, token] sits in 128 TMEM lanes x
// Tn columns.  Split K: CTA (tile, s) writes partial s of the result; the consumer kernel
// (residual-add + norm, or bias + rotary) adds the partials in a fixed order, so the sum
// is deterministic and costs no pass of its own.
//
// Roles (192 threads): warp 0 issues TMA loads (one elected lane), warp 1 allocates TMEM
// and issues the MMAs (one elected lane), warps 2..5 read the accumulator back
// (tcgen05.ld, each warp its quarter of the lanes) and store the result.  Stages are
// handed over with mbarriers: full[s] (TMA bytes landed), empty[s] (tcgen05.commit: the
// MMAs that read stage s are done), done (all MMAs of the tile are done).
//
// Shared-memory tiles are [rows][64 bf16] = 128-byte rows in the 128-byte swizzle that
// both TMA (CU_TENSOR_MAP_SWIZZLE_128B) and the MMA descriptor (layout type 2, 1024-byte
// stride between 8-row groups) understand; a k-step of 16 elements advances the
// descriptor's start address by 32 bytes inside the swizzle atom.
//
// The kernel is launched as a programmatic dependent of the kernel before it: it may start
// while that kernel is still running, sets up its barriers and tensor memory and already
// streams the first weight tiles (weights are written by nobody), and only then waits
// (griddepcontrol.wait) for the kernel before it to finish, before it touches the
// activations or writes its output.
//
// Every wait is bounded.  When a wait runs out, the waiting role records where in
// `status` (a host-visible word), raises a CTA-wide abort flag that ends the other roles'
// waits, the producer waits (bounded again) for its copies in flight, TMEM is freed and
// the CTA returns.  No TMA load uses cluster multicast.
#include "blackwell.cuh"

namespace tc {
using namespace bw;

constexpr int BM = 128;        // weight rows per CTA = MMA M
constexpr int BK = 64;         // k elements per stage: 128 bytes of bf16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr size_t A_BYTES = BM * BK * 2;

enum : int { ERR_NONE = 0, ERR_PRODUCER = 1, ERR_MMA = 2, ERR_EPILOGUE = 3, ERR_DRAIN = 4 };

struct Shared {
  unsigned long long full[MAX_STAGES];
  unsigned long long empty[MAX_STAGES];
  unsigned long long done;
  unsigned tmem_base;
  volatile int abort;
};

__device__ __forceinline__ void tmem_load16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

struct Args {
  void* out;            // [splits][T][N] float32 when splits > 1, else [T][N] of out_dtype
  const float* bias;    // [N] or null; added by split 0
  int* status;          // host-visible; first failing role is recorded
  int tokens, n, k, tn; // tn: token columns of the MMA (multiple of 16, at most 256)
  int kblocks_per_split, stages, out_dtype;
  int gated;            // the weight rows come in runs of 16 gate rows and the 16 up rows of the same
                        // features; out is [T][N / 2] bfloat16 = silu(gate) * up
};

__global__ void __launch_bounds__(THREADS, 3)
gemm_swap_ab_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Args args) {
  extern __shared__ unsigned char smem_raw[];
  // tiles want 1024-byte alignment (the swizzle pattern repeats every 1024 bytes)
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const size_t b_bytes = static_cast<size_t>(args.tn) * BK * 2;
  const size_t stage_bytes = A_BYTES + b_bytes;
  Shared* sh = reinterpret_cast<Shared*>(tiles + stage_bytes * args.stages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, split = blockIdx.y, t0 = blockIdx.z * args.tn;
  const int total_kblocks = (args.k + BK - 1) / BK;
  const int kb_begin = split * args.kblocks_per_split;
  const int kb_end = min(total_kblocks, kb_begin + args.kblocks_per_split);
  const int num_kb = max(0, kb_end - kb_begin);
  unsigned tmem_cols = 32;
  while (tmem_cols < static_cast<unsigned>(args.tn)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < args.stages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    mbar_init(&sh->done, 1);
    sh->abort = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, tmem_cols);
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  // dependents may start only now that this CTA holds its tensor memory: a dependent that also
  // wants tensor memory must not be able to starve a CTA it is waiting for
  let_dependents_start();
  const unsigned tmem_d = sh->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      // weights first: they do not depend on the kernel before this one
      const int early = min(num_kb, args.stages);
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&sh->full[i], static_cast<unsigned>(stage_bytes));
        tma_load_2d(tiles + stage_bytes * i, &map_w, &sh->full[i], (kb_begin + i) * BK, n0);
      }
      wait_for_previous();
      for (int i = 0; i < early; ++i)
        tma_load_2d(tiles + stage_bytes * i + A_BYTES, &map_x, &sh->full[i], (kb_begin + i) * BK, t0);
      int issued = early;
      for (int i = early; i < num_kb; ++i) {
        const int s = i % args.stages;
        const unsigned phase = (i / args.stages) & 1;
        if (!mbar_wait(&sh->empty[s], phase ^ 1, &sh->abort, args.status, ERR_PRODUCER)) break;
        mbar_expect_tx(&sh->full[s], static_cast<unsigned>(stage_bytes));
        unsigned char* a_tile = tiles + stage_bytes * s;
        tma_load_2d(a_tile, &map_w, &sh->full[s], (kb_begin + i) * BK, n0);
        tma_load_2d(a_tile + A_BYTES, &map_x, &sh->full[s], (kb_begin + i) * BK, t0);
        issued = i + 1;
      }
      if (sh->abort) {
        // copies may still be in flight: wait for the stages armed last before leaving
        for (int i = max(0, issued - args.stages); i < issued; ++i) {
          const int s = i % args.stages;
          const unsigned phase = (i / args.stages) & 1;
          bool landed = false;
          for (unsigned tries = 0; tries < WAIT_LIMIT && !landed; ++tries) landed = mbar_try_wait(&sh->full[s], phase);
          if (!landed && args.status != nullptr) *args.status = ERR_DRAIN;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = instruction_descriptor(BM, args.tn, false);
      bool ok = true;
      // the token tiles are loaded only after the kernel before this one has finished: wait for it
      // here too, so that the bounded waits below measure this kernel's own loads alone
      wait_for_previous();
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % args.stages;
        const unsigned phase = (i / args.stages) & 1;
        ok = mbar_wait(&sh->full[s], phase, &sh->abort, args.status, ERR_MMA);
        if (!ok) break;
        fence_after_sync();
        const unsigned a_addr = smem_u32(tiles + stage_bytes * s);
        const unsigned b_addr = a_addr + static_cast<unsigned>(A_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma(tmem_d, smem_descriptor(a_addr + kk * UMMA_K * 2), smem_descriptor(b_addr + kk * UMMA_K * 2), idesc,
               (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh->empty[s]);   // frees the stage once these MMAs have read it
      }
      if (ok) umma_commit(&sh->done);
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    const int row = n0 + quarter * 32 + lane;   // weight row = output column
    wait_for_previous();   // the output may still be read by the kernel before
    bool ok = true;
    if (num_kb > 0) ok = mbar_wait(&sh->done, 0, &sh->abort, args.status, ERR_EPILOGUE);
    fence_after_sync();
    if (ok && args.gated) {
      // A warp's 32 rows are 16 gate rows and the 16 up rows of the same features.  Lanes below
      // 16 finish tokens 0..7 of a block of 16, the others tokens 8..15; each half sends the
      // other what it needs.  Gate and up are rounded to bfloat16 first, as the separate
      // activation kernel finds them, so both ways give the same bits.
      const int feature = (n0 >> 1) + quarter * 16 + (lane & 15);
      const int half_n = args.n >> 1;
      for (int c0 = 0; c0 < args.tn; c0 += 16) {
        unsigned v[16];
        if (num_kb > 0) {
          tmem_load16(tmem_d + (static_cast<unsigned>(quarter * 32) << 16) + static_cast<unsigned>(c0), v);
          tmem_wait_load();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned mine = lane < 16 ? v[j] : v[8 + j];
          const unsigned sent = lane < 16 ? v[8 + j] : v[j];
          const unsigned other = __shfl_xor_sync(0xffffffffu, sent, 16);
          const float gate = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lane < 16 ? mine : other)));
          const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lane < 16 ? other : mine)));
          const int t = t0 + c0 + j + (lane < 16 ? 0 : 8);
          if (t < args.tokens && n0 + quarter * 32 + lane < args.n)
            static_cast<__nv_bfloat16*>(args.out)[static_cast<size_t>(t) * half_n + feature] =
                __float2bfloat16_rn(silu_times<__nv_bfloat16>(gate, up));
        }
      }
    } else if (ok) {
      const bool partial = gridDim.y > 1;
      const float bias = (args.bias != nullptr && split == 0 && row < args.n) ? args.bias[row] : 0.f;
      for (int c0 = 0; c0 < args.tn; c0 += 16) {
        unsigned v[16];
        if (num_kb > 0) {
          tmem_load16(tmem_d + (static_cast<unsigned>(quarter * 32) << 16) + static_cast<unsigned>(c0), v);
          tmem_wait_load();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
        if (row < args.n) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t >= args.tokens) break;
            const float value = __uint_as_float(v[j]) + bias;
            const size_t at = static_cast<size_t>(t) * args.n + row;
            if (partial) static_cast<float*>(args.out)[static_cast<size_t>(split) * args.tokens * args.n + at] = value;
            else if (args.out_dtype == SHRIKE_F32) static_cast<float*>(args.out)[at] = value;
            else static_cast<__nv_bfloat16*>(args.out)[at] = __float2bfloat16_rn(value);
          }
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_free(tmem_d, tmem_cols);
  }
}

}  // namespace tc

// How K is split for a product with `tokens` rows.  Two CTAs live on an SM, and as long as
// all CTAs of the product are resident together, more of them stream faster: measured at the
// projection shapes of three model sizes, the time falls with every further split until the
// grid exceeds the resident places (2 x 148), and jumps by a third right after.  So: the most
// splits that keep the grid resident, at least three k-blocks each, none empty; at most 8 (what
// the norm kernel adds in one round trip: a ninth slice costs it what the product gains), or 16
// where eight would not even give every SM a CTA.  The same function sizes the partial stack.
SHRIKE_API int shrike_gemm_tc_splits(int tokens, int n, int k) {
  (void)tokens;
  const int tiles = (n + tc::BM - 1) / tc::BM;
  const int kblocks = (k + tc::BK - 1) / tc::BK;
  const int resident = 2 * shrike_device().sm_count;
  const int most = tiles * 8 < resident / 2 ? 16 : 8;
  int best = 1;
  for (int splits = 2; splits <= most && tiles * splits <= resident; ++splits) {
    const int per = (kblocks + splits - 1) / splits;
    if (per < 3) break;
    if ((kblocks + per - 1) / per == splits) best = splits;   // else the last split would be empty
  }
  return best;
}

// x [tokens, k] and w [n, k] bfloat16 row-major, k a multiple of 8 (TMA wants 16-byte row
// strides) and both 16-byte aligned.  splits == 1: out is [tokens, n] of out_dtype.
// splits > 1 (as shrike_gemm_tc_splits says): out is [splits, tokens, n] float32.
static int launch_gemm_tc(const void* x, const void* w, const float* bias, void* out, int out_dtype, int tokens,
                          int n, int k, int splits, int gated, int* status, cudaStream_t stream) {
  using namespace tc;
  if (tokens <= 0 || n <= 0) return SHRIKE_OK;
  if (k <= 0 || k % 8 || splits < 1 || (out_dtype != SHRIKE_F32 && out_dtype != SHRIKE_BF16)) return SHRIKE_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return SHRIKE_BAD_ARGUMENT;
  int tn = 16;
  while (tn < tokens && tn < 256) tn *= 2;
  const int token_tiles = (tokens + tn - 1) / tn;
  const int kblocks = (k + BK - 1) / BK;
  const int per_split = (kblocks + splits - 1) / splits;
  if ((kblocks + per_split - 1) / per_split != splits) return SHRIKE_BAD_ARGUMENT;
  const size_t stage_bytes = A_BYTES + static_cast<size_t>(tn) * BK * 2;
  const long long ctas = static_cast<long long>((n + BM - 1) / BM) * splits * token_tiles;
  // Shared memory one CTA may take for its stages.  Half an SM's worth lets two CTAs live on
  // an SM, so that one streams weights while the other starts up or stores its result, and
  // still gives each a pipeline deep enough to cover the memory latency alone (three CTAs of
  // three stages each measured 7% slower over a whole decode step).  A product of many waves
  // (an output head) does better with four shallower CTAs per SM.
  const ShrikeDevice& device = shrike_device();
  const int budget = tn <= 16 && ctas >= 6LL * device.sm_count ? 48 * 1024 : 100 * 1024;
  int stages = static_cast<int>(budget / stage_bytes);
  if (stages < 2) stages = 2;
  stages = stages > MAX_STAGES ? MAX_STAGES : stages;
  if (stages > per_split) stages = per_split < 2 ? 2 : per_split;
  const size_t smem = stage_bytes * stages + sizeof(Shared) + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(gemm_swap_ab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, device.max_smem);
    if (err != cudaSuccess) return static_cast<int>(err);
    configured = true;
  }
  CUtensorMap map_w, map_x;
  int rc = tensor_map_bf16(w, n, k, BM, &map_w);
  if (rc != SHRIKE_OK) return rc;
  rc = tensor_map_bf16(x, tokens, k, tn, &map_x);
  if (rc != SHRIKE_OK) return rc;
  Args args;
  args.out = out;
  args.bias = bias;
  args.status = status;
  args.tokens = tokens;
  args.n = n;
  args.k = k;
  args.tn = tn;
  args.kblocks_per_split = per_split;
  args.stages = stages;
  args.gated = gated;
  args.out_dtype = out_dtype;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((n + BM - 1) / BM, splits, token_tiles);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&config, gemm_swap_ab_kernel, map_w, map_x, args);
  if (err != cudaSuccess) return static_cast<int>(err);
  return shrike_launch_status();
}

SHRIKE_API int shrike_gemm_tc(const void* x, const void* w, const float* bias, void* out, int out_dtype, int tokens,
                              int n, int k, int splits, int* status, cudaStream_t stream) {
  return launch_gemm_tc(x, w, bias, out, out_dtype, tokens, n, k, splits, 0, status, stream);
}

// The gated feed-forward's first product with its activation: w [n, k] holds, in runs of 32 rows,
// 16 gate rows and the 16 up rows of the same features (n a multiple of 32); out [tokens, n / 2]
// bfloat16 = silu(x w_gate^T) * (x w_up^T), gate and up rounded to bfloat16 before the activation.
SHRIKE_API int shrike_gemm_tc_gated(const void* x, const void* w, void* out, int tokens, int n, int k, int* status,
                                    cudaStream_t stream) {
  if (n % 32) return SHRIKE_BAD_ARGUMENT;
  return launch_gemm_tc(x, w, nullptr, out, SHRIKE_BF16, tokens, n, k, 1, 1, status, stream);
}
