// Sampling: one block per row of float32 logits.
//
// temperature == 0: the largest logit, lowest index on ties
//   (shrike/engine/sampler.py:15-17).
// otherwise: p = softmax(logits / temperature) in float32 (sampler.py:21-22);
//   with top_p < 1 a token is kept while the probability mass strictly above it is
//   below top_p (sampler.py:24-28: the most probable token is always kept); one
//   token is then drawn from the kept ones in proportion to p.  The draw is the
//   Gumbel-max form of a categorical sample, token = argmax(logit / T + g_i), with
//   g_i = -log(-log(u_i)) and u_i a hash of (seed, i): the same seed gives the same
//   token whatever else is in the batch (the reference's torch.multinomial on the
//   global generator, sampler.py:29, does not have that property).
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 33;
  x *= 0xFF51AFD7ED558CCDull;
  x ^= x >> 33;
  x *= 0xC4CEB9FE1A85EC53ull;
  x ^= x >> 33;
  return x;
}
__device__ __forceinline__ float gumbel(unsigned long long seed, int index) {
  const unsigned long long word = mix64(seed + static_cast<unsigned long long>(index) * 0x9E3779B97F4A7C15ull);
  const float u = (static_cast<float>(word >> 40) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

struct Best {
  float value;
  int index;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}
__device__ Best block_best(Best mine, Best* scratch /* 33 entries */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, mine.value, offset);
    other.index = __shfl_xor_sync(0xffffffffu, mine.index, offset);
    mine = better(mine, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    Best w = lane < warps ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      Best other;
      other.value = __shfl_xor_sync(0xffffffffu, w.value, offset);
      other.index = __shfl_xor_sync(0xffffffffu, w.index, offset);
      w = better(w, other);
    }
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

// A row whose logits are all NaN has no winner (no comparison with NaN holds): it yields token
// 0, a valid id, and leaves ERR_NO_FINITE_LOGIT in the status word when the caller gave one.
constexpr int ERR_NO_FINITE_LOGIT = 31;
__device__ __forceinline__ int valid_token(int index, int vocab, int* status) {
  if (index >= 0 && index < vocab) return index;
  if (status != nullptr && *status == 0) *status = ERR_NO_FINITE_LOGIT;
  return 0;
}

// Stage 1: the vocabulary of every row is cut into `chunks` slices; each block finds the
// best (score, index) of its slice, the score being the logit (greedy) or
// logit / T + Gumbel noise (sampled without top_p).  Rows with top_p < 1 are left to
// stage 2, which needs the whole row's probabilities.
constexpr int SLICE_THREADS = 256;
__global__ void __launch_bounds__(SLICE_THREADS)
sample_slices_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                     const float* __restrict__ top_p, const long long* __restrict__ seeds,
                     float* __restrict__ partial_value, int* __restrict__ partial_index, int vocab, int chunks) {
  __shared__ Best best_scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const float temp = temperature[row];
  if (temp != 0.f && top_p[row] < 1.0f) return;
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = chunk * per, end = min(vocab, begin + per);
  const float* x = logits + static_cast<size_t>(row) * vocab;
  Best mine{-INFINITY, 0x7fffffff};
  if (temp == 0.f) {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) mine = better(mine, Best{x[i], i});
  } else {
    const float inv_temp = 1.0f / temp;
    const unsigned long long seed = static_cast<unsigned long long>(seeds[row]);
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x)
      mine = better(mine, Best{x[i] * inv_temp + gumbel(seed, i), i});
  }
  const Best top = block_best(mine, best_scratch);
  if (threadIdx.x == 0) {
    partial_value[static_cast<size_t>(row) * chunks + chunk] = top.value;
    partial_index[static_cast<size_t>(row) * chunks + chunk] = top.index;
  }
}

// Stage 2: one block per row.  Rows handled by stage 1 only pick the best slice result;
// rows with top_p < 1 run the whole nucleus procedure here.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const long long* __restrict__ seeds, int* __restrict__ out,
              const float* __restrict__ partial_value, const int* __restrict__ partial_index, int vocab,
              int chunks, int* __restrict__ status) {
  __shared__ float scratch[33];
  __shared__ Best best_scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int row = blockIdx.x;
  const float* x = logits + static_cast<size_t>(row) * vocab;
  const float temp = temperature[row];
  const float nucleus = top_p[row];

  if (temp == 0.f || nucleus >= 1.0f) {
    Best mine{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < chunks; i += blockDim.x)
      mine = better(mine, Best{partial_value[static_cast<size_t>(row) * chunks + i],
                               partial_index[static_cast<size_t>(row) * chunks + i]});
    const Best top = block_best(mine, best_scratch);
    if (threadIdx.x == 0) out[row] = valid_token(top.index, vocab, status);
    return;
  }

  const float inv_temp = 1.0f / temp;
  float local_max = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) local_max = fmaxf(local_max, x[i]);
  const float row_max = block_max(local_max, scratch);
  float local_sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) local_sum += expf((x[i] - row_max) * inv_temp);
  const float total = block_sum(local_sum, scratch);
  const float inv_total = 1.0f / total;
  // Bisection on the bit pattern of a positive float: mass_above(lo) >= top_p and
  // mass_above(hi) < top_p hold throughout; at the end no probability lies
  // strictly between lo and hi, and the kept set is {p > lo}.
  unsigned lo = 0u, hi = __float_as_uint(1.0f);  // mass_above(0) = 1 >= top_p; mass_above(1) = 0
  while (hi - lo > 1u) {
    const unsigned mid = lo + (hi - lo) / 2u;
    const float cut = __uint_as_float(mid);
    float above = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float p = expf((x[i] - row_max) * inv_temp) * inv_total;
      if (p > cut) above += p;
    }
    above = block_sum(above, scratch);
    if (above < nucleus) hi = mid;
    else lo = mid;
  }
  const float threshold = lo == 0u ? -1.f : __uint_as_float(lo);
  Best mine{-INFINITY, 0x7fffffff};
  const unsigned long long seed = static_cast<unsigned long long>(seeds[row]);
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float p = expf((x[i] - row_max) * inv_temp) * inv_total;
    if (p > threshold) mine = better(mine, Best{x[i] * inv_temp + gumbel(seed, i), i});
  }
  const Best top = block_best(mine, best_scratch);
  if (threadIdx.x == 0) out[row] = valid_token(top.index, vocab, status);
}

// How many slices stage 1 cuts a row into; scratch must hold rows * slices floats and ints.
SHRIKE_API int shrike_sample_slices(int vocab) {
  const int slices = (vocab + 2047) / 2048;
  return slices < 1 ? 1 : (slices > 128 ? 128 : slices);
}

SHRIKE_API int shrike_sample(const float* logits, const float* temperature, const float* top_p,
                             const long long* seeds, int* out, float* scratch_value, int* scratch_index,
                             int rows, int vocab, int* status, cudaStream_t stream) {
  if (rows <= 0) return SHRIKE_OK;
  if (vocab <= 0 || rows > 65535 || scratch_value == nullptr || scratch_index == nullptr) return SHRIKE_BAD_ARGUMENT;
  const int chunks = shrike_sample_slices(vocab);
  launch_dependent(sample_slices_kernel, dim3(chunks, rows), SLICE_THREADS, 0, stream, logits, temperature, top_p, seeds,
                   scratch_value, scratch_index, vocab, chunks);
  launch_dependent(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, temperature, top_p, seeds, out,
                   static_cast<const float*>(scratch_value), static_cast<const int*>(scratch_index), vocab, chunks,
                   status);
  return shrike_launch_status();
}

// ------------------------------------------------------------------------------------
// The same two kernels with their scratch in a fixed device array, for callers that
// must not allocate (sampling_no_alloc.h says who they are and what the limits are).
#include <mutex>

#include "sampling_no_alloc.h"

static __device__ __align__(256) unsigned char sample_no_alloc_scratch[SHRIKE_SAMPLE_NO_ALLOC_BYTES];

namespace {
constexpr int NO_ALLOC_MAX_DEVICES = 64;
std::mutex no_alloc_mutex;
void* no_alloc_address[NO_ALLOC_MAX_DEVICES] = {};

// In host code `sample_no_alloc_scratch` is only a handle for the symbol, not an address a
// kernel can use; the device address is asked for once per device, with that device current.
int no_alloc_scratch(void** address) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (device < 0 || device >= NO_ALLOC_MAX_DEVICES) return SHRIKE_SAMPLE_NO_ALLOC_BAD_DEVICE;
  std::lock_guard<std::mutex> guard(no_alloc_mutex);
  if (no_alloc_address[device] == nullptr) {
    void* found = nullptr;
    err = cudaGetSymbolAddress(&found, sample_no_alloc_scratch);
    if (err != cudaSuccess) return static_cast<int>(err);
    no_alloc_address[device] = found;
  }
  *address = no_alloc_address[device];
  return SHRIKE_OK;
}
}  // namespace

SHRIKE_API int shrike_sample_no_alloc(const float* logits, const float* temperature, const float* top_p,
                                      const long long* seeds, int* out, int rows, int vocab,
                                      cudaStream_t stream) {
  if (rows <= 0) return SHRIKE_OK;
  if (vocab <= 0) return SHRIKE_BAD_ARGUMENT;
  if (rows > SHRIKE_SAMPLE_NO_ALLOC_MAX_ROWS) return SHRIKE_SAMPLE_NO_ALLOC_TOO_MANY_ROWS;
  const int chunks = shrike_sample_slices(vocab);  // never more than SHRIKE_SAMPLE_NO_ALLOC_MAX_SLICES
  void* base = nullptr;
  const int status = no_alloc_scratch(&base);
  if (status != SHRIKE_OK) return status;
  float* values = static_cast<float*>(base);
  int* indices = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + SHRIKE_SAMPLE_NO_ALLOC_BYTES / 2);
  sample_slices_kernel<<<dim3(chunks, rows), SLICE_THREADS, 0, stream>>>(logits, temperature, top_p, seeds,
                                                                         values, indices, vocab, chunks);
  sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, temperature, top_p, seeds, out, values, indices,
                                                     vocab, chunks, nullptr);
  return shrike_launch_status();
}

SHRIKE_API const char* shrike_sample_no_alloc_message(int code) {
  if (code == SHRIKE_OK) return "ok";
  if (code == SHRIKE_SAMPLE_NO_ALLOC_TOO_MANY_ROWS)
    return "shrike_sample_no_alloc: more than 256 rows in one call; the fixed scratch array holds 256 "
           "(split the batch, or use shrike_sample with scratch of your own)";
  if (code == SHRIKE_BAD_ARGUMENT) return "shrike_sample_no_alloc: bad argument (vocab must be positive)";
  if (code == SHRIKE_SAMPLE_NO_ALLOC_BAD_DEVICE)
    return "shrike_sample_no_alloc: the current device's index is 64 or more; the library keeps the scratch "
           "address of devices 0 to 63 only";
  return cudaGetErrorString(static_cast<cudaError_t>(code));
}
