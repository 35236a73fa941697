// Shared helpers for the sm_100a kernels: element types, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SHRIKE_API extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { SHRIKE_F32 = 0, SHRIKE_BF16 = 1, SHRIKE_NONE = -1 };

// Status codes returned by every launcher (0 = launched).
enum : int { SHRIKE_OK = 0, SHRIKE_BAD_ARGUMENT = -1 };

static inline int shrike_launch_status() {
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? SHRIKE_OK : static_cast<int>(err);
}

// What launchers need to know of the current device (grids and shared-memory budgets follow
// from it), asked once per device; the figures of a B200 stand in if the query fails.
struct ShrikeDevice {
  int sm_count = 0;
  int max_smem = 0;   // most dynamic shared memory a CTA may ask for
};
static inline const ShrikeDevice& shrike_device() {
  static ShrikeDevice facts[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
  ShrikeDevice& f = facts[device];
  if (f.sm_count == 0) {
    int sms = 0, smem = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    if (cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess || smem <= 0)
      smem = 227 * 1024;
    f.max_smem = smem;
    f.sm_count = sms;
  }
  return f;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Programmatic dependent launch.  Every kernel of this package is launched so that it may
// start while the kernel before it on the stream is still running (its launch latency and
// set-up are hidden that way), and every kernel begins with
//   let_dependents_start();   the kernel after this one may start now
//   wait_for_previous();      block until the kernel before this one has finished and its
//                             writes are visible
// before it reads or writes any memory that another kernel touches.  Only work on memory
// that no kernel writes (weights) may come before wait_for_previous().
__device__ __forceinline__ void let_dependents_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_previous() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launches `kernel` as a programmatic dependent of the work before it on `stream`.
template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// The same for a kernel whose CTAs form clusters of `cluster_x` along x (gridDim.x a multiple of it).
template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch_dependent_clusters(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                                    cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  attributes[1].id = cudaLaunchAttributeClusterDimension;
  attributes[1].val.clusterDim.x = cluster_x;
  attributes[1].val.clusterDim.y = 1;
  attributes[1].val.clusterDim.z = 1;
  config.attrs = attributes;
  config.numAttrs = 2;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// silu(g) * u, silu(g) = g / (1 + exp(-g)), with one rounding of the product.  bfloat16 results
// keep 8 bits of mantissa, so that path may use the hardware exponential and reciprocal
// (relative error about 2^-22); the float32 path uses the exact functions.  Shared by the
// activation kernel and the tensor-core product's activation epilogue: both give the same bits.
template <typename T> __device__ __forceinline__ float silu_times(float g, float u);
template <> __device__ __forceinline__ float silu_times<float>(float g, float u) {
  return __fmul_rn(g / (1.0f + expf(-g)), u);
}
template <> __device__ __forceinline__ float silu_times<__nv_bfloat16>(float g, float u) {
  return __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), u);
}

// base[0] + base[stride] + ... over `partials` slices (the stack a K-split product leaves),
// added in ascending order.  Up to 16 loads are issued together before the first addition,
// so the sum costs one memory latency, not one per slice.
__device__ __forceinline__ float sum_partials(const float* base, long long stride, int partials) {
  if (partials == 1) return base[0];
  float held[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) held[i] = (i == 0 || i < partials) ? base[i * stride] : 0.f;
  float sum = held[0];
#pragma unroll
  for (int i = 1; i < 16; ++i)
    if (i < partials) sum = __fadd_rn(sum, held[i]);
  for (int i = 16; i < partials; ++i) sum = __fadd_rn(sum, base[i * stride]);
  return sum;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order
// of additions depends only on the block size, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    float w = lane < warps ? scratch[lane] : 0.f;
    w = warp_sum(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    float w = lane < warps ? scratch[lane] : -INFINITY;
    w = warp_max(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
