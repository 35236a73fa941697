// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]), all float32 with float32 FMA on the CUDA
// cores: no TF32, no reduced-precision staging.  This is the matrix product of the
// true 32-bit path.  Every output element sums its K products in ascending k, in
// one chain, whatever M is, so a row's result does not depend on the batch it was in.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int GEMM_THREADS = 256;

__global__ void __launch_bounds__(GEMM_THREADS)
gemm_fp32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                 float* __restrict__ C, int M, int N, int K, int vec_ok) {
  __shared__ __align__(16) float a_tile[BK][BM + 4];
  __shared__ __align__(16) float w_tile[BK][BN + 4];
  let_dependents_start();
  wait_for_previous();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int load_row = tid >> 2, load_k = (tid & 3) * 4;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float a_reg[4] = {0.f, 0.f, 0.f, 0.f}, w_reg[4] = {0.f, 0.f, 0.f, 0.f};
    const int k = k0 + load_k;
    const int am = m0 + load_row, wn = n0 + load_row;
    if (am < M) {
      const float* src = A + static_cast<size_t>(am) * K + k;
      if (vec_ok && k + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        a_reg[0] = v.x; a_reg[1] = v.y; a_reg[2] = v.z; a_reg[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) if (k + i < K) a_reg[i] = src[i];
      }
    }
    if (wn < N) {
      const float* src = W + static_cast<size_t>(wn) * K + k;
      if (vec_ok && k + 3 < K) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src));
        w_reg[0] = v.x; w_reg[1] = v.y; w_reg[2] = v.z; w_reg[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) if (k + i < K) w_reg[i] = __ldg(src + i);
      }
    }
    __syncthreads();  // the previous tile has been consumed
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a_tile[load_k + i][load_row] = a_reg[i];
      w_tile[load_k + i][load_row] = w_reg[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&a_tile[kk][ty * 4]);
      const float4 w = *reinterpret_cast<const float4*>(&w_tile[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[static_cast<size_t>(m) * N + n] = bias ? acc[i][j] + bias[n] : acc[i][j];
    }
  }
}

SHRIKE_API int shrike_gemm_fp32(const float* A, const float* W, const float* bias, float* C, int M, int N,
                                int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SHRIKE_OK;
  if (K <= 0) return SHRIKE_BAD_ARGUMENT;
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return SHRIKE_BAD_ARGUMENT;
  const int vec_ok = (K % 4 == 0) && (reinterpret_cast<uintptr_t>(A) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(W) % 16 == 0);
  gemm_fp32_kernel<<<grid, GEMM_THREADS, 0, stream>>>(A, W, bias, C, M, N, K, vec_ok);
  return shrike_launch_status();
}
