// True float32 matrix product on CUDA cores: Y[T, N] (+)= X[T, K] . W[N, K]^T.
// No tensor cores, no reduced-precision mode.  Each output element is summed
// over k = 0..K-1 in that order by one thread, so its value does not depend on
// how many rows the batch has or on where the row sits in the batch.
// Formula: crates/janus-engine/src/compute/shaders/gemm_f32.wgsl:23-75
// (weights [N, K] row-major, f32 accumulation over 16-wide k tiles).
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <int ACCUMULATE>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ X, const float* __restrict__ W,
                                                       float* __restrict__ Y, int T, int N, int K, int ldx,
                                                       int ldy) {
  __shared__ float xs[TK][TM + 1];
  __shared__ float ws[TK][TN + 1];
  const int t0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // tx -> n, ty -> t
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      const int r = e / TK, k = e % TK;
      const int gt = t0 + r, gn = n0 + r, gk = k0 + k;
      xs[k][r] = (gt < T && gk < K) ? X[(size_t)gt * ldx + gk] : 0.0f;
      ws[k][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gt = t0 + ty + 16 * i;
    if (gt >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx + 16 * j;
      if (gn >= N) continue;
      float* y = Y + (size_t)gt * ldy + gn;
      if (ACCUMULATE) *y += acc[i][j];
      else *y = acc[i][j];
    }
  }
}

}  // namespace

JB_EXPORT int jb_gemm_f32(const float* X, const float* W, float* Y, int T, int N, int K, int ldx, int ldy,
                          int accumulate, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  JB_REFUSE(K <= 0, "gemm_f32: K must be positive, got %d", K);
  dim3 grid((N + TN - 1) / TN, (T + TM - 1) / TM);
  if (accumulate)
    gemm_f32_kernel<1><<<grid, 256, 0, stream>>>(X, W, Y, T, N, K, ldx, ldy);
  else
    gemm_f32_kernel<0><<<grid, 256, 0, stream>>>(X, W, Y, T, N, K, ldx, ldy);
  JB_CHECK_LAUNCH();
  return 0;
}
