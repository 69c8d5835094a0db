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

// Up to 16 tokens (decode steps, the head over a few wanted rows): the product streams the weights, so a block
// takes 32 weight rows in slices of 64 k (256 contiguous bytes a row and load: whole memory sectors), keeps the
// next slice's loads in flight in registers while it computes the present one, and 8 blocks share an SM.
// A thread owns one weight row and two tokens and adds its products in the order k = 0, 1, 2, ... with the
// same fused multiply-adds as the kernel above: the results are the same bit for bit, whichever kernel a
// step's size selects.
constexpr int SN = 32, SK = 64, ST = 16;

template <int ACCUMULATE>
__global__ void __launch_bounds__(256) gemm_f32_small_kernel(const float* __restrict__ X, const float* __restrict__ W,
                                                             float* __restrict__ Y, int T, int N, int K, int ldx,
                                                             int ldy) {
  __shared__ float ws[SK][SN + 1];   // [k][row]: a thread reads its row at one k, neighbours neighbouring banks
  __shared__ __align__(16) float xs[ST][SK];   // [token][k]: read by all rows' threads at once (a broadcast)
  const int n0 = blockIdx.x * SN;
  const int n = threadIdx.x % SN, tq = threadIdx.x / SN;   // tokens 2 tq, 2 tq + 1
  // this thread's loads: two 16-byte pieces of the weight slice, one of the token slice
  const int x_tok = (int)threadIdx.x / 16, c4 = (int)threadIdx.x % 16;
  const int w_row[2] = {x_tok, x_tok + 16};
  float4 wreg[2], xreg;
  auto fetch = [&](int k0) {
    const int k = k0 + 4 * c4;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int gn = n0 + w_row[i];
      wreg[i] = (gn < N && k < K) ? *reinterpret_cast<const float4*>(W + (size_t)gn * K + k)
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    xreg = (x_tok < T && k < K) ? *reinterpret_cast<const float4*>(X + (size_t)x_tok * ldx + k)
                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  };
  float acc[2] = {0.0f, 0.0f};
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += SK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ws[4 * c4 + 0][w_row[i]] = wreg[i].x;
      ws[4 * c4 + 1][w_row[i]] = wreg[i].y;
      ws[4 * c4 + 2][w_row[i]] = wreg[i].z;
      ws[4 * c4 + 3][w_row[i]] = wreg[i].w;
    }
    *reinterpret_cast<float4*>(&xs[x_tok][4 * c4]) = xreg;
    __syncthreads();
    if (k0 + SK < K) fetch(k0 + SK);
#pragma unroll 16
    for (int k = 0; k < SK; ++k) {
      const float w = ws[k][n];
      acc[0] = fmaf(xs[2 * tq][k], w, acc[0]);
      acc[1] = fmaf(xs[2 * tq + 1][k], w, acc[1]);
    }
    __syncthreads();
  }
  const int gn = n0 + n;
  if (gn < N) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int gt = 2 * tq + i;
      if (gt < T) {
        float* y = Y + (size_t)gt * ldy + gn;
        if (ACCUMULATE) *y += acc[i];
        else *y = acc[i];
      }
    }
  }
}

}  // namespace

JB_EXPORT int jb_gemm_f32(const float* X, const float* W, float* Y, int T, int N, int K, int ldx, int ldy,
                          int accumulate, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  JB_REFUSE(K <= 0, "gemm_f32: K must be positive, got %d", K);
  // rows of whole 16-byte vectors (K and the rows' starts) for the small kernel's loads
  if (T <= ST && K % 4 == 0 && ldx % 4 == 0 && (((uintptr_t)X | (uintptr_t)W) & 15) == 0) {
    const dim3 small((N + SN - 1) / SN);
    if (accumulate)
      gemm_f32_small_kernel<1><<<small, 256, 0, stream>>>(X, W, Y, T, N, K, ldx, ldy);
    else
      gemm_f32_small_kernel<0><<<small, 256, 0, stream>>>(X, W, Y, T, N, K, ldx, ldy);
    JB_CHECK_LAUNCH();
    return 0;
  }
  dim3 grid((N + TN - 1) / TN, (T + TM - 1) / TM);
  if (accumulate)
    gemm_f32_kernel<1><<<grid, 256, 0, stream>>>(X, W, Y, T, N, K, ldx, ldy);
  else
    gemm_f32_kernel<0><<<grid, 256, 0, stream>>>(X, W, Y, T, N, K, ldx, ldy);
  JB_CHECK_LAUNCH();
  return 0;
}
