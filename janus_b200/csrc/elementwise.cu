// Embedding gather, RMSNorm, residual add and SwiGLU gating.
//
// The residual stream is float32 in both engine dtypes; norms read it and
// write the layer input in the engine dtype.  Statistics are float32.
// Formulas: crates/janus-engine/src/compute/shaders/embed.wgsl:46-62,
// activations.wgsl:20-35 (SiLU), activations.wgsl:81-133 (RMSNorm).
#include <stdio.h>

#include "common.cuh"

namespace {

template <typename TT>
__global__ void embed_gather_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H) {
  const int t = blockIdx.x;
  const TT* row = table + (size_t)ids[t] * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = jb::to_f32(row[i]);
}

// One block per output row.  y = (x / sqrt(mean(x^2) + eps)) * gamma.
template <typename TG, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                               const TG* __restrict__ gamma, float eps, TO* __restrict__ out, int H) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t src = row_index ? (size_t)row_index[r] : (size_t)r;
  const float* xr = x + src * H;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = xr[i];
    ss += v * v;
  }
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = jb::from_f32<TO>((xr[i] / rms) * jb::to_f32(gamma[i]));
}

template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ residual, const TD* __restrict__ delta, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) residual[i] += jb::to_f32(delta[i]);
}

// gate_up: [T, 2I] with gate in columns [0, I) and up in [I, 2I).
template <typename TT>
__global__ void swiglu_kernel(const TT* __restrict__ gate_up, TT* __restrict__ out, int I, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / I, c = i % I;
  const float g = jb::to_f32(gate_up[t * 2 * I + c]);
  const float u = jb::to_f32(gate_up[t * 2 * I + I + c]);
  const float s = g * (1.0f / (1.0f + expf(-g)));
  out[i] = jb::from_f32<TT>(s * u);
}

}  // namespace

JB_EXPORT int jb_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T, int H,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == JB_F32)
    embed_gather_kernel<float><<<T, threads, 0, stream>>>((const float*)table, ids, out, H);
  else if (table_dtype == JB_BF16)
    embed_gather_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, H);
  else
    return JB_ERR_BAD_DTYPE;
  JB_CHECK_LAUNCH();
  return 0;
}

JB_EXPORT int jb_rmsnorm(const float* x, const int* row_index, const void* gamma, int gamma_dtype, float eps,
                         void* out, int out_dtype, int rows, int H, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define JB_LAUNCH_NORM(TG, TO) \
  rmsnorm_kernel<TG, TO><<<rows, threads, 0, stream>>>(x, row_index, (const TG*)gamma, eps, (TO*)out, H)
  if (gamma_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_NORM(float, float);
  else if (gamma_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_NORM(float, __nv_bfloat16);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_F32) JB_LAUNCH_NORM(__nv_bfloat16, float);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_NORM(__nv_bfloat16, __nv_bfloat16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_NORM
  JB_CHECK_LAUNCH();
  return 0;
}

JB_EXPORT int jb_residual_add(float* residual, const void* delta, int delta_dtype, long long n,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  if (delta_dtype == JB_F32)
    residual_add_kernel<float><<<blocks, threads, 0, stream>>>(residual, (const float*)delta, (size_t)n);
  else if (delta_dtype == JB_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(residual, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return JB_ERR_BAD_DTYPE;
  JB_CHECK_LAUNCH();
  return 0;
}

JB_EXPORT int jb_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream) {
  const size_t n = (size_t)T * I;
  if (n == 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  if (dtype == JB_F32)
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, n);
  else if (dtype == JB_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I, n);
  else
    return JB_ERR_BAD_DTYPE;
  JB_CHECK_LAUNCH();
  return 0;
}
