// Embedding gather, RMSNorm, residual add, SwiGLU gating and a zero fill.
//
// The residual stream is float32 in both engine dtypes; norms read it and
// write the layer input in the engine dtype.  Statistics are float32.
// Formulas: crates/janus-engine/src/compute/shaders/embed.wgsl:46-62,
// activations.wgsl:20-35 (SiLU), activations.wgsl:81-133 (RMSNorm).
//
// Rows whose width is a multiple of 4 (8 for bf16 tables) move as 16-byte
// vectors; any other width takes the scalar kernels.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

// ---- 4-element vector access for float and bf16 ------------------------------
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ---- embedding ------------------------------------------------------------------
template <typename TT>
__global__ void embed_gather_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, const int* __restrict__ feedback,
                                    const int* __restrict__ token_slot) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0) id = feedback[token_slot[t]];  // the token sampled for this slot by the step before
  const TT* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  if ((H & 3) == 0) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) store4(o + i, load4(row + i));
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = jb::to_f32(row[i]);
  }
}

// A norm can also clear a scratch buffer for the part that runs after it (the target of a
// product whose slices of K meet by atomic adds): each block clears its share.
__device__ __forceinline__ void clear_slice(float4* __restrict__ clear, size_t n4) {
  if (clear == nullptr) return;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
    clear[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

// ---- RMSNorm: one block per output row; y = (x / sqrt(mean(x^2) + eps)) * gamma -----
// Rows of up to 2,048 floats take blocks of 128 threads, wider ones 256: what an SM has in flight is its
// resident blocks' rows, and sixteen small blocks hold twice the bytes of eight (34,808 rows of 2,048: 166 us
// with 256 threads).  The block's sum takes one barrier: every warp leaves its part, every thread adds the parts
// in the same order.
// NORM_CACHE float4 per thread stay in registers between the two passes: 4 cover rows of 2,048 (128 threads)
// and of 4,096 (256 threads) at 40 registers a thread, 8 cover rows of 8,192; wider rows are read twice.

template <int THREADS>
__device__ __forceinline__ float norm_block_sum(float v, float* scratch) {
  v = jb::warp_sum(v);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) t += scratch[w];
  return t;
}

template <typename TG, typename TO, int THREADS, int NORM_CACHE>
__global__ void __launch_bounds__(THREADS, NORM_CACHE == 4 ? 1280 / THREADS : 1) rmsnorm_vec_kernel(const float* __restrict__ x,
                                                             const int* __restrict__ row_index,
                                                             const TG* __restrict__ gamma, float eps,
                                                             TO* __restrict__ out, int H,
                                                             float4* __restrict__ clear, size_t clear_n4) {
  __shared__ float scratch[THREADS / 32];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  clear_slice(clear, clear_n4);
  const int r = blockIdx.x;
  const size_t src = row_index ? (size_t)row_index[r] : (size_t)r;
  const float* xr = x + src * H;
  const int n4 = H >> 2;
  float4 cache[NORM_CACHE];
  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < NORM_CACHE; ++c) {
    const int i = threadIdx.x + c * THREADS;
    if (i < n4) {
      cache[c] = load4(xr + 4 * i);
      ss += cache[c].x * cache[c].x + cache[c].y * cache[c].y + cache[c].z * cache[c].z + cache[c].w * cache[c].w;
    }
  }
  for (int i = threadIdx.x + NORM_CACHE * THREADS; i < n4; i += THREADS) {
    const float4 v = load4(xr + 4 * i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = norm_block_sum<THREADS>(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int c = 0; c < NORM_CACHE; ++c) {
    const int i = threadIdx.x + c * THREADS;
    if (i < n4) {
      const float4 g = load4(gamma + 4 * i), v = cache[c];
      store4(o + 4 * i, make_float4((v.x / rms) * g.x, (v.y / rms) * g.y, (v.z / rms) * g.z, (v.w / rms) * g.w));
    }
  }
  for (int i = threadIdx.x + NORM_CACHE * THREADS; i < n4; i += THREADS) {
    const float4 g = load4(gamma + 4 * i), v = load4(xr + 4 * i);
    store4(o + 4 * i, make_float4((v.x / rms) * g.x, (v.y / rms) * g.y, (v.z / rms) * g.z, (v.w / rms) * g.w));
  }
}

template <typename TG, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                               const TG* __restrict__ gamma, float eps, TO* __restrict__ out, int H,
                               float4* __restrict__ clear, size_t clear_n4) {
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  clear_slice(clear, clear_n4);
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
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) residual[i] += jb::to_f32(delta[i]);
}

// gate_up: [T, 2I] with gate in columns [0, I) and up in [I, 2I).
template <typename TT>
__global__ void swiglu_kernel(const TT* __restrict__ gate_up, TT* __restrict__ out, int I, size_t n) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / I, c = i % I;
  const float g = jb::to_f32(gate_up[t * 2 * I + c]);
  const float u = jb::to_f32(gate_up[t * 2 * I + I + c]);
  const float s = g * (1.0f / (1.0f + expf(-g)));
  out[i] = jb::from_f32<TT>(s * u);
}

// gate_up: float32 [T, ld], gate of feature c in column c, up in column up_col + c; out: bfloat16 [T, I].
// VEC = 4: four features a thread (I, ld and up_col multiples of 4, 16-byte aligned rows).
template <int VEC>
__global__ void swiglu_f32_bf16_kernel(const float* __restrict__ gate_up, bf16* __restrict__ out, int I, int ld, int up_col,
                                       size_t n) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= n) return;
  const size_t t = i / I, c = i % I;
  const float* row = gate_up + t * ld + c;
  float g[VEC], u[VEC];
  if (VEC == 4) {
    const float4 g4 = *reinterpret_cast<const float4*>(row), u4 = *reinterpret_cast<const float4*>(row + up_col);
    g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
    u[0] = u4.x; u[1] = u4.y; u[2] = u4.z; u[3] = u4.w;
  } else {
    g[0] = row[0];
    u[0] = row[up_col];
  }
  bf16 y[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) y[e] = __float2bfloat16_rn(g[e] * (1.0f / (1.0f + expf(-g[e]))) * u[e]);
  if (VEC == 4) {
    *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<const uint2*>(y);
  } else {
    out[i] = y[0];
  }
}

__global__ void zero_f32_kernel(float4* __restrict__ p, size_t n4) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) p[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

}  // namespace

// ids[t] < 0 means: take feedback[token_slot[t]] (both may be null if no id is negative).
JB_EXPORT int jb_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T, int H,
                              const int* feedback, const int* token_slot, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  jb::Launch cfg(dim3(T), dim3(threads), 0, stream);
  cudaError_t e;
  if (table_dtype == JB_F32)
    e = cudaLaunchKernelEx(&cfg.c, embed_gather_kernel<float>, (const float*)table, ids, out, H, feedback, token_slot);
  else if (table_dtype == JB_BF16)
    e = cudaLaunchKernelEx(&cfg.c, embed_gather_kernel<bf16>, (const bf16*)table, ids, out, H, feedback, token_slot);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)e;
}

// clear (may be null): clear_n floats (a multiple of 4, 16-byte aligned) that the kernel sets to zero besides.
JB_EXPORT int jb_rmsnorm(const float* x, const int* row_index, const void* gamma, int gamma_dtype, float eps,
                         void* out, int out_dtype, int rows, int H, float* clear, long long clear_n,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  JB_REFUSE(clear != nullptr && ((clear_n & 3) != 0 || ((uintptr_t)clear & 15) != 0),
            "rmsnorm: the buffer to clear is not made of whole 16-byte vectors");
  float4* clear4 = (float4*)clear;
  const size_t clear_n4 = clear ? (size_t)clear_n >> 2 : 0;
  const bool vec = (H & 3) == 0, narrow = H <= 2048, wide = H > 4096;
  jb::Launch cfg(dim3(rows), dim3(vec ? (narrow ? 128 : 256) : (H >= 512 ? 256 : 128)), 0, stream);
  cudaError_t e;
#define JB_LAUNCH_NORM(TG, TO)                                                                                          \
  e = !vec     ? cudaLaunchKernelEx(&cfg.c, rmsnorm_kernel<TG, TO>, x, row_index, (const TG*)gamma, eps, (TO*)out, H,   \
                                    clear4, clear_n4)                                                                   \
      : narrow ? cudaLaunchKernelEx(&cfg.c, rmsnorm_vec_kernel<TG, TO, 128, 4>, x, row_index, (const TG*)gamma, eps,    \
                                    (TO*)out, H, clear4, clear_n4)                                                      \
      : wide   ? cudaLaunchKernelEx(&cfg.c, rmsnorm_vec_kernel<TG, TO, 256, 8>, x, row_index, (const TG*)gamma, eps,    \
                                    (TO*)out, H, clear4, clear_n4)                                                      \
               : cudaLaunchKernelEx(&cfg.c, rmsnorm_vec_kernel<TG, TO, 256, 4>, x, row_index, (const TG*)gamma, eps,    \
                                    (TO*)out, H, clear4, clear_n4)
  if (gamma_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_NORM(float, float);
  else if (gamma_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_NORM(float, bf16);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_F32) JB_LAUNCH_NORM(bf16, float);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_NORM(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_NORM
  return (int)e;
}

JB_EXPORT int jb_residual_add(float* residual, const void* delta, int delta_dtype, long long n,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  jb::Launch cfg(dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream);
  cudaError_t e;
  if (delta_dtype == JB_F32)
    e = cudaLaunchKernelEx(&cfg.c, residual_add_kernel<float>, residual, (const float*)delta, (size_t)n);
  else if (delta_dtype == JB_BF16)
    e = cudaLaunchKernelEx(&cfg.c, residual_add_kernel<bf16>, residual, (const bf16*)delta, (size_t)n);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)e;
}

JB_EXPORT int jb_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream) {
  const size_t n = (size_t)T * I;
  if (n == 0) return 0;
  const int threads = 256;
  jb::Launch cfg(dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream);
  cudaError_t e;
  if (dtype == JB_F32)
    e = cudaLaunchKernelEx(&cfg.c, swiglu_kernel<float>, (const float*)gate_up, (float*)out, I, n);
  else if (dtype == JB_BF16)
    e = cudaLaunchKernelEx(&cfg.c, swiglu_kernel<bf16>, (const bf16*)gate_up, (bf16*)out, I, n);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)e;
}

// out[t, c] = silu(gate_up[t, c]) * gate_up[t, up_col + c] with float32 in (rows of ld floats) and bfloat16 out
// [T, I]: the activation of a gated product that was run as a plain product of the stacked gate and up rows.
JB_EXPORT int jb_swiglu_f32_to_bf16(const float* gate_up, int ld, int up_col, void* out, int T, int I, cudaStream_t stream) {
  const size_t n = (size_t)T * I;
  if (n == 0) return 0;
  JB_REFUSE(ld < up_col + I || up_col < I, "swiglu: rows of %d floats do not hold %d gate and %d up features from column %d",
            ld, I, I, up_col);
  const bool vec = I % 4 == 0 && ld % 4 == 0 && up_col % 4 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0;
  const size_t threads_needed = vec ? n / 4 : n;
  jb::Launch cfg(dim3((unsigned)((threads_needed + 255) / 256)), dim3(256), 0, stream);
  if (vec)
    return (int)cudaLaunchKernelEx(&cfg.c, swiglu_f32_bf16_kernel<4>, gate_up, (bf16*)out, I, ld, up_col, n);
  return (int)cudaLaunchKernelEx(&cfg.c, swiglu_f32_bf16_kernel<1>, gate_up, (bf16*)out, I, ld, up_col, n);
}

// Fill n floats with zero (n a multiple of 4, p 16-byte aligned): the target of a
// product whose slices of K meet by atomic adds.
JB_EXPORT int jb_zero_f32(float* p, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  JB_REFUSE((n & 3) != 0 || ((uintptr_t)p & 15) != 0, "zero_f32: %lld floats at %p are not whole 16-byte vectors", n, (void*)p);
  const size_t n4 = (size_t)n >> 2;
  jb::Launch cfg(dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, zero_f32_kernel, (float4*)p, n4);
}

// ---------------------------------------------------------------------------
// Weights of the bfloat16 products, laid out for streaming: the row-major [N, K] matrix is cut into tiles
// of 128 rows x 64 columns (16 KB, zero-padded at the edges), stored one after another as
// [row tile][k tile][128 rows][128 bytes], and inside a tile the 16-byte chunk c of row r lies at chunk
// position c ^ (r & 7): the 128-byte swizzle the tensor core reads from shared memory.  A product then
// fetches a tile as ONE contiguous 16 KB block (a TMA box over rows of 128 bytes, no swizzle in the copy)
// instead of 128 row pieces that lie 2 K bytes apart: contiguous blocks stream 6 - 9 % faster from HBM.
// ---------------------------------------------------------------------------
namespace {
__global__ void pack_weight_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int N, int K, int k_tiles,
                                   size_t n_chunks) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // destination chunk
  if (i >= n_chunks) return;
  const int p = (int)(i & 7), r = (int)((i >> 3) & 127);
  const size_t tile = i >> 10;
  const int kt = (int)(tile % k_tiles);
  const size_t rt = tile / k_tiles;
  const int c = p ^ (r & 7);
  const size_t row = rt * 128 + r;
  const int col = kt * 64 + c * 8;
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (row < (size_t)N && col < K) v = src[(row * K + col) >> 3];
  dst[i] = v;
}
}  // namespace

// src: [N, K] bf16 row-major, K a multiple of 8, 16-byte aligned; dst: ceil(N/128) * ceil(K/64) tiles of 16 KB.
JB_EXPORT int jb_pack_weight_bf16(const void* src, int N, int K, void* dst, cudaStream_t stream) {
  if (N <= 0 || K <= 0) return 0;
  JB_REFUSE(K % 8 != 0 || (((uintptr_t)src | (uintptr_t)dst) & 15), "pack_weight: K = %d must be a multiple of 8 and the tensors 16-byte aligned", K);
  const int k_tiles = (K + 63) / 64;
  const size_t n_chunks = (size_t)((N + 127) / 128) * k_tiles * 1024;
  pack_weight_kernel<<<(unsigned)((n_chunks + 255) / 256), 256, 0, stream>>>((const uint4*)src, (uint4*)dst, N, K, k_tiles,
                                                                             n_chunks);
  return (int)cudaGetLastError();
}
