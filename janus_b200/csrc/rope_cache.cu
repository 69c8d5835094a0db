// Rotary position encoding of q and k (half-split pairs, table lookup at each
// token's own position) fused with the append of k (rotated) and v to the
// paged cache.  Formulas: crates/janus-engine/src/compute/shaders/rope.wgsl:55-76,
// update_cache.wgsl:44-64 (K is cached after rotation, V raw).
//
// qkv row layout: [q heads | k heads | v heads], each head `hd` wide.
// Cache layout of one layer: [page][kv_head][PAGE][hd]; dest[t] = page*PAGE + row.
// Head sizes that are a multiple of 8 move as 4-element vectors.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

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

// VEC = 4: four pairs per thread step (needs hd % 8 == 0 and 16-byte aligned rows); VEC = 1: one pair.
template <typename TI, typename TT, int VEC>
__global__ void rope_cache_kernel(const TI* __restrict__ qkv, int qkv_stride, TT* __restrict__ q_out,
                                  const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                  const int* __restrict__ dest, TT* __restrict__ k_cache,
                                  TT* __restrict__ v_cache, int nh, int nkv, int hd, int page_size,
                                  int rotate, int write_kv) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const int half = hd >> 1;
  const TI* row = qkv + (size_t)t * qkv_stride;
  const int pos = positions[t];
  const float* cs = cos_sin + (size_t)pos * half * 2;
  const int n_rot_heads = write_kv ? nh + nkv : nh;
  size_t kv_base = 0;
  if (write_kv) {
    const int d = dest[t];
    const int page = d / page_size, off = d % page_size;
    kv_base = ((size_t)page * nkv * page_size + off) * hd;  // + kvh * page_size * hd
  }
  const int steps = half / VEC;
  for (int idx = threadIdx.x; idx < n_rot_heads * steps; idx += blockDim.x) {
    const int head = idx / steps, i = (idx % steps) * VEC;
    TT* o = head < nh ? q_out + ((size_t)t * nh + head) * hd
                      : k_cache + kv_base + (size_t)(head - nh) * page_size * hd;
    if (VEC == 4) {
      const float4 x0 = load4(row + head * hd + i), x1 = load4(row + head * hd + i + half);
      float4 y0 = x0, y1 = x1;
      if (rotate) {
        const float4 a = load4(cs + 2 * i), b = load4(cs + 2 * i + 4);  // (c0 s0 c1 s1) (c2 s2 c3 s3)
        y0 = make_float4(x0.x * a.x - x1.x * a.y, x0.y * a.z - x1.y * a.w, x0.z * b.x - x1.z * b.y,
                         x0.w * b.z - x1.w * b.w);
        y1 = make_float4(x0.x * a.y + x1.x * a.x, x0.y * a.w + x1.y * a.z, x0.z * b.y + x1.z * b.x,
                         x0.w * b.w + x1.w * b.z);
      }
      store4(o + i, y0);
      store4(o + i + half, y1);
    } else {
      const float x0 = jb::to_f32(row[head * hd + i]), x1 = jb::to_f32(row[head * hd + i + half]);
      float y0 = x0, y1 = x1;
      if (rotate) {
        const float c = cs[2 * i], s = cs[2 * i + 1];
        y0 = x0 * c - x1 * s;
        y1 = x0 * s + x1 * c;
      }
      o[i] = jb::from_f32<TT>(y0);
      o[i + half] = jb::from_f32<TT>(y1);
    }
  }
  if (write_kv) {
    const TI* vrow = row + (size_t)(nh + nkv) * hd;
    for (int idx = threadIdx.x * VEC; idx < nkv * hd; idx += blockDim.x * VEC) {
      const int kvh = idx / hd, d = idx % hd;
      TT* o = v_cache + kv_base + (size_t)kvh * page_size * hd + d;
      if (VEC == 4) store4(o, load4(vrow + idx));
      else *o = jb::from_f32<TT>(jb::to_f32(vrow[idx]));
    }
  }
}

}  // namespace

// rotate = 0 leaves q and k unrotated (a mixer without rotary positions);
// write_kv = 0 rotates q only (a layer that reads another layer's cache).
// in_dtype is the dtype of qkv (float32 accumulators of the projection, or the
// engine dtype), out_dtype that of q_out and of the cache.
JB_EXPORT int jb_rope_cache_write(const void* qkv, int qkv_stride, int in_dtype, void* q_out, int out_dtype,
                                  const float* cos_sin, const int* positions, const int* dest, void* k_cache,
                                  void* v_cache, int T, int nh, int nkv, int hd, int page_size, int rotate,
                                  int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(hd % 2 != 0, "rope: head_dim %d must be even", hd);
  const bool vec = hd % 8 == 0 && qkv_stride % 4 == 0 &&
                   (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_sin) & 15) == 0;
  const int work = (nh + nkv) * (hd / 2) / (vec ? 4 : 1);
  jb::Launch cfg(dim3(T), dim3(work >= 512 ? 256 : 128), 0, stream);
  cudaError_t e;
#define JB_LAUNCH_ROPE(TI, TT)                                                                                   \
  e = vec ? cudaLaunchKernelEx(&cfg.c, rope_cache_kernel<TI, TT, 4>, (const TI*)qkv, qkv_stride, (TT*)q_out, cos_sin, \
                               positions, dest, (TT*)k_cache, (TT*)v_cache, nh, nkv, hd, page_size, rotate, write_kv) \
          : cudaLaunchKernelEx(&cfg.c, rope_cache_kernel<TI, TT, 1>, (const TI*)qkv, qkv_stride, (TT*)q_out, cos_sin, \
                               positions, dest, (TT*)k_cache, (TT*)v_cache, nh, nkv, hd, page_size, rotate, write_kv)
  if (in_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_ROPE(float, float);
  else if (in_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_ROPE(float, bf16);
  else if (in_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_ROPE(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_ROPE
  return (int)e;
}
