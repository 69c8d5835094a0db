// Rotary position encoding of q and k (half-split pairs, table lookup at each
// token's own position) fused with the append of k (rotated) and v to the
// paged cache.  Formulas: crates/janus-engine/src/compute/shaders/rope.wgsl:55-76,
// update_cache.wgsl:44-64 (K is cached after rotation, V raw).
//
// qkv row layout: [q heads | k heads | v heads], each head `hd` wide.
// Cache layout of one layer: [page][kv_head][PAGE][hd]; dest[t] = page*PAGE + row.
#include <stdio.h>

#include "common.cuh"

namespace {

template <typename TI, typename TT>
__global__ void rope_cache_kernel(const TI* __restrict__ qkv, int qkv_stride, TT* __restrict__ q_out,
                                  const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                  const int* __restrict__ dest, TT* __restrict__ k_cache,
                                  TT* __restrict__ v_cache, int nh, int nkv, int hd, int page_size,
                                  int rotate, int write_kv) {
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
  // rotation of q heads and k heads
  for (int idx = threadIdx.x; idx < n_rot_heads * half; idx += blockDim.x) {
    const int head = idx / half, i = idx % half;
    const float x0 = jb::to_f32(row[head * hd + i]);
    const float x1 = jb::to_f32(row[head * hd + i + half]);
    float y0 = x0, y1 = x1;
    if (rotate) {
      const float c = cs[2 * i], s = cs[2 * i + 1];
      y0 = x0 * c - x1 * s;
      y1 = x0 * s + x1 * c;
    }
    if (head < nh) {
      TT* o = q_out + ((size_t)t * nh + head) * hd;
      o[i] = jb::from_f32<TT>(y0);
      o[i + half] = jb::from_f32<TT>(y1);
    } else {
      TT* o = k_cache + kv_base + (size_t)(head - nh) * page_size * hd;
      o[i] = jb::from_f32<TT>(y0);
      o[i + half] = jb::from_f32<TT>(y1);
    }
  }
  if (write_kv) {
    const TI* vrow = row + (size_t)(nh + nkv) * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
      const int kvh = idx / hd, d = idx % hd;
      v_cache[kv_base + (size_t)kvh * page_size * hd + d] = jb::from_f32<TT>(jb::to_f32(vrow[idx]));
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
  const int work = (nh + nkv) * (hd / 2);
  const int threads = work >= 1024 ? 256 : 128;
#define JB_LAUNCH_ROPE(TI, TT)                                                                                  \
  rope_cache_kernel<TI, TT><<<T, threads, 0, stream>>>((const TI*)qkv, qkv_stride, (TT*)q_out, cos_sin, positions, \
                                                       dest, (TT*)k_cache, (TT*)v_cache, nh, nkv, hd, page_size,  \
                                                       rotate, write_kv)
  if (in_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_ROPE(float, float);
  else if (in_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_ROPE(float, __nv_bfloat16);
  else if (in_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_ROPE(__nv_bfloat16, __nv_bfloat16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_ROPE
  JB_CHECK_LAUNCH();
  return 0;
}
