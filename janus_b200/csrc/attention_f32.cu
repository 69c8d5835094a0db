// Float32 grouped-query attention over the paged cache, for prefill and decode
// alike: one warp per (token, query head); the token attends to the keys of
// its own sequence at positions [max(0, pos-window+1), pos] (window 0 = all).
// Formulas: crates/janus-engine/src/compute/shaders/attention.wgsl:96-115
// (kv head = h*nkv/nh, score = dot * scale), softmax.wgsl:29-50 (exp(s-max)/sum),
// attention.wgsl:170-185 (sum of p*v).  The softmax runs online over chunks of
// 32 keys that start at multiples of 32 of the absolute key index, so a
// token's result does not depend on how its sequence was cut into steps.
//
// Cache layout of one layer: [page][kv_head][PAGE][hd]; block_table[slot][i] is
// the page of keys [i*PAGE, (i+1)*PAGE) of the sequence in `slot`.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

// VEC: head sizes that are multiples of 4 (16-byte loads of the keys).
template <bool VEC>
__global__ void __launch_bounds__(WARPS * 32) attention_f32_kernel(
    const float* __restrict__ q, const float* __restrict__ k_cache, const float* __restrict__ v_cache,
    float* __restrict__ out, const int* __restrict__ block_table, const int* __restrict__ token_slot,
    const int* __restrict__ positions, int T, int nh, int nkv, int hd, int page_size, int max_pages,
    int window, float scale) {
  __shared__ __align__(16) float q_s[WARPS][MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)T * nh) return;  // whole warp leaves together
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int kvh = (h * nkv) / nh;
  const int pos = positions[t];
  const int* pages = block_table + (size_t)token_slot[t] * max_pages;
  const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  const float* qv = q + ((size_t)t * nh + h) * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = qv[d];
  __syncwarp();

  float m = -CUDART_INF_F, l = 0.0f;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int j = 0; j < MAX_HD / 32; ++j) acc[j] = 0.0f;

  for (int c0 = (kstart / 32) * 32; c0 <= pos; c0 += 32) {
    const int key = c0 + lane;
    const bool valid = key >= kstart && key <= pos;
    float s = -CUDART_INF_F;
    if (valid) {
      const int page = pages[key / page_size], row = key % page_size;
      const float* kr = k_cache + (((size_t)page * nkv + kvh) * page_size + row) * hd;
      float dot = 0.0f;
      if (VEC) {
        // 16-byte loads, eight in flight, consumed in the order d = 0, 1, 2, ... (the sum is the same as below)
        const float4* kr4 = reinterpret_cast<const float4*>(kr);
        const float4* q4 = reinterpret_cast<const float4*>(q_s[warp]);
#pragma unroll 8
        for (int d4 = 0; d4 < hd / 4; ++d4) {
          const float4 kk = kr4[d4], qq = q4[d4];
          dot = fmaf(qq.x, kk.x, dot);
          dot = fmaf(qq.y, kk.y, dot);
          dot = fmaf(qq.z, kk.z, dot);
          dot = fmaf(qq.w, kk.w, dot);
        }
      } else {
        for (int d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], kr[d], dot);
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, jb::warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.0f;
    const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first chunk
    l = l * corr + jb::warp_sum(p);
#pragma unroll
    for (int j = 0; j < MAX_HD / 32; ++j) acc[j] *= corr;
    const int n_keys = min(32, pos - c0 + 1);
    // eight value rows are loaded before their products are added, in key order (the same sums as one by one,
    // with eight rows' latencies at a time instead of one)
    const int first = max(c0, kstart) - c0;
    for (int kk0 = first; kk0 < n_keys; kk0 += 8) {
      float vreg[8][MAX_HD / 32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int key2 = c0 + min(kk0 + u, n_keys - 1);
        const int page = pages[key2 / page_size], row = key2 % page_size;
        const float* vr = v_cache + (((size_t)page * nkv + kvh) * page_size + row) * hd;
#pragma unroll
        for (int j = 0; j < MAX_HD / 32; ++j) {
          const int d = lane + 32 * j;
          vreg[u][j] = d < hd ? vr[d] : 0.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (kk0 + u < n_keys) {   // uniform across the warp
          const float pk = __shfl_sync(0xffffffffu, p, kk0 + u);
#pragma unroll
          for (int j = 0; j < MAX_HD / 32; ++j)
            if (lane + 32 * j < hd) acc[j] = fmaf(pk, vreg[u][j], acc[j]);
        }
      }
    }
    m = m_new;
  }
  float* o = out + ((size_t)t * nh + h) * hd;
#pragma unroll
  for (int j = 0; j < MAX_HD / 32; ++j) {
    const int d = lane + 32 * j;
    if (d < hd) o[d] = acc[j] / l;
  }
}

}  // namespace

JB_EXPORT int jb_attention_f32(const float* q, const float* k_cache, const float* v_cache, float* out,
                               const int* block_table, const int* token_slot, const int* positions, int T,
                               int nh, int nkv, int hd, int page_size, int max_pages, int window, float scale,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(hd > MAX_HD || hd <= 0, "attention_f32: head_dim %d is outside (0, %d]", hd, MAX_HD);
  JB_REFUSE(nkv <= 0 || nh % nkv != 0, "attention_f32: %d heads are not a multiple of %d kv heads", nh, nkv);
  const long long items = (long long)T * nh;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (hd % 4 == 0 && (((uintptr_t)k_cache) & 15) == 0)
    attention_f32_kernel<true><<<blocks, WARPS * 32, 0, stream>>>(q, k_cache, v_cache, out, block_table, token_slot,
                                                                  positions, T, nh, nkv, hd, page_size, max_pages,
                                                                  window, scale);
  else
    attention_f32_kernel<false><<<blocks, WARPS * 32, 0, stream>>>(q, k_cache, v_cache, out, block_table, token_slot,
                                                                   positions, T, nh, nkv, hd, page_size, max_pages,
                                                                   window, scale);
  JB_CHECK_LAUNCH();
  return 0;
}
