// bfloat16 grouped-query attention over the paged cache, compiled for one head
// size (-DJB_HEAD_DIM=..., a multiple of 8 up to 256; in shared memory rows are
// zero-padded to the next multiple of 16, the k extent of one MMA).
//
// Rows of a tile are (token, query head of one kv group) pairs, so the query
// heads that share a kv head share every K/V tile that is read.  Scores and
// the online softmax are float32 (exp2 of log2e-scaled scores); P is rounded to
// bf16 for the P.V product, whose accumulators are float32.
//   prefill:  one CTA per (row tile of 64, kv head, sequence); each of 4 warps owns 16 rows
//             and walks the causal range of 64-key pages.
//   decode:   one CTA per (sequence, kv head x row block of 16 heads, split of the keys); the
//             4 warps share the rows and each takes 16 keys of every page; partial
//             (max, sum, out) meet in shared memory, and across splits in a scratch buffer
//             reduced by a second kernel.
// Formulas: crates/janus-engine/src/compute/shaders/attention.wgsl:96-115,170-185 and
// softmax.wgsl:29-50; kv head of query head h is floor(h * nkv / nh).
//
// Cache layout of one layer: [page][kv_head][64][HD]; block_table[seq][i] is the
// page of keys [64 i, 64 i + 64).
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

#ifndef JB_HEAD_DIM
#define JB_HEAD_DIM 128
#endif

namespace {

typedef __nv_bfloat16 bf16;

constexpr int HD = JB_HEAD_DIM;
static_assert(HD % 8 == 0 && HD >= 8 && HD <= 256, "head size must be a multiple of 8 in [8, 256]");
constexpr int HDP = (HD + 15) / 16 * 16;  // head size as the MMAs see it
constexpr int PAGE = 64;
constexpr int LD = HDP + 8;           // padded smem row: an odd number of 16-byte chunks, conflict-free ldmatrix
constexpr int CHUNKS = HD / 8;        // 16-byte chunks per row that exist in global memory
constexpr int THREADS = 128;
constexpr int KV_TILE = PAGE * LD;    // elements
constexpr float LOG2E = 1.4426950408889634f;
// K/V pages in the decode kernel's ring: picked at the launch from 2, 3 and 5 (`decode_stages_for`);
// JB_DECODE_STAGES forces one depth.
#ifndef JB_DECODE_STAGES
#define JB_DECODE_STAGES 0
#endif
constexpr int RED_LD = HD + 8;                   // row stride (floats) of the warps' exchange of partial outputs

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0 fills the 16 bytes with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
#ifndef JB_KV_EVICT_FIRST
#define JB_KV_EVICT_FIRST 1   // a decode step's K/V pages (read once a step) are the first to leave L2: +1.2 % decode
#endif
// 16 bytes of a cached page into shared memory, optionally with an evict-first L2 policy.
__device__ __forceinline__ void cp_async16_kv(void* dst, const void* src, uint64_t policy) {
#if JB_KV_EVICT_FIRST
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "l"(policy)
               : "memory");
#else
  (void)policy;
  cp_async16(dst, src, true);
#endif
}
__device__ __forceinline__ uint64_t kv_policy() {
  uint64_t p = 0;
#if JB_KV_EVICT_FIRST
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
#endif
  return p;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy one [64, HD] page tile into padded shared memory (all 128 threads).
__device__ __forceinline__ void load_page(bf16* dst, const bf16* src) {
  for (int ch = threadIdx.x; ch < PAGE * CHUNKS; ch += THREADS) {
    const int row = ch / CHUNKS, col = ch % CHUNKS;
    cp_async16(dst + row * LD + col * 8, src + (size_t)row * HD + col * 8, true);
  }
}

// The columns [HD, HDP) of `rows` padded rows are never written by a load: zero them once.
__device__ __forceinline__ void zero_pad_columns(bf16* base, int rows) {
  if constexpr (HDP != HD) {
    constexpr int PAD = HDP - HD;
    for (int i = threadIdx.x; i < rows * PAD; i += THREADS)
      base[(i / PAD) * LD + HD + i % PAD] = __float2bfloat16_rn(0.0f);
  }
}

// Per-warp flash-attention state for 16 rows: thread (g = lane/4, c = lane%4)
// owns rows g and g + 8.
struct RowState {
  float m[2], l[2];
  float o[HDP / 8][4];
  __device__ __forceinline__ void init() {
    m[0] = m[1] = -CUDART_INF_F;
    l[0] = l[1] = 0.0f;
#pragma unroll
    for (int j = 0; j < HDP / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
  }
};

// S = Q[16 rows] . K[NT*8 keys]^T for the keys starting at `k_tile` (smem, padded rows).
template <int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const bf16* q_rows, const bf16* k_tile, int lane) {
#pragma unroll
  for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
  for (int ks = 0; ks < HDP / 16; ++ks) {
    uint32_t a[4];
    ldmatrix_x4(a, q_rows + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b[4];
      const int key = j * 8 + (lane & 7) + ((lane >> 4) << 3);
      ldmatrix_x4(b, k_tile + key * LD + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[j], a, b[0], b[1]);
      mma_bf16(s[j + 1], a, b[2], b[3]);
    }
  }
}

// Online-softmax update with the scores of NT*8 keys, then O += P . V.
// key_pos0: position of key column 0; row_pos[2]: positions of this thread's rows
// (negative = row unused); keys outside [row_lo, row_pos] are masked.
template <int NT>
__device__ __forceinline__ void softmax_pv(RowState& st, float (&s)[NT][4], const bf16* v_tile, int key_pos0,
                                           const int (&row_pos)[2], const int (&row_lo)[2], float scale_log2,
                                           int lane) {
  const int c = lane & 3;
  float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const int kp = key_pos0 + j * 8 + 2 * c + (e & 1);
      const bool ok = kp <= row_pos[r] && kp >= row_lo[r];
      s[j][e] = ok ? s[j][e] * scale_log2 : -CUDART_INF_F;
      mx[r] = fmaxf(mx[r], s[j][e]);
    }
  }
  float corr[2], m_use[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(st.m[r], mx[r]);
    m_use[r] = m_new == -CUDART_INF_F ? 0.0f : m_new;
    corr[r] = exp2f(st.m[r] - m_use[r]);  // 0 when nothing was seen before
    st.m[r] = m_new;
    st.l[r] *= corr[r];
  }
#pragma unroll
  for (int j = 0; j < HDP / 8; ++j) {
    st.o[j][0] *= corr[0];
    st.o[j][1] *= corr[0];
    st.o[j][2] *= corr[1];
    st.o[j][3] *= corr[1];
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(s[j][e] - m_use[e >> 1]);
      s[j][e] = p;
      st.l[e >> 1] += p;
    }
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int j = 0; j < HDP / 8; j += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, v_tile + (kk * 16 + (lane & 15)) * LD + j * 8 + (lane >> 4) * 8);
      mma_bf16(st.o[j], a, b[0], b[1]);
      mma_bf16(st.o[j + 1], a, b[2], b[3]);
    }
  }
}

// ------------------------------- prefill ------------------------------------
__global__ void __launch_bounds__(THREADS) prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    bf16* __restrict__ out, const int* __restrict__ block_table, const int* __restrict__ q_start,
    const int* __restrict__ kv_len, int nh, int nkv, int max_pages, int window, float scale_log2) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [64][LD]
  bf16* kv_s = q_s + 64 * LD;                     // [2 stages][K, V][64][LD]
  const int G = nh / nkv;
  const int tpt = 64 / G;                         // tokens per tile
  // kv heads run fastest in the order CTAs are handed out and tiles go backwards: across all heads the
  // longest key ranges start first
  const int seq = blockIdx.z, kvh = blockIdx.x, tile = gridDim.y - 1 - blockIdx.y;
  const int qs = q_start[seq], q_len = q_start[seq + 1] - qs;
  const int tok0 = tile * tpt;
  if (tok0 >= q_len) return;
  const int n_tok = min(tpt, q_len - tok0);
  const int len = kv_len[seq];
  const int pos0 = len - q_len + tok0;            // position of the tile's first token
  const int* pages = block_table + (size_t)seq * max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  zero_pad_columns(q_s, 64 + 4 * PAGE);  // q tile and the four K/V tiles lie back to back
  // Q rows: r -> (token tok0 + r / G, head kvh * G + r % G)
  for (int ch = threadIdx.x; ch < 64 * CHUNKS; ch += THREADS) {
    const int r = ch / CHUNKS, col = ch % CHUNKS;
    const int tl = r / G;
    const bool valid = tl < n_tok;
    const bf16* src = q + ((size_t)(qs + tok0 + (valid ? tl : 0)) * nh + kvh * G + r % G) * HD + col * 8;
    cp_async16(q_s + r * LD + col * 8, src, valid);
  }
  const int pos_last = pos0 + n_tok - 1;
  const int kb_end = pos_last / PAGE;
  const int kb_start = window > 0 ? max(0, pos0 - window + 1) / PAGE : 0;
  auto issue = [&](int kb, int stage) {
    const size_t page = (size_t)pages[kb];
    const size_t off = (page * nkv + kvh) * PAGE * HD;
    load_page(kv_s + (size_t)stage * 2 * KV_TILE, k_cache + off);
    load_page(kv_s + (size_t)stage * 2 * KV_TILE + KV_TILE, v_cache + off);
  };
  issue(kb_start, 0);
  cp_async_commit();

  int row_pos[2], row_lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + (lane >> 2) + 8 * r;
    const int tl = row / G;
    row_pos[r] = tl < n_tok ? pos0 + tl : -1;
    row_lo[r] = window > 0 ? max(0, row_pos[r] - window + 1) : 0;
  }
  RowState st;
  st.init();
  for (int kb = kb_start; kb <= kb_end; ++kb) {
    const int stage = (kb - kb_start) & 1;
    if (kb < kb_end) {
      issue(kb + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* k_tile = kv_s + (size_t)stage * 2 * KV_TILE;
    float s[8][4];
    qk_product<8>(s, q_s + warp * 16 * LD, k_tile, lane);
    softmax_pv<8>(st, s, k_tile + KV_TILE, kb * PAGE, row_pos, row_lo, scale_log2, lane);
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = st.l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = warp * 16 + (lane >> 2) + 8 * r;
    const int tl = row / G;
    if (tl < n_tok) {
      const float inv = 1.0f / l;
      bf16* o = out + ((size_t)(qs + tok0 + tl) * nh + kvh * G + row % G) * HD + 2 * (lane & 3);
#pragma unroll
      for (int j = 0; j < HDP / 8; ++j)
        if (j * 8 < HD)
          *reinterpret_cast<uint32_t*>(o + j * 8) = pack_bf16(st.o[j][2 * r] * inv, st.o[j][2 * r + 1] * inv);
    }
  }
}

// ------------------------------- decode -------------------------------------
// Optional fused input of the decode kernel: instead of rotated bf16 queries and a cache that
// already holds the new token, the q/k/v projection's float32 output [seq][q heads | k heads | v heads];
// the kernel rotates q and k at the token's position (cos_sin null = no rotation), appends k and v
// to the cache (write_kv) and uses them.  qkv == nullptr turns this off.
struct FusedInput {
  const float* qkv;
  int qkv_stride;
  const float* cos_sin;  // [positions][HD / 2][2]
  const int* dest;       // [seq] cache row (page * 64 + row) of the new token
  bf16* k_out;
  bf16* v_out;
  int write_kv;
};

__device__ __forceinline__ void rotate_pair(float x0, float x1, const float* cs, int i, float& y0, float& y1) {
  if (cs == nullptr) {
    y0 = x0;
    y1 = x1;
    return;
  }
  const float c = cs[2 * i], s = cs[2 * i + 1];
  y0 = x0 * c - x1 * s;
  y1 = x0 * s + x1 * c;
}

// part_o: [seq][head][split][HD] float32 (unnormalised), part_ml: [seq][head][split][2] (max, sum).
template <int DECODE_STAGES>
__global__ void __launch_bounds__(THREADS) decode_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const int* __restrict__ block_table, const int* __restrict__ kv_len, int nh, int nkv, int max_pages,
    int window, float scale_log2, int n_splits, FusedInput fused) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  jb::pdl_launch_dependents();
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [16][LD]
  bf16* new_kv = q_s + 16 * LD;                   // [2][LD]: the new token's rotated key and its value (fused input)
  bf16* kv_s = new_kv + 2 * LD;                   // [DECODE_STAGES][K, V][64][LD]; reused as float scratch at the end
  const int G = nh / nkv;
  const int n_rb = (G + 15) / 16;
  const int seq = blockIdx.x, kvh = blockIdx.y / n_rb, rb = blockIdx.y % n_rb, split = blockIdx.z;
  const int g0 = rb * 16, n_rows = min(16, G - g0);
  const int len = kv_len[seq];
  const int pos = len - 1;                        // the one new token is the sequence's last
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kb_first = lo / PAGE, kb_last = pos / PAGE;
  const int n_blocks = kb_last - kb_first + 1;
  // the pages are cut evenly: split s walks pages [s n / S, (s + 1) n / S), so that no split is left
  // without pages while another walks a rounded-up share
  const int kb_start = kb_first + (int)(((long long)split * n_blocks) / n_splits);
  const int kb_end = kb_first + (int)(((long long)(split + 1) * n_blocks) / n_splits) - 1;
  const int* pages = block_table + (size_t)seq * max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  RowState st;
  st.init();
  // The lengths, the block table and the cached pages were written before this step's kernels began, so
  // the first pages are asked for BEFORE the wait on the kernel that produces q: their latency hides
  // behind that kernel's end.  The one page that may be written in this step (the last one, which takes
  // the new token from the kernel before this one, unless this kernel appends it itself) waits.
  const bool appends_here = fused.qkv != nullptr && fused.write_kv;
  const bool early = appends_here || kb_start + DECODE_STAGES - 2 < kb_last;
  // Every warp loads, waits for and computes ITS OWN 16 keys of each page, so the ring needs no barrier of
  // the whole CTA: a warp asks for its rows of the page after next as soon as it is done with its rows of
  // this one, whatever the other warps are doing.
  const uint64_t kv_pol = kv_policy();
  auto issue = [&](int kb, int stage) {
    const size_t page = (size_t)pages[kb];
    const size_t off = ((page * nkv + kvh) * PAGE + warp * 16) * HD;
    bf16* k_rows = kv_s + (size_t)stage * 2 * KV_TILE + warp * 16 * LD;
    for (int ch = lane; ch < 16 * CHUNKS; ch += 32) {
      const int row = ch / CHUNKS, col = ch % CHUNKS;
      cp_async16_kv(k_rows + row * LD + col * 8, k_cache + off + (size_t)row * HD + col * 8, kv_pol);
      cp_async16_kv(k_rows + KV_TILE + row * LD + col * 8, v_cache + off + (size_t)row * HD + col * 8, kv_pol);
    }
  };
  // ring of DECODE_STAGES pages: DECODE_STAGES - 1 loads are in flight while one page is computed
  auto issue_first_pages = [&]() {
#pragma unroll
    for (int s = 0; s < DECODE_STAGES - 1; ++s) {
      if (kb_start + s <= kb_end) issue(kb_start + s, s);
      cp_async_commit();  // a group per stage, empty or not, keeps the group count in step with the pages
    }
  };
  if (kb_start <= kb_end && early) issue_first_pages();
  jb::pdl_wait();
  if (kb_start <= kb_end) {
    zero_pad_columns(q_s, 16 + 2 + 2 * DECODE_STAGES * PAGE);
    const bool patch_new = appends_here && kb_end == kb_last;  // this CTA sees the new key
    if (!early) issue_first_pages();
    if (fused.qkv == nullptr) {
      // rotated queries of the kernel before: plain loads, visible after the loop's first barrier
      for (int ch = threadIdx.x; ch < 16 * CHUNKS; ch += THREADS) {
        const int r = ch / CHUNKS, col = ch % CHUNKS;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)seq * nh + kvh * G + g0 + r) * HD + col * 8);
        *reinterpret_cast<uint4*>(q_s + r * LD + col * 8) = v;
      }
    }
    if (fused.qkv != nullptr) {
      // (after the first page loads are in flight, so that the rotation hides behind them)
      // q (and the new k, v) come as the projection's float32 accumulators: rotate here
      constexpr int HALF = HD / 2;
      const float* row = fused.qkv + (size_t)seq * fused.qkv_stride;
      const float* cs = fused.cos_sin ? fused.cos_sin + (size_t)pos * HD : nullptr;  // [HALF][2] at this position
      for (int idx = threadIdx.x; idx < n_rows * HALF; idx += THREADS) {  // the rows that exist
        const int r = idx / HALF, i = idx % HALF;
        const float* x = row + (size_t)(kvh * G + g0 + r) * HD;
        float y0, y1;
        rotate_pair(x[i], x[i + HALF], cs, i, y0, y1);
        q_s[r * LD + i] = __float2bfloat16_rn(y0);
        q_s[r * LD + i + HALF] = __float2bfloat16_rn(y1);
      }
      for (int idx = n_rows * HD + threadIdx.x; idx < 16 * HD; idx += THREADS)  // the rest of the 16-row tile
        q_s[(idx / HD) * LD + idx % HD] = __float2bfloat16_rn(0.0f);
      if (patch_new) {
        const float* kx = row + (size_t)(nh + kvh) * HD;
        const float* vx = row + (size_t)(nh + nkv + kvh) * HD;
        const int dst = fused.dest[seq];
        const size_t g_off = (((size_t)(dst / PAGE) * nkv + kvh) * PAGE + dst % PAGE) * HD;
        for (int i = threadIdx.x; i < HALF; i += THREADS) {
          float y0, y1;
          rotate_pair(kx[i], kx[i + HALF], cs, i, y0, y1);
          const bf16 k0 = __float2bfloat16_rn(y0), k1 = __float2bfloat16_rn(y1);
          const bf16 v0 = __float2bfloat16_rn(vx[i]), v1 = __float2bfloat16_rn(vx[i + HALF]);
          new_kv[i] = k0; new_kv[i + HALF] = k1;
          new_kv[LD + i] = v0; new_kv[LD + i + HALF] = v1;
          if (rb == 0) {  // one CTA per (sequence, kv head) appends to the cache for the steps to come
            fused.k_out[g_off + i] = k0; fused.k_out[g_off + i + HALF] = k1;
            fused.v_out[g_off + i] = v0; fused.v_out[g_off + i + HALF] = v1;
          }
        }
      }
    }
    int row_pos[2], row_lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      row_pos[r] = ((lane >> 2) + 8 * r) < n_rows ? pos : -1;
      row_lo[r] = lo;
    }
    __syncthreads();  // q (and the new key and value) are in shared memory for every warp
    for (int kb = kb_start; kb <= kb_end; ++kb) {
      const int stage = (kb - kb_start) % DECODE_STAGES;
      if (kb + DECODE_STAGES - 1 <= kb_end)
        issue(kb + DECODE_STAGES - 1, (kb - kb_start + DECODE_STAGES - 1) % DECODE_STAGES);
      cp_async_commit();
      cp_async_wait<DECODE_STAGES - 1>();  // everything but the newest DECODE_STAGES - 1 groups: page kb has landed
      __syncwarp();
      bf16* k_tile = kv_s + (size_t)stage * 2 * KV_TILE;
      if (patch_new && kb == kb_last && warp == (pos % PAGE) / 16) {
        // the page as loaded holds a stale row at the new position: the warp that owns the row puts the
        // new key and value there
        const int r = pos % PAGE;
        for (int i = lane; i < 2 * HD; i += 32) {
          const int which = i / HD, d = i % HD;
          k_tile[which * KV_TILE + r * LD + d] = new_kv[which * LD + d];
        }
        __syncwarp();
      }
      // this warp's 16 keys of the page
      float s[2][4];
      qk_product<2>(s, q_s, k_tile + warp * 16 * LD, lane);
      softmax_pv<2>(st, s, k_tile + KV_TILE + warp * 16 * LD, kb * PAGE + warp * 16, row_pos, row_lo,
                    scale_log2, lane);
      __syncwarp();  // the warp is done with its rows of this stage before its next loads overwrite them
    }
  }
  __syncthreads();  // every warp has left the ring: its memory becomes the exchange buffer
  // ---- the four warps' partial results meet in shared memory ----
  float* red_o = reinterpret_cast<float*>(kv_s);           // [4][16][RED_LD]: padded rows, no 8-way bank conflicts
  float* red_ml = red_o + 4 * 16 * RED_LD;                  // [4][16][2]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = st.l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = (lane >> 2) + 8 * r;
    if ((lane & 3) == 0) {
      red_ml[(warp * 16 + row) * 2] = st.m[r];
      red_ml[(warp * 16 + row) * 2 + 1] = l;
    }
#pragma unroll
    for (int j = 0; j < HDP / 8; ++j) {
      if (j * 8 < HD) {
        float* o = red_o + ((size_t)(warp * 16 + row)) * RED_LD + j * 8 + 2 * (lane & 3);
        o[0] = st.o[j][2 * r];
        o[1] = st.o[j][2 * r + 1];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_rows * HD; idx += THREADS) {
    const int row = idx / HD, d = idx % HD;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, red_ml[(w * 16 + row) * 2]);
    const float m_use = m == -CUDART_INF_F ? 0.0f : m;
    float o = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(red_ml[(w * 16 + row) * 2] - m_use);
      o += red_o[((size_t)(w * 16 + row)) * RED_LD + d] * f;
      l += red_ml[(w * 16 + row) * 2 + 1] * f;
    }
    const int head = kvh * G + g0 + row;
    if (n_splits == 1) {
      out[((size_t)seq * nh + head) * HD + d] = __float2bfloat16_rn(o / l);
    } else {
      const size_t base = ((size_t)seq * nh + head) * n_splits + split;
      part_o[base * HD + d] = o;
      if (d == 0) {
        part_ml[base * 2] = m;
        part_ml[base * 2 + 1] = l;
      }
    }
  }
}

__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      bf16* __restrict__ out, int n_splits) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const size_t item = blockIdx.x;  // seq * nh + head
  const float* ml = part_ml + item * n_splits * 2;
  float m = -CUDART_INF_F;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float o = 0.0f, l = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
      const float f = exp2f(ml[2 * s] - m);  // a split without keys has max -inf and weighs 0
      o += part_o[(item * n_splits + s) * HD + d] * f;
      l += ml[2 * s + 1] * f;
    }
    out[item * HD + d] = __float2bfloat16_rn(o / l);
  }
}

constexpr int PREFILL_SMEM = (64 * LD + 4 * KV_TILE) * 2;
constexpr int DECODE_RED_BYTES = (4 * 16 * RED_LD + 4 * 16 * 2) * 4;
constexpr int decode_smem(int stages) {
  const int kv = 2 * stages * KV_TILE * 2;
  return (16 + 2) * LD * 2 + (kv > DECODE_RED_BYTES ? kv : DECODE_RED_BYTES);
}
constexpr int SMEM_PER_SM = 228 * 1024;   // of which every resident CTA takes 1 KB for the system besides its own
constexpr int ctas_per_sm(int stages) { return SMEM_PER_SM / (decode_smem(stages) + 1024); }

// How deep the ring of the decode kernel is for a launch of `ctas` CTAs.  Three pages (two loads in flight
// while one page is computed) serve every head size.  Small heads move few bytes per page and per warp, so
// what pays depends on how many CTAs there are: more than fit the SMs at once run fastest with a ring of two
// pages (five CTAs an SM at head size 64 instead of three: 64 sequences of 704 keys 24.0 -> 18.4 us), few CTAs
// of many pages with a ring of five (8 sequences of 2,816 keys 14.3 -> 12.2 us).
int decode_stages_for(long long ctas, int pages_per_cta) {
  if (JB_DECODE_STAGES) return JB_DECODE_STAGES;
  if (HD > 64) return 3;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long fit3 = (long long)sms * ctas_per_sm(3);
  const long long fit5 = (long long)sms * ctas_per_sm(5);
  if (ctas > fit3) return 2;
  if (ctas <= fit5 && pages_per_cta >= 8) return 5;
  return 3;
}

template <int ST>
cudaError_t decode_go(dim3 grid, cudaStream_t stream, bool pdl, const bf16* q, const bf16* k_cache, const bf16* v_cache,
                      bf16* out, float* part_o, float* part_ml, const int* block_table, const int* kv_len, int nh,
                      int nkv, int max_pages, int window, float scale_log2, int n_splits, const FusedInput& fused) {
  static bool configured = false;   // one flag per ring depth
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, decode_smem(ST));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  if (pdl) {
    jb::Launch cfg(grid, dim3(THREADS), decode_smem(ST), stream);
    return cudaLaunchKernelEx(&cfg.c, decode_kernel<ST>, q, k_cache, v_cache, out, part_o, part_ml, block_table, kv_len,
                              nh, nkv, max_pages, window, scale_log2, n_splits, fused);
  }
  decode_kernel<ST><<<grid, THREADS, decode_smem(ST), stream>>>(q, k_cache, v_cache, out, part_o, part_ml, block_table,
                                                               kv_len, nh, nkv, max_pages, window, scale_log2, n_splits,
                                                               fused);
  return cudaGetLastError();
}

// The decode kernel with the ring depth that suits the launch (`max_pages` bounds a sequence's pages).
cudaError_t decode_dispatch(dim3 grid, cudaStream_t stream, bool pdl, const bf16* q, const bf16* k_cache,
                            const bf16* v_cache, bf16* out, float* part_o, float* part_ml, const int* block_table,
                            const int* kv_len, int nh, int nkv, int max_pages, int window, float scale_log2,
                            int n_splits, const FusedInput& fused) {
  const long long ctas = (long long)grid.x * grid.y * grid.z;
  const int stages = decode_stages_for(ctas, max(1, max_pages / max(1, n_splits)));
#define JB_DECODE_GO(ST)                                                                                      \
  return decode_go<ST>(grid, stream, pdl, q, k_cache, v_cache, out, part_o, part_ml, block_table, kv_len, nh, nkv, \
                       max_pages, window, scale_log2, n_splits, fused)
  switch (stages) {
    case 2: JB_DECODE_GO(2);
    case 5: JB_DECODE_GO(5);
#if JB_DECODE_STAGES != 0 && JB_DECODE_STAGES != 2 && JB_DECODE_STAGES != 3 && JB_DECODE_STAGES != 5
    case JB_DECODE_STAGES: JB_DECODE_GO(JB_DECODE_STAGES);
#endif
    default: JB_DECODE_GO(3);
  }
#undef JB_DECODE_GO
}

}  // namespace

JB_EXPORT int jb_attention_bf16_head_dim() { return HD; }

JB_EXPORT int jb_attention_bf16_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* block_table, const int* q_start, const int* kv_len,
                                        int n_seqs, int max_q_len, int nh, int nkv, int hd, int page_size,
                                        int max_pages, int window, float scale, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  JB_REFUSE(hd != HD, "attention_bf16: built for head_dim %d, called with %d", HD, hd);
  JB_REFUSE(page_size != PAGE, "attention_bf16: page size %d (need %d)", page_size, PAGE);
  JB_REFUSE(nkv <= 0 || nh % nkv != 0, "attention_bf16: %d heads are not a multiple of %d kv heads", nh, nkv);
  const int G = nh / nkv;
  JB_REFUSE(G > 64, "attention_bf16 prefill: more than 64 query heads per kv head (%d)", G);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tpt = 64 / G;
  dim3 grid(nkv, (max_q_len + tpt - 1) / tpt, n_seqs);
  jb::Launch cfg(grid, dim3(THREADS), PREFILL_SMEM, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, prefill_kernel, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                 (bf16*)out, block_table, q_start, kv_len, nh, nkv, max_pages, window,
                                 scale * LOG2E);
}

// Scratch (when n_splits > 1): part_o float32 [n_seqs * nh * n_splits * hd], part_ml float32
// [n_seqs * nh * n_splits * 2].
namespace {
int decode_launch(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                  const int* block_table, const int* kv_len, int n_seqs, int nh, int nkv, int hd, int page_size,
                  int max_pages, int window, float scale, int n_splits, const FusedInput& fused,
                  cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(hd != HD, "attention_bf16: built for head_dim %d, called with %d", HD, hd);
  JB_REFUSE(page_size != PAGE, "attention_bf16: page size %d (need %d)", page_size, PAGE);
  JB_REFUSE(nkv <= 0 || nh % nkv != 0, "attention_bf16: %d heads are not a multiple of %d kv heads", nh, nkv);
  JB_REFUSE(n_splits < 1 || (n_splits > 1 && (!part_o || !part_ml)), "attention_bf16 decode: bad split setup");
  const int G = nh / nkv;
  const int n_rb = (G + 15) / 16;
  dim3 grid(n_seqs, nkv * n_rb, n_splits);
  cudaError_t le = decode_dispatch(grid, stream, true, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                   (bf16*)out, part_o, part_ml, block_table, kv_len, nh, nkv, max_pages, window,
                                   scale * LOG2E, n_splits, fused);
  if (le != cudaSuccess) return (int)le;
  if (n_splits > 1) {
    jb::Launch cfg2(dim3(n_seqs * nh), dim3(HD >= 128 ? 128 : 64), 0, stream);
    le = cudaLaunchKernelEx(&cfg2.c, decode_combine_kernel, (const float*)part_o, (const float*)part_ml, (bf16*)out,
                            n_splits);
    if (le != cudaSuccess) return (int)le;
  }
  return 0;
}
}  // namespace

JB_EXPORT int jb_attention_bf16_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       float* part_o, float* part_ml, const int* block_table,
                                       const int* kv_len, int n_seqs, int nh, int nkv, int hd, int page_size,
                                       int max_pages, int window, float scale, int n_splits,
                                       cudaStream_t stream) {
  return decode_launch(q, k_cache, v_cache, out, part_o, part_ml, block_table, kv_len, n_seqs, nh, nkv, hd,
                       page_size, max_pages, window, scale, n_splits, FusedInput{}, stream);
}

// As jb_attention_bf16_decode, but q, k and v of the new tokens come as the projection's float32
// output qkv[seq][q heads | k heads | v heads] (row stride qkv_stride floats): the kernel rotates q
// and k with cos_sin[position] (null = no rotation), appends k and v at cache row dest[seq]
// (write_kv = 0: a layer that reads another layer's cache; only q is used) and attends.
JB_EXPORT int jb_attention_bf16_decode_fused(const float* qkv, int qkv_stride, const float* cos_sin,
                                             const int* dest, void* k_cache, void* v_cache, void* out,
                                             float* part_o, float* part_ml, const int* block_table,
                                             const int* kv_len, int n_seqs, int nh, int nkv, int hd,
                                             int page_size, int max_pages, int window, float scale,
                                             int n_splits, int write_kv, cudaStream_t stream) {
  JB_REFUSE(qkv == nullptr || (write_kv && dest == nullptr), "attention_bf16 fused decode: missing input");
  JB_REFUSE(hd % 2 != 0, "attention_bf16 fused decode: head_dim %d must be even for the rotation", hd);
  FusedInput fused{qkv, qkv_stride, cos_sin, dest, (bf16*)k_cache, (bf16*)v_cache, write_kv};
  return decode_launch(nullptr, k_cache, v_cache, out, part_o, part_ml, block_table, kv_len, n_seqs, nh, nkv, hd,
                       page_size, max_pages, window, scale, n_splits, fused, stream);
}

// ---------------------------------------------------------------------------
// Entry point that allocates nothing (see attention_bf16_noalloc.h).
// ---------------------------------------------------------------------------
#include <atomic>

#include "attention_bf16_noalloc.h"

namespace {

// Scratch for the key splits' partial results.  In host code this name is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float noalloc_scratch[JB_NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
// per device: address of noalloc_scratch there.  Threads that make a device's first call at the same
// time each look the address up and store the same value.
std::atomic<float*> noalloc_device_ptr[NOALLOC_MAX_DEVICES];

}  // namespace

JB_EXPORT int jb_attention_bf16_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                               const int* block_table, const int* kv_len, int n_seqs, int nh,
                                               int nkv, int hd, int page_size, int max_pages, int window,
                                               float scale, int n_splits, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(hd != HD, "attention_bf16: built for head_dim %d, called with %d", HD, hd);
  JB_REFUSE(page_size != PAGE, "attention_bf16: page size %d (need %d)", page_size, PAGE);
  JB_REFUSE(nkv <= 0 || nh % nkv != 0, "attention_bf16: %d heads are not a multiple of %d kv heads", nh, nkv);
  JB_REFUSE(n_splits < 1, "attention_bf16 decode: n_splits must be at least 1, got %d", n_splits);
  // one split writes straight to `out`: no scratch is touched, whatever the batch
  const size_t o_floats = n_splits > 1 ? (size_t)n_seqs * nh * n_splits * HD : 0;
  const size_t ml_floats = n_splits > 1 ? (size_t)n_seqs * nh * n_splits * 2 : 0;
  JB_REFUSE(o_floats + ml_floats > JB_NOALLOC_SCRATCH_FLOATS,
            "attention_bf16 decode without allocation: %zu scratch floats are needed (n_seqs %d x heads %d x "
            "splits %d x (head_dim %d + 2)), the built-in array holds %u",
            o_floats + ml_floats, n_seqs, nh, n_splits, HD, (unsigned)JB_NOALLOC_SCRATCH_FLOATS);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  JB_REFUSE(device < 0 || device >= NOALLOC_MAX_DEVICES, "attention_bf16 decode without allocation: device %d", device);
  float* scratch = noalloc_device_ptr[device].load();
  if (scratch == nullptr) {
    // set-up, once per device, with that device current
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch = static_cast<float*>(p);
    noalloc_device_ptr[device].store(scratch);
  }
  float* part_o = n_splits > 1 ? scratch : nullptr;
  float* part_ml = n_splits > 1 ? scratch + o_floats : nullptr;
  const int G = nh / nkv;
  const int n_rb = (G + 15) / 16;
  dim3 grid(n_seqs, nkv * n_rb, n_splits);
  // the same kernel and ring depth as the ordinary entry point picks (a plain launch; the first launch of a
  // ring depth also raises that kernel's shared-memory limit, which allocates nothing)
  e = decode_dispatch(grid, stream, false, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out,
                      part_o, part_ml, block_table, kv_len, nh, nkv, max_pages, window, scale * LOG2E, n_splits,
                      FusedInput{});
  if (e != cudaSuccess) return (int)e;
  if (n_splits > 1) {
    decode_combine_kernel<<<n_seqs * nh, HD >= 128 ? 128 : 64, 0, stream>>>(part_o, part_ml, (bf16*)out, n_splits);
    JB_CHECK_LAUNCH();
  }
  return 0;
}
