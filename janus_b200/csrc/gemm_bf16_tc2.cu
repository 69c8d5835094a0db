// bfloat16 matrix product on tcgen05 with CTA pairs (cta_group::2): two CTAs on neighbouring SMs
// compute one 256 x BN tile of  D[f, t] = sum_k W[f, k] * X[t, k].  Each CTA holds 128 of the 256
// weight rows (its half of the accumulator lives in its own TMEM) and loads only HALF of the token
// tile; the MMA, issued by the pair's first CTA, reads the token halves of both.  Per CTA a stage of
// the ring is 16 KB of weights + BN/2 x 128 B of tokens, so the ring is deeper than the single-CTA
// kernel's at the same tile width and the shared-memory traffic per MMA is lower: this is the kernel
// for prefill-sized token counts; gemm_bf16_tc.cu stays the kernel for decode.
//
//   warp 0     TMA producer (both CTAs): its weight tile(s) and its half of the token tile; the
//              transaction bytes of both CTAs complete the FIRST CTA's `full` barrier
//   warp 1     allocates TMEM (cta_group::2, both CTAs); in the first CTA one lane issues
//              tcgen05.mma.cta_group::2 and commits to the `empty` / `acc_full` barriers of both CTAs
//   warps 2-5  epilogue of this CTA's 128 rows (store f32 / store bf16 / add / SiLU-gate), then an
//              arrival on the first CTA's `acc_empty` barrier
// The SiLU-gated product turns the tile round: the TOKENS lie on the 256 rows of the pair (128 per CTA) and
// the 256 columns are 128 gate rows of the weight (loaded by the first CTA) beside the 128 up rows of the
// same features (loaded by the second), so one MMA per k-step computes both and a thread of the epilogue
// finds gate and up of a feature in two columns of its own TMEM lane.
// The stacked q/k/v projection of a prompt lies the same way (tokens on the rows, 256 features = whole heads
// on the columns): its epilogue rotates q and k by the token's position and writes q as bfloat16 and k, v
// straight into the paged cache, so the projection's float32 output never goes to memory.
// The kernel is persistent (pair p computes tiles p, p + pairs, ...) with two accumulator buffers.  An adding
// product may be cut along K: the slices of an output tile are tiles of their own, next to each other in the
// order, and meet by atomic adds (few output tiles would leave most SMs idle otherwise).
// Every mbarrier wait is bounded in time (status codes 21-23).  No TMA load uses multicast.
#include <cuda.h>
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;   // weight rows per CTA (256 per pair)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
// Epilogue warps per CTA: 4 (one per quarter of the TMEM lanes), 8 or 16 (two or four per quarter, which share
// a tile's columns 16 by 16).
#ifndef JB_PAIR_EPI_WARPS
#define JB_PAIR_EPI_WARPS 16
#endif
constexpr int EPI_WARPS = JB_PAIR_EPI_WARPS;
static_assert(EPI_WARPS == 4 || EPI_WARPS == 8 || EPI_WARPS == 16, "4, 8 or 16 epilogue warps");
constexpr int EPI_PARTS = EPI_WARPS / 4;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address: the pair's first CTA

enum Mode { STORE_BF16 = 0, STORE_F32 = 1, ADD_F32 = 2, SWIGLU = 3, QKV_ROPE = 4 };

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// arrive (+ expected bytes) on a barrier given by a shared::cluster address (own CTA or the pair's first)
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (global_ns() - t0 > WAIT_LIMIT_NS) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
// TMA load of this CTA's tile; the bytes complete the barrier `bar` (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// when the MMAs issued so far are done, arrive on the barrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D f32, A and B bf16, both K-major, M = 256 (the pair), N = n.
__host__ __device__ constexpr uint32_t instr_desc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

constexpr int BN = 256;   // columns of the pair's MMA; each CTA loads 128 rows of the column operand
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = (BN / 2) * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_COLS = BN;
constexpr int TMEM_COLS = 512;    // two accumulator buffers
#ifndef JB_PAIR_STAGES
#define JB_PAIR_STAGES 6
#endif
constexpr int STAGES = JB_PAIR_STAGES;   // 32 KB each

// Where the q/k/v epilogue writes: rotated queries, and keys and values at their cache rows.
struct RopeOut {
  __nv_bfloat16* q_out;      // [T, nh * hd]
  __nv_bfloat16* k_cache;    // [pages, nkv, page_size, hd]
  __nv_bfloat16* v_cache;
  const float* cos_sin;      // [positions, hd / 2, 2]
  const int* positions;      // [T]
  const int* dest;           // [T] cache row of each token: page * page_size + row
  int nh, nkv, hd, page_size;
};

// A tile is 256 features x 256 tokens; tokens on the rows: 256 tokens x 128 (gated) or 256 (q/k/v) features.
__host__ __device__ constexpr bool tokens_on_rows(int mode) { return mode == SWIGLU || mode == QKV_ROPE; }
struct TileCoord {
  int t0, f0;
  int k_lo, k_hi;   // k-tiles of this tile's slice of K (the whole of K unless an adding product is cut)
};
// Output tiles are numbered token tile fastest inside bands of TOK_BAND token tiles: the pairs that run at the
// same time then work on a few token tiles times a few weight tiles, and a band's tokens (2,048 rows of X) stay
// in L2 while the weight tiles pass by.  With one number space over all token tiles a prompt of 65,536 tokens
// would fetch X (0.5 to 1.9 GB a product) from DRAM once per weight tile; banded, X is read once and the
// weights once per band.  Up to TOK_BAND token tiles the order is the plain one.
constexpr int TOK_BAND = 8;
template <int MODE>
__device__ __forceinline__ TileCoord tile_coord(int tile, int n_tok_tiles, int n_w_tiles, int k_tiles, int k_per,
                                                int splits) {
  TileCoord c;
  const int slice = tile % splits;   // slices of one output tile are neighbours: they run at the same time
  tile /= splits;
  const int band_tiles = TOK_BAND * n_w_tiles;
  const int band = tile / band_tiles, rem = tile - band * band_tiles;
  const int in_band = min(TOK_BAND, n_tok_tiles - band * TOK_BAND);   // the last band may hold fewer token tiles
  c.t0 = (band * TOK_BAND + rem % in_band) * 256;
  c.f0 = (rem / in_band) * (MODE == SWIGLU ? 128 : 256);
  c.k_lo = slice * k_per;
  c.k_hi = min(k_tiles, c.k_lo + k_per);
  return c;
}

// The work of one pair, in the order all three roles walk it: items pair, pair + pairs, ...  An item is a tile,
// or one of `splits` slices of K of a tile (an adding product cut along K).  With `n_whole` > 0 only the tiles
// from n_whole on are cut: the tiles that fill whole waves of pairs run uncut, and the last, partial wave is cut
// into slices so that its pieces fill the pairs again (128 tiles on 74 pairs: 74 whole tiles, then 54 tiles in
// 4 slices each = 216 pieces in three rounds of a quarter tile: 1.75 waves' time instead of 2).
template <int MODE>
struct Walk {
  int n_items, n_tok_tiles, n_w_tiles, k_tiles, k_per, splits, n_pairs, n_whole;
  int item;
  __device__ Walk(int pair, int n_pairs_, int n_items_, int n_tok_tiles_, int n_w_tiles_, int k_tiles_, int k_per_,
                  int splits_, int n_whole_)
      : n_items(n_items_), n_tok_tiles(n_tok_tiles_), n_w_tiles(n_w_tiles_), k_tiles(k_tiles_), k_per(k_per_),
        splits(splits_), n_pairs(n_pairs_), n_whole(n_whole_), item(pair) {}
  __device__ __forceinline__ bool next(TileCoord& c) {
    if (item >= n_items) return false;
    if (item < n_whole) {
      c = tile_coord<MODE>(item, n_tok_tiles, n_w_tiles, k_tiles, k_tiles, 1);
    } else {
      c = tile_coord<MODE>(n_whole * splits + (item - n_whole), n_tok_tiles, n_w_tiles, k_tiles, k_per, splits);
    }
    item += n_pairs;
    return true;
  }
};

template <int MODE>
__global__ void __launch_bounds__(THREADS) gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_w,
                                                           const __grid_constant__ CUtensorMap map_x, void* __restrict__ Y,
                                                           int T, int N_out, int ldy, int k_tiles, int n_tiles,
                                                           int n_tok_tiles, int k_per, int splits, int n_whole,
                                                           int up_tile_offset, RopeOut rope, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
  const uint32_t acc_full0 = full0 + 16 * STAGES, acc_empty0 = acc_full0 + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int n_w_tiles = (N_out + (MODE == SWIGLU ? 128 : 256) - 1) / (MODE == SWIGLU ? 128 : 256);
  jb::pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 2);   // one arrival (with its byte count) from each CTA's producer
      mbar_init(empty0 + 8 * s, 1);  // the MMA's commit, sent to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 2 * EPI_WARPS);  // the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();   // the peer's barriers are initialised before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  jb::pdl_wait();

  if (warp == 0) {
    // ---------------- producer (both CTAs) ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      Walk<MODE> walk(pair, n_pairs, n_tiles, n_tok_tiles, n_w_tiles, k_tiles, k_per, splits, n_whole);
      TileCoord tc;
      while (ok && walk.next(tc)) {
        // rows of this CTA's two loads: its 128 rows of the pair's M side, its half of the column operand
        // this CTA's weight row tile (the weights are packed: a tile is one contiguous 16 KB block)
        const int w_tile = MODE == SWIGLU ? (rank ? up_tile_offset + tc.f0 / BM : tc.f0 / BM) : tc.f0 / BM + (int)rank;
        constexpr bool TOK_ROWS = tokens_on_rows(MODE);
        const int x_row = tc.t0 + (int)rank * BM;
        for (int i = tc.k_lo; i < tc.k_hi; ++i, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, status, 21)) { ok = false; break; }
          const uint32_t stage = smem_base + s * STAGE_BYTES;
          const uint32_t bar = (full0 + 8 * s) & PEER_MASK;   // the first CTA's barrier collects both CTAs' bytes
          mbar_expect_tx_cluster(bar, STAGE_BYTES);
          const int kx = i * BK;
          const int wy = (w_tile * k_tiles + i) * BM;   // beyond the packed matrix: filled with zeros
          if (TOK_ROWS) {
            tma_load_2d_pair(stage, &map_x, bar, kx, x_row);
            tma_load_2d_pair(stage + A_BYTES, &map_w, bar, 0, wy);
          } else {
            tma_load_2d_pair(stage, &map_w, bar, 0, wy);
            tma_load_2d_pair(stage + A_BYTES, &map_x, bar, kx, x_row);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (first CTA of the pair) ----------------
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = instr_desc_pair(BN);
      bool ok = true;
      int it = 0, j = 0;
      Walk<MODE> walk(pair, n_pairs, n_tiles, n_tok_tiles, n_w_tiles, k_tiles, k_per, splits, n_whole);
      TileCoord tc;
      for (; ok && walk.next(tc); ++j) {
        const int buf = j & 1;
        ok = mbar_wait(acc_empty0 + 8 * buf, ((j >> 1) & 1) ^ 1, status, 22);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
        for (int i = tc.k_lo; i < tc.k_hi; ++i, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, status, 22);
          if (!ok) break;
          tc_fence_after();
          const uint32_t stage = smem_base + s * STAGE_BYTES;
          const uint64_t a_desc = smem_desc_sw128(stage);
          const uint64_t b_desc = smem_desc_sw128(stage + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_pair(acc_addr, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > tc.k_lo || k > 0) ? 1u : 0u);
          umma_commit_pair(empty0 + 8 * s);
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * buf);
      }
    }
  } else {
    // ---------------- epilogue (this CTA's 128 rows) ----------------
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;   // which of the columns' 16-wide chunks (every EPI_PARTS-th) this warp takes
    int j = 0;
    Walk<MODE> walk(pair, n_pairs, n_tiles, n_tok_tiles, n_w_tiles, k_tiles, k_per, splits, n_whole);
    TileCoord tc;
    for (; walk.next(tc); ++j) {
      const int buf = j & 1;
      if (!mbar_wait(acc_full0 + 8 * buf, (j >> 1) & 1, status, 23)) break;
      tc_fence_after();
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
      if (MODE == SWIGLU) {
        // this lane is a token; columns c and 128 + c are gate and up of feature f0 + c
        const int t = tc.t0 + (int)rank * BM + quarter * 32 + lane;
        __nv_bfloat16* yrow = (__nv_bfloat16*)Y + (size_t)t * ldy;
        const bool vec_ok = (ldy % 8) == 0 && (((uintptr_t)Y) & 15) == 0;
#pragma unroll 1
        for (int c0 = 16 * part; c0 < 128; c0 += 16 * EPI_PARTS) {
          if (tc.f0 + c0 >= N_out) break;
          uint32_t r[16], u[16];
          tmem_ld16(lane_base + c0, r);
          tmem_ld16(lane_base + 128 + c0, u);
          tmem_ld_wait();
          if (t < T) {
            uint32_t packed[8];
#pragma unroll
            for (int jj = 0; jj < 16; jj += 2) {
              const float g0 = __uint_as_float(r[jj]), g1 = __uint_as_float(r[jj + 1]);
              const float a0 = g0 * (1.0f / (1.0f + expf(-g0))) * __uint_as_float(u[jj]);
              const float a1 = g1 * (1.0f / (1.0f + expf(-g1))) * __uint_as_float(u[jj + 1]);
              const __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
              packed[jj / 2] = *(const uint32_t*)&h;
            }
            const int f = tc.f0 + c0;
            if (vec_ok && f + 16 <= N_out) {
              uint4* dst = (uint4*)(yrow + f);
              dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj)
                if (f + jj < N_out)
                  yrow[f + jj] = __ushort_as_bfloat16((unsigned short)(packed[jj / 2] >> (16 * (jj & 1))));
            }
          }
        }
      } else if (MODE == QKV_ROPE) {
        // this lane is a token; the 256 columns are whole heads of q, k or v
        const int t = tc.t0 + (int)rank * BM + quarter * 32 + lane;
        const bool t_ok = t < T;
        const int hd = rope.hd, half = hd >> 1;
        const int pos = t_ok ? rope.positions[t] : 0;
        const int dst = t_ok ? rope.dest[t] : 0;
        const float* cs = rope.cos_sin + (size_t)pos * hd;
#pragma unroll 1
        for (int c = 0; c < BN; c += hd) {
          const int f = tc.f0 + c;
          if (f >= N_out) break;
          const int head = f / hd;
          __nv_bfloat16* out;
          const bool rotate = head < rope.nh + rope.nkv;
          if (head < rope.nh) {
            out = rope.q_out + ((size_t)t * rope.nh + head) * hd;
          } else {
            const int kvh = (head - rope.nh) % rope.nkv;
            __nv_bfloat16* base = head < rope.nh + rope.nkv ? rope.k_cache : rope.v_cache;
            out = base + (((size_t)(dst / rope.page_size) * rope.nkv + kvh) * rope.page_size + dst % rope.page_size) * hd;
          }
#pragma unroll 1
          for (int i = 16 * part; i < half; i += 16 * EPI_PARTS) {   // (half is a multiple of 16 * EPI_PARTS or the parts idle)
            uint32_t lo[16], hi[16];
            tmem_ld16(lane_base + c + i, lo);
            tmem_ld16(lane_base + c + half + i, hi);
            tmem_ld_wait();
            if (t_ok) {
              uint32_t plo[8], phi[8];
#pragma unroll
              for (int jj = 0; jj < 16; jj += 2) {
                float y0[2], y1[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const float x0 = __uint_as_float(lo[jj + e]), x1 = __uint_as_float(hi[jj + e]);
                  if (rotate) {
                    const float2 k = *reinterpret_cast<const float2*>(cs + 2 * (i + jj + e));   // (cos, sin)
                    y0[e] = x0 * k.x - x1 * k.y;
                    y1[e] = x0 * k.y + x1 * k.x;
                  } else {
                    y0[e] = x0;
                    y1[e] = x1;
                  }
                }
                const __nv_bfloat162 a = __floats2bfloat162_rn(y0[0], y0[1]), b = __floats2bfloat162_rn(y1[0], y1[1]);
                plo[jj / 2] = *(const uint32_t*)&a;
                phi[jj / 2] = *(const uint32_t*)&b;
              }
              uint4* d0 = (uint4*)(out + i);
              uint4* d1 = (uint4*)(out + half + i);
              d0[0] = make_uint4(plo[0], plo[1], plo[2], plo[3]);
              d0[1] = make_uint4(plo[4], plo[5], plo[6], plo[7]);
              d1[0] = make_uint4(phi[0], phi[1], phi[2], phi[3]);
              d1[1] = make_uint4(phi[4], phi[5], phi[6], phi[7]);
            }
          }
        }
      } else {
        const int f = tc.f0 + (int)rank * BM + quarter * 32 + lane;
        const bool f_ok = f < N_out;
#pragma unroll 1
        for (int c0 = 16 * part; c0 < BN; c0 += 16 * EPI_PARTS) {
          if (tc.t0 + c0 >= T) break;
          uint32_t r[16];
          tmem_ld16(lane_base + c0, r);
          tmem_ld_wait();
          if (f_ok) {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              const int t = tc.t0 + c0 + jj;
              if (t < T) {
                const float v = __uint_as_float(r[jj]);
                const size_t o = (size_t)t * ldy + f;
                if (MODE == STORE_BF16) {
                  ((__nv_bfloat16*)Y)[o] = __float2bfloat16_rn(v);
                } else if (MODE == STORE_F32) {
                  ((float*)Y)[o] = v;
                } else {
                  atomicAdd(((float*)Y) + o, v);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster((acc_empty0 + 8 * buf) & PEER_MASK);
    }
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync();   // neither CTA leaves while its pair may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map of packed weights (jb_pack_weight_bf16): `tiles` blocks of 128 rows x 128 bytes, already swizzled.
bool make_packed_map(CUtensorMap* map, const void* base, uint64_t tiles) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)BK, tiles * BM};
  const cuuint64_t strides[1] = {(cuuint64_t)BK * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

template <int MODE>
int launch(const void* X, const void* W, long long w_tiles, int up_tile_offset, void* Y, int T, int N_out, int K, int ldy,
           const RopeOut& rope, int* status, cudaStream_t stream, int split_k = 1, int whole_tiles = 0) {
  constexpr int smem = STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap mw, mx;
  {
    const long long kt = (K + BK - 1) / BK, rt = (N_out + BM - 1) / BM;
    const long long need = MODE == SWIGLU ? (up_tile_offset + rt) * kt : rt * kt;
    JB_REFUSE(w_tiles < need || (MODE == SWIGLU && up_tile_offset < rt) || w_tiles * BM > 0x7fffffffLL,
              "gemm_bf16_pair: the packed weight holds %lld tiles, the product needs %lld", w_tiles, need);
  }
  if (!make_packed_map(&mw, W, (uint64_t)w_tiles)) return JB_ERR_TENSORMAP;
  if (!make_map(&mx, X, (uint64_t)T, (uint64_t)K, BM)) return JB_ERR_TENSORMAP;
  const int k_tiles = (K + BK - 1) / BK;
  constexpr int F_TILE = MODE == SWIGLU ? 128 : 256;
  const int n_tok_tiles = (T + 255) / 256, n_w_tiles = (N_out + F_TILE - 1) / F_TILE;
  // only a product that adds can be cut along K: its slices meet by atomic adds (no slice is empty)
  const int half_sms = sm_count() / 2;
  const int out_tiles_i = n_tok_tiles * n_w_tiles;
  const int want = MODE == ADD_F32 ? max(1, min(split_k, k_tiles)) : 1;
  // `whole_tiles` of an adding product's tiles (those that fill whole waves of pairs) stay uncut, the rest is cut
  const int n_whole = (MODE == ADD_F32 && want > 1) ? max(0, min(whole_tiles, out_tiles_i)) : 0;
  const int k_per = (k_tiles + want - 1) / want;
  const int splits = (k_tiles + k_per - 1) / k_per;
  const long long all_tiles = n_whole + (long long)(out_tiles_i - n_whole) * splits;
  JB_REFUSE(all_tiles > 0x7fffffffLL || (long long)n_tok_tiles * n_w_tiles > 0x7fffffffLL,
            "gemm_bf16_pair: too many tiles (%lld)", all_tiles);
  const int n_tiles = (int)all_tiles;
  const int pairs = n_tiles < half_sms ? n_tiles : half_sms;
  cudaLaunchConfig_t cfg = cudaLaunchConfig_t{};
  cudaLaunchAttribute attrs[2];
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  if (jb::pdl_enabled()) {
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  return (int)cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<MODE>, mw, mx, Y, T, N_out, ldy, k_tiles, n_tiles,
                                 n_tok_tiles, k_per, splits, n_whole, MODE == SWIGLU ? up_tile_offset : 0, rope, status);
}

}  // namespace

// Same contract as jb_gemm_bf16: Y (+)= X . W^T with X [T, K] and W packed (jb_pack_weight_bf16); `split_k` > 1
// cuts K of an adding product (mode ADD_F32) into that many slices, which meet in Y by atomic adds; the first
// `whole_tiles` output tiles (256 x 256, token tile fastest) stay uncut: the tiles that fill whole waves of CTA
// pairs, so that only the last, partial wave is cut.
// Meant for prompt-sized T.  status codes of a timed-out wait: 21 producer, 22 MMA, 23 epilogue.
JB_EXPORT int jb_gemm_bf16_pair(const void* X, const void* W, long long w_tiles, int up_tile_offset, void* Y, int T,
                                int N_out, int K, int ldy, int mode, int split_k, int whole_tiles, int* status,
                                cudaStream_t stream) {
  if (T <= 0 || N_out <= 0) return 0;
  JB_REFUSE(K <= 0 || K % 8 != 0, "gemm_bf16_pair: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  JB_REFUSE(((uintptr_t)X | (uintptr_t)W) & 15, "gemm_bf16_pair: operands must be 16-byte aligned");
  switch (mode) {
    case STORE_BF16: return launch<STORE_BF16>(X, W, w_tiles, up_tile_offset, Y, T, N_out, K, ldy, RopeOut{}, status, stream);
    case STORE_F32: return launch<STORE_F32>(X, W, w_tiles, up_tile_offset, Y, T, N_out, K, ldy, RopeOut{}, status, stream);
    case ADD_F32: return launch<ADD_F32>(X, W, w_tiles, up_tile_offset, Y, T, N_out, K, ldy, RopeOut{}, status, stream, split_k, whole_tiles);
    case SWIGLU: return launch<SWIGLU>(X, W, w_tiles, up_tile_offset, Y, T, N_out, K, ldy, RopeOut{}, status, stream);
    default: JB_REFUSE(true, "gemm_bf16_pair: unknown mode %d", mode);
  }
}

// The stacked q/k/v projection of prompt tokens with its consumers fused in: X [T, K] . W [(nh + 2 nkv) hd, K]^T,
// q and k rotated by cos_sin[positions[t]] (pairs i, i + hd/2), q written to q_out [T, nh hd] and k, v to the
// paged cache at row dest[t], all bfloat16.  hd must divide 256 and hd/2 be a multiple of 16 (32, 64, 128, 256).
JB_EXPORT int jb_gemm_bf16_pair_qkv_rope(const void* X, const void* W, long long w_tiles, int T, int K, void* q_out, void* k_cache,
                                         void* v_cache, const float* cos_sin, const int* positions, const int* dest,
                                         int nh, int nkv, int hd, int page_size, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(K <= 0 || K % 8 != 0, "gemm_bf16_pair_qkv_rope: K = %d must be a positive multiple of 8", K);
  JB_REFUSE(((uintptr_t)X | (uintptr_t)W | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15,
            "gemm_bf16_pair_qkv_rope: tensors must be 16-byte aligned");
  JB_REFUSE(hd <= 0 || 256 % hd != 0 || (hd / 2) % 16 != 0,
            "gemm_bf16_pair_qkv_rope: head_dim %d is not one of 32, 64, 128, 256", hd);
  JB_REFUSE(nh <= 0 || nkv <= 0 || page_size <= 0 || !cos_sin || !positions || !dest, "gemm_bf16_pair_qkv_rope: bad arguments");
  RopeOut rope{(__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, cos_sin, positions, dest,
               nh, nkv, hd, page_size};
  return launch<QKV_ROPE>(X, W, w_tiles, 0, nullptr, T, (nh + 2 * nkv) * hd, K, 0, rope, status, stream);
}
