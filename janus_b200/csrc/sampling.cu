// On-device sampling from float32 logits, one thread block per row.
//
// Options and their order follow the reference's sampler
// (crates/janus-engine/src/model/sampler.rs): repetition penalty over the
// tokens generated so far, once per occurrence (599-613); temperature 0 means
// argmax (200-206), the lowest index winning ties as in
// crates/janus-engine/src/compute/shaders/argmax.wgsl:43-51; otherwise top-k
// on the logits (653-673, ties with the k-th value stay), division by the
// temperature (629-632), softmax with the maximum subtracted (726-747), top-p
// as the smallest set of largest probabilities whose sum reaches p (683-717;
// here all entries equal to the cut-off value stay), and an inverse-CDF walk in
// index order (756-772).  The uniform number comes from a counter-based
// generator keyed by (seed, sequence, step), so a sequence's draws do not
// depend on what else is in the batch.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ float uniform_for(unsigned long long seed, unsigned long long sequence,
                                             unsigned long long step) {
  unsigned long long x = seed * 0x9E3779B97F4A7C15ull + sequence * 0xBF58476D1CE4E5B9ull +
                         step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ unsigned ordered_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowView {
  const float* logits;
  const int* counts;  // occurrences of each token among the generated ones, or null
  float penalty;
  __device__ __forceinline__ float at(int v) const {
    float x = logits[v];
    if (counts) {
      for (int c = counts[v]; c > 0; --c) x = x > 0.0f ? x / penalty : x * penalty;
    }
    return x;
  }
};

// Largest (value, lowest index) over the block; result in smem_val[0], smem_idx[0].
__device__ void block_argmax(float v, int i, float* smem_val, int* smem_idx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
  __syncthreads();
  if (lane == 0) { smem_val[warp] = v; smem_idx[warp] = i; }
  __syncthreads();
  if (warp == 0) {
    v = smem_val[lane];  // THREADS / 32 == 32 warps
    i = smem_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    if (lane == 0) { smem_val[0] = v; smem_idx[0] = i; }
  }
  __syncthreads();
}

// Inclusive sums over a warp's lanes (lane 31 ends with the sum of all).
__device__ __forceinline__ float warp_inclusive(float v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

__global__ void __launch_bounds__(THREADS, 1) sample_kernel(
    const float* __restrict__ logits, int V, int* __restrict__ out_ids, float temperature, int top_k,
    float top_p, float penalty, int* __restrict__ counts, const int* __restrict__ count_rows,
    unsigned long long seed, const int* __restrict__ seq_ids, const int* __restrict__ steps,
    int* __restrict__ feedback) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_red[33];
  __shared__ unsigned s_hist[256];
  __shared__ float s_fhist[256];
  __shared__ unsigned s_sel[2];   // chosen digit, remaining rank
  __shared__ float s_fsel;        // mass above the chosen digit
  __shared__ float s_warp[THREADS / 32];
  __shared__ int s_result;
  extern __shared__ float s_iter[];   // [THREADS / 32][ceil(V / (4 THREADS))]: sums of pieces of 128 indices

  const int row = blockIdx.x, tid = threadIdx.x;
  int* my_counts = (counts && penalty != 1.0f) ? counts + (size_t)count_rows[row] * V : nullptr;
  RowView view{logits + (size_t)row * V, my_counts, penalty};

  // ---- maximum and argmax (needed by both modes) -------------------------
  float best = -CUDART_INF_F;
  int best_i = 0x7fffffff;
  if (my_counts == nullptr && (V & 3) == 0) {
    // plain logits in rows of whole 16-byte vectors: four at a time, several vectors in flight per thread
    // (a thread's indices still rise, so the first of equal values stays)
    const float4* row4 = reinterpret_cast<const float4*>(view.logits);
#pragma unroll 4
    for (int i = tid; i < (V >> 2); i += THREADS) {
      const float4 x = row4[i];
      if (x.x > best) { best = x.x; best_i = 4 * i; }
      if (x.y > best) { best = x.y; best_i = 4 * i + 1; }
      if (x.z > best) { best = x.z; best_i = 4 * i + 2; }
      if (x.w > best) { best = x.w; best_i = 4 * i + 3; }
    }
  } else {
    for (int v = tid; v < V; v += THREADS) {
      const float x = view.at(v);
      if (x > best) { best = x; best_i = v; }
    }
  }
  block_argmax(best, best_i, s_val, s_idx);
  const float x_max = s_val[0];
  int token = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];

  if (temperature > 0.0f) {
    // ---- top-k threshold: key of the k-th largest value -------------------
    unsigned thr_key = 0u;
    if (top_k > 0 && top_k < V) {
      unsigned prefix = 0u, mask = 0u, rank = (unsigned)top_k;
      for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) s_hist[tid] = 0u;
        __syncthreads();
        for (int v = tid; v < V; v += THREADS) {
          const unsigned key = ordered_key(view.at(v));
          if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
          unsigned above = 0u;
          int b = 255;
          for (; b > 0; --b) {
            if (above + s_hist[b] >= rank) break;
            above += s_hist[b];
          }
          s_sel[0] = (unsigned)b;
          s_sel[1] = rank - above;
        }
        __syncthreads();
        prefix |= s_sel[0] << shift;
        mask |= 255u << shift;
        rank = s_sel[1];
        __syncthreads();
      }
      thr_key = prefix;
    }
    // weight = exp((x - max) / temperature) as 2^(x a - max a), a = log2(e) / temperature: one fused
    // multiply-add and one exponential a value; the same code in every pass, so passes agree bit for bit
    const float w_a = 1.4426950408889634f / temperature, w_b = x_max * w_a;
    auto weight_of = [&](float x) -> float {
      if (ordered_key(x) < thr_key || !(x == x)) return 0.0f;
      return exp2f(fmaf(x, w_a, -w_b));   // -inf gives 0
    };
    auto weight = [&](int v) -> float { return weight_of(view.at(v)); };
    // ---- normaliser (only the top-p threshold needs it) ----------------------
    float z = 0.0f;
    if (top_p < 1.0f) {
      for (int v = tid; v < V; v += THREADS) z += weight(v);
      z = jb::block_sum(z, s_red);
    }
    // ---- top-p threshold on the weights -------------------------------------
    unsigned thr_bits = 0u;
    if (top_p < 1.0f) {
      const float target = top_p * z;
      unsigned prefix = 0u, mask = 0u;
      float above_mass = 0.0f;
      for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) s_fhist[tid] = 0.0f;
        __syncthreads();
        for (int v = tid; v < V; v += THREADS) {
          const float w = weight(v);
          const unsigned key = __float_as_uint(w);
          if (w > 0.0f && (key & mask) == prefix) atomicAdd(&s_fhist[(key >> shift) & 255u], w);
        }
        __syncthreads();
        if (tid == 0) {
          float above = above_mass;
          int b = 255;
          for (; b > 0; --b) {
            if (above + s_fhist[b] >= target) break;
            above += s_fhist[b];
          }
          s_sel[0] = (unsigned)b;
          s_fsel = above;
        }
        __syncthreads();
        prefix |= s_sel[0] << shift;
        mask |= 255u << shift;
        above_mass = s_fsel;
        __syncthreads();
      }
      thr_bits = prefix;
    }
    auto kept_of = [&](float x) -> float {
      const float w = weight_of(x);
      return (__float_as_uint(w) >= thr_bits) ? w : 0.0f;
    };
    // ---- inverse CDF in index order ------------------------------------------
    // Warp w owns the indices [w * iters * 128, (w + 1) * iters * 128) in pieces of 128 consecutive ones, four
    // to a lane (one 16-byte load).  A piece's sum is the lanes' own sums of four, scanned over the warp; the
    // running sums of a warp's pieces and then of the warps are added up in index order by the same code for
    // every thread, so the interval that holds the target has exactly one owner.
    const int warp = tid >> 5, lane = tid & 31;
    const int iters = (V + 4 * THREADS - 1) / (4 * THREADS);
    const bool vec = my_counts == nullptr && (V & 3) == 0;
    auto four = [&](int v0, float* w) {   // the kept weights of indices v0 .. v0 + 3
      if (vec) {
        float4 x = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        if (v0 < V) x = *reinterpret_cast<const float4*>(view.logits + v0);
        w[0] = kept_of(x.x), w[1] = kept_of(x.y), w[2] = kept_of(x.z), w[3] = kept_of(x.w);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = v0 + j < V ? kept_of(view.at(v0 + j)) : 0.0f;
      }
    };
    float* my_iter = s_iter + warp * iters;
#pragma unroll 4
    for (int k = 0; k < iters; ++k) {
      float w[4];
      four(((warp * iters + k) * 32 + lane) * 4, w);
      const float t = warp_inclusive(((w[0] + w[1]) + w[2]) + w[3]);
      if (lane == 31) my_iter[k] = t;
    }
    __syncwarp();
    if (lane == 0) {
      float run = 0.0f;
      for (int k = 0; k < iters; ++k) {
        run += my_iter[k];
        my_iter[k] = run;   // the warp's pieces up to and with piece k
      }
      s_warp[warp] = run;
      if (tid == 0) s_result = -1;
    }
    __syncthreads();
    float before = 0.0f, my_before = 0.0f;
    for (int w2 = 0; w2 < THREADS / 32; ++w2) {
      if (w2 == warp) my_before = before;
      before += s_warp[w2];
    }
    const float total = before;
    const float u = uniform_for(seed, (unsigned long long)seq_ids[row], (unsigned long long)steps[row]);
    const float target = u * total;
    const float my_total = s_warp[warp];
    // my_before + my_total is, bit for bit, the next warp's my_before: one warp owns the target
    if (my_total > 0.0f && target >= my_before && target < my_before + my_total) {
      int k_pick = iters - 1;
      for (int k0 = 0; k0 < iters; k0 += 32) {
        const int k = k0 + lane;
        const unsigned hit = __ballot_sync(0xffffffffu, k < iters && target < my_before + my_iter[k]);
        if (hit) {
          k_pick = k0 + __ffs(hit) - 1;
          break;
        }
      }
      const float run0 = my_before + (k_pick > 0 ? my_iter[k_pick - 1] : 0.0f);
      const int v0 = ((warp * iters + k_pick) * 32 + lane) * 4;
      float w[4];
      four(v0, w);
      const float mine = ((w[0] + w[1]) + w[2]) + w[3];
      float run = run0 + (warp_inclusive(mine) - mine);   // what lies before this lane's four
      // the first kept index whose running sum passes the target; if rounding lets none pass, the piece's last
      int hit_j = -1, last_j = -1;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (w[j] > 0.0f) {
          run += w[j];
          last_j = j;
          if (hit_j < 0 && target < run) hit_j = j;
        }
      }
      const unsigned passed = __ballot_sync(0xffffffffu, hit_j >= 0);
      const unsigned any_kept = __ballot_sync(0xffffffffu, last_j >= 0);
      const int pick_lane = passed ? __ffs(passed) - 1 : (any_kept ? 31 - __clz(any_kept) : -1);
      if (pick_lane == lane) s_result = v0 + (passed ? hit_j : last_j);
    }
    __syncthreads();
    if (s_result >= 0) token = s_result;  // else rounding left no owner: keep the argmax
  }
  if (tid == 0) {
    out_ids[row] = token;
    if (my_counts) my_counts[token] += 1;
    if (feedback) feedback[count_rows[row]] = token;  // the next step may read its input token from here
  }
}

}  // namespace

// counts: [rows, V] int32 occurrences of generated tokens per sequence (may be
// null when penalty == 1); count_rows[b] selects the row of `counts` for batch
// row b.  The kernel adds the sampled token to its row of `counts`.  feedback (may be null):
// int32 per cache slot; the token of batch row b is also stored at feedback[count_rows[b]].
JB_EXPORT int jb_sample(const float* logits, int B, int V, int* out_ids, float temperature, int top_k,
                        float top_p, float penalty, int* counts, const int* count_rows,
                        unsigned long long seed, const int* seq_ids, const int* steps, int* feedback,
                        cudaStream_t stream) {
  if (B <= 0) return 0;
  JB_REFUSE(V <= 0, "sample: vocabulary size %d", V);
  JB_REFUSE(temperature < 0.0f, "sample: negative temperature %f", temperature);
  JB_REFUSE(penalty <= 0.0f, "sample: repetition penalty %f must be positive", penalty);
  JB_REFUSE(feedback != nullptr && count_rows == nullptr, "sample: feedback needs the rows' slots");
  // shared memory for the sums of the pieces of 128 indices (used when temperature > 0)
  const size_t smem = temperature > 0.0f ? (size_t)((V + 4 * THREADS - 1) / (4 * THREADS)) * (THREADS / 32) * sizeof(float) : 0;
  JB_REFUSE(smem > 200 * 1024, "sample: a vocabulary of %d is too large for temperature sampling", V);
  static size_t smem_allowed = 48 * 1024;
  if (smem > smem_allowed) {
    const cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    smem_allowed = smem;
  }
  sample_kernel<<<B, THREADS, smem, stream>>>(logits, V, out_ids, temperature, top_k, top_p, penalty, counts,
                                              count_rows, seed, seq_ids, steps, feedback);
  JB_CHECK_LAUNCH();
  return 0;
}
