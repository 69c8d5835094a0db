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

__global__ void __launch_bounds__(THREADS) sample_kernel(
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
  __shared__ float s_scan[THREADS];
  __shared__ int s_result;

  const int row = blockIdx.x, tid = threadIdx.x;
  int* my_counts = (counts && penalty != 1.0f) ? counts + (size_t)count_rows[row] * V : nullptr;
  RowView view{logits + (size_t)row * V, my_counts, penalty};

  // ---- maximum and argmax (needed by both modes) -------------------------
  float best = -CUDART_INF_F;
  int best_i = 0x7fffffff;
  for (int v = tid; v < V; v += THREADS) {
    const float x = view.at(v);
    if (x > best) { best = x; best_i = v; }
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
    const float inv_shift = x_max / temperature;
    auto weight = [&](int v) -> float {
      const float x = view.at(v);
      if (ordered_key(x) < thr_key || !(x == x) || x == -CUDART_INF_F) return 0.0f;
      return expf(x / temperature - inv_shift);
    };
    // ---- normaliser --------------------------------------------------------
    float z = 0.0f;
    for (int v = tid; v < V; v += THREADS) z += weight(v);
    z = jb::block_sum(z, s_red);
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
    auto kept = [&](int v) -> float {
      const float w = weight(v);
      return (__float_as_uint(w) >= thr_bits) ? w : 0.0f;
    };
    // ---- inverse CDF in index order ------------------------------------------
    const int chunk = (V + THREADS - 1) / THREADS;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
    float local = 0.0f;
    for (int v = lo; v < hi; ++v) local += kept(v);
    s_scan[tid] = local;
    __syncthreads();
    if (tid == 0) {
      // Serial scan over 1024 partial sums keeps the order of the sum fixed.
      float run = 0.0f;
      for (int i = 0; i < THREADS; ++i) {
        const float t = s_scan[i];
        s_scan[i] = run;
        run += t;
      }
      s_red[0] = run;
      s_result = -1;
    }
    __syncthreads();
    const float total = s_red[0];
    const float u = uniform_for(seed, (unsigned long long)seq_ids[row], (unsigned long long)steps[row]);
    const float target = u * total;
    const float before = s_scan[tid];
    if (local > 0.0f && target >= before && target < before + local) {
      float run = before;
      int pick = -1, last_kept = -1;
      for (int v = lo; v < hi; ++v) {
        const float w = kept(v);
        if (w > 0.0f) {
          last_kept = v;
          run += w;
          if (target < run) { pick = v; break; }
        }
      }
      s_result = pick >= 0 ? pick : last_kept;
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
  sample_kernel<<<B, THREADS, 0, stream>>>(logits, V, out_ids, temperature, top_k, top_p, penalty, counts,
                                           count_rows, seed, seq_ids, steps, feedback);
  JB_CHECK_LAUNCH();
  return 0;
}
