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
constexpr int DIGITS0 = 4096;   // digits of the radix select's first pass (12 bits; then 10 and 10)

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

// A row of logits with the repetition penalty applied where a token has been generated before.
struct RowView {
  const float* logits;
  const int* counts;  // occurrences of each token among the generated ones, or null
  float penalty;
  int V;
  __device__ __forceinline__ float penalised(float x, int c) const {
    for (; c > 0; --c) x = x > 0.0f ? x / penalty : x * penalty;
    return x;
  }
  __device__ __forceinline__ float at(int v) const {
    const float x = logits[v];
    return counts ? penalised(x, counts[v]) : x;
  }
  // rows of whole 16-byte vectors are read four values at a time
  __device__ __forceinline__ bool vectors() const { return (V & 3) == 0; }
  __device__ __forceinline__ float4 at4(int v0) const {   // v0 a multiple of 4, v0 + 3 < V
    float4 x = *reinterpret_cast<const float4*>(logits + v0);
    if (counts) {
      const int4 c = *reinterpret_cast<const int4*>(counts + v0);
      if (c.x | c.y | c.z | c.w) {
        x.x = penalised(x.x, c.x), x.y = penalised(x.y, c.y), x.z = penalised(x.z, c.z), x.w = penalised(x.w, c.w);
      }
    }
    return x;
  }
  // f(index, value) for every index, each thread's indices rising
  template <typename F>
  __device__ __forceinline__ void for_all(F&& f) const {
    if (vectors()) {
#pragma unroll 4
      for (int i = threadIdx.x; i < (V >> 2); i += THREADS) {
        const float4 x = at4(4 * i);
        f(4 * i, x.x), f(4 * i + 1, x.y), f(4 * i + 2, x.z), f(4 * i + 3, x.w);
      }
    } else {
      for (int v = threadIdx.x; v < V; v += THREADS) f(v, at(v));
    }
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

// Radix select, one digit: `value(d)` is what digit d holds (a count or a mass), d < n_digits = per * THREADS.
// Picks the highest digit d such that the digits >= d, together with `above0`, reach `target` (digit 0 if none
// does), and what lies above d.  Every thread gets both.  A thread owns `per` neighbouring digits; sums over the
// threads above it come from warp scans and the warps' totals.
template <typename F>
__device__ __forceinline__ void pick_digit(F&& value, int per, unsigned long long above0, unsigned long long target,
                                           unsigned long long* s_warp_tot, unsigned* s_pick, unsigned long long* s_above,
                                           unsigned& digit, unsigned long long& above) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long mine = 0ull;
  for (int j = 0; j < per; ++j) mine += value(tid * per + j);
  unsigned long long at_or_above = mine;   // over the lanes >= this one
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_down_sync(0xffffffffu, at_or_above, o);
    if (lane + o < 32) at_or_above += t;
  }
  if (lane == 0) s_warp_tot[warp] = at_or_above;
  if (tid == 0) {
    *s_pick = 0u;
    *s_above = 0ull;
  }
  __syncthreads();
  unsigned long long higher = above0 + (at_or_above - mine);   // above this thread's digits
  for (int w = warp + 1; w < THREADS / 32; ++w) higher += s_warp_tot[w];
  int found = -1;
  unsigned long long found_above = 0ull;
  for (int j = per - 1; j >= 0; --j) {
    const unsigned long long v = value(tid * per + j);
    if (found < 0 && higher + v >= target) {
      found = tid * per + j;
      found_above = higher;
    }
    higher += v;
  }
  if (found > 0) atomicMax(s_pick, (unsigned)found);
  __syncthreads();
  digit = *s_pick;
  if (found >= 0 && (unsigned)found == digit) *s_above = found_above;
  if (digit == 0u && tid == 0 && found != 0) *s_above = higher - value(0);   // nothing reached the target
  __syncthreads();
  above = *s_above;
  __syncthreads();
}

__global__ void __launch_bounds__(THREADS, 1) sample_kernel(
    const float* __restrict__ logits, int V, int* __restrict__ out_ids, float temperature, int top_k,
    float top_p, float penalty, int* __restrict__ counts, const int* __restrict__ count_rows,
    unsigned long long seed, const int* __restrict__ seq_ids, const int* __restrict__ steps,
    int* __restrict__ feedback) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ unsigned long long s_warp_tot[THREADS / 32];
  __shared__ unsigned s_pick;
  __shared__ unsigned long long s_above;
  __shared__ float s_warp[THREADS / 32];
  __shared__ int s_result;
  // dynamic: the radix select's histograms [3][4096] (counts use the first; masses three limbs), then
  // [THREADS / 32][ceil(V / (4 THREADS))] sums of pieces of 128 indices
  extern __shared__ unsigned s_dyn[];
  unsigned* s_hist = s_dyn;
  float* s_iter = reinterpret_cast<float*>(s_dyn + 3 * DIGITS0);

  const int row = blockIdx.x, tid = threadIdx.x;
  int* my_counts = (counts && penalty != 1.0f) ? counts + (size_t)count_rows[row] * V : nullptr;
  const RowView view{logits + (size_t)row * V, my_counts, penalty, V};

  // ---- maximum and argmax (needed by both modes) -------------------------
  float best = -CUDART_INF_F;
  int best_i = 0x7fffffff;
  if (my_counts == nullptr && view.vectors()) {
    // plain logits, four at a time (a thread's indices rise, so the first of equal values stays)
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
    view.for_all([&](int v, float x) {
      if (x > best) { best = x; best_i = v; }
    });
  }
  block_argmax(best, best_i, s_val, s_idx);
  const float x_max = s_val[0];
  int token = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];

  if (temperature > 0.0f) {
    // ---- top-k threshold: key of the k-th largest value -------------------
    // three passes over digits of 12, 10 and 10 bits of the ordered keys
    unsigned thr_key = 0u;
    if (top_k > 0 && top_k < V) {
      unsigned prefix = 0u, mask = 0u;
      unsigned long long rank = (unsigned long long)top_k;
      for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 20 : pass == 1 ? 10 : 0, n_digits = pass == 0 ? DIGITS0 : 1024;
        for (int i = tid; i < n_digits; i += THREADS) s_hist[i] = 0u;
        __syncthreads();
        view.for_all([&](int, float x) {
          const unsigned key = ordered_key(x);
          if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & (n_digits - 1)], 1u);
        });
        __syncthreads();
        unsigned digit;
        unsigned long long above;
        pick_digit([&](int d) { return (unsigned long long)s_hist[d]; }, n_digits / THREADS, 0ull, rank, s_warp_tot,
                   &s_pick, &s_above, digit, above);
        prefix |= digit << shift;
        mask |= (unsigned)(n_digits - 1) << shift;
        rank -= above;
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
    // ---- top-p threshold on the weights -------------------------------------
    // The smallest weight t such that the weights >= t together reach top_p of all the mass: a radix
    // select over the weights' bit patterns in digits of 12, 10 and 10 bits, with the mass of each digit
    // in a histogram.  Masses are added as integers: a weight (at most 1) in units of 2^-33, as three
    // limbs of 11 bits in 32-bit histograms (2^20 limbs fit), because shared memory adds 32-bit integers
    // natively, and integer sums are exact whatever their order: the threshold is the same every run.
    unsigned thr_bits = 0u;
    if (top_p < 1.0f) {
      unsigned prefix = 0u, mask = 0u;
      unsigned long long above = 0ull, target = 0ull;
      for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 20 : pass == 1 ? 10 : 0, n_digits = pass == 0 ? DIGITS0 : 1024;
        for (int i = tid; i < 3 * DIGITS0; i += THREADS) s_hist[i] = 0u;
        __syncthreads();
        view.for_all([&](int, float x) {
          const float w = weight_of(x);
          const unsigned key = __float_as_uint(w);
          if (w > 0.0f && (key & mask) == prefix) {
            const unsigned long long fx = __float2ull_rn(w * 8589934592.0f);
            unsigned* h = s_hist + ((key >> shift) & (n_digits - 1));
            atomicAdd(h, (unsigned)(fx & 2047u));
            atomicAdd(h + DIGITS0, (unsigned)((fx >> 11) & 2047u));
            atomicAdd(h + 2 * DIGITS0, (unsigned)(fx >> 22));
          }
        });
        __syncthreads();
        auto mass = [&](int d) {
          return ((unsigned long long)s_hist[2 * DIGITS0 + d] << 22) + ((unsigned long long)s_hist[DIGITS0 + d] << 11) +
                 (unsigned long long)s_hist[d];
        };
        if (pass == 0) {   // the first pass has seen every weight: the mass to reach
          unsigned dummy;
          unsigned long long all;
          pick_digit(mass, n_digits / THREADS, 0ull, ~0ull, s_warp_tot, &s_pick, &s_above, dummy, all);
          all += mass(0);
          target = (unsigned long long)((double)top_p * (double)all);
        }
        unsigned digit;
        pick_digit(mass, n_digits / THREADS, above, target, s_warp_tot, &s_pick, &s_above, digit, above);
        prefix |= digit << shift;
        mask |= (unsigned)(n_digits - 1) << shift;
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
    auto four = [&](int v0, float* w) {   // the kept weights of indices v0 .. v0 + 3
      if (view.vectors()) {
        float4 x = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        if (v0 < V) x = view.at4(v0);
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
  // shared memory (used when temperature > 0): the radix select's histograms and the sums of the pieces of
  // 128 indices
  const size_t smem = temperature > 0.0f ? 3 * DIGITS0 * sizeof(unsigned) +
                                               (size_t)((V + 4 * THREADS - 1) / (4 * THREADS)) * (THREADS / 32) * sizeof(float)
                                         : 0;
  JB_REFUSE(smem > 200 * 1024, "sample: a vocabulary of %d is too large for temperature sampling", V);
  if (smem > 48 * 1024) {   // the limit is raised per device, the first time a launch on it needs more
    static size_t smem_allowed[64];
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= 64 || smem > smem_allowed[device]) {
      e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      if (device >= 0 && device < 64) smem_allowed[device] = smem;
    }
  }
  sample_kernel<<<B, THREADS, smem, stream>>>(logits, V, out_ids, temperature, top_k, top_p, penalty, counts,
                                              count_rows, seed, seq_ids, steps, feedback);
  JB_CHECK_LAUNCH();
  return 0;
}
