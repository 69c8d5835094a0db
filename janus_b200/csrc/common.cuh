// Shared helpers of the janus_b200 kernels (sm_100a only).
//
// Every exported function is `extern "C"`, takes raw device pointers and a
// stream, launches on that stream and returns 0 or an error code; it never
// allocates and never synchronises.  Element types are passed as codes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define JB_F32 0
#define JB_BF16 1

// Error codes above any cudaError_t value.
#define JB_ERR_BAD_SIZE 10001     // a size the kernel cannot take (message printed to stderr)
#define JB_ERR_BAD_DTYPE 10002
#define JB_ERR_TENSORMAP 10003

#define JB_EXPORT extern "C" __attribute__((visibility("default")))

#define JB_CHECK_LAUNCH()                                   \
  do {                                                      \
    cudaError_t e_ = cudaGetLastError();                    \
    if (e_ != cudaSuccess) return (int)e_;                  \
  } while (0)

#define JB_REFUSE(cond, ...)                                \
  do {                                                      \
    if (cond) {                                             \
      fprintf(stderr, "janus_b200 kernel refused: ");       \
      fprintf(stderr, __VA_ARGS__);                         \
      fprintf(stderr, "\n");                                \
      return JB_ERR_BAD_SIZE;                               \
    }                                                       \
  } while (0)

namespace jb {

// ---- programmatic dependent launch ------------------------------------------------
// Every kernel of this library is launched so that it may start while the kernel
// before it in the stream is still running (`Launch` below).  A kernel first lets
// its own successor start (`pdl_launch_dependents`), does what does not depend on
// earlier kernels (barrier set-up, TMEM allocation, loading weights), and calls
// `pdl_wait` in EVERY thread before it touches anything an earlier kernel wrote.
// Because each kernel waits before it finishes, completion is transitive along the
// stream.  JANUS_PDL=0 in the environment turns the launch attribute off.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("JANUS_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

struct Launch {
  cudaLaunchConfig_t c;
  cudaLaunchAttribute attr[1];
  Launch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    c = cudaLaunchConfig_t{};
    c.gridDim = grid;
    c.blockDim = block;
    c.dynamicSmemBytes = smem;
    c.stream = stream;
    c.attrs = nullptr;
    c.numAttrs = 0;
    if (pdl_enabled()) {
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      c.attrs = attr;
      c.numAttrs = 1;
    }
  }
  Launch(const Launch&) = delete;
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace jb
