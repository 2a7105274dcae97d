// Shared helpers for the sm_100a kernels of this engine.
//
// Every launcher is an extern "C" function over raw device pointers and a
// stream; it returns 0 on success or a negative code for a refused argument
// (see SB_ERR_*), or the positive cudaError_t of a failed launch. Activations
// and weights are float (dtype code 0) or __nv_bfloat16 (dtype code 1); the
// residual stream, softmax statistics, norms, rotation angles and logits are
// float in both modes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SB_DTYPE_F32 0
#define SB_DTYPE_BF16 1

#define SB_ERR_DTYPE (-1)      // unsupported dtype code
#define SB_ERR_SHAPE (-2)      // a size the kernel refuses
#define SB_ERR_ALIGN (-3)      // a pointer or stride not aligned as the kernel needs
#define SB_ERR_LIMIT (-4)      // a size beyond a stated maximum

#define SB_EXPORT extern "C" __attribute__((visibility("default")))

#define SB_LAUNCH_CHECK()                      \
  do {                                         \
    cudaError_t e_ = cudaGetLastError();       \
    if (e_ != cudaSuccess) return (int)e_;     \
  } while (0)

#include <stdlib.h>

namespace sb {

// Programmatic dependent launch: a kernel launched through launch_pdl may start while its predecessor in the
// stream is still running. It must call pdl_wait() before it reads anything an earlier kernel wrote, and before
// it writes anything an earlier kernel may still read; what it does before that (fetching weights and tables the
// step does not change, computing addresses) overlaps with the predecessor's tail. pdl_launch_dependents() lets
// the successor be scheduled as early as possible. Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool pdl_enabled() {
  static const bool on = (getenv("SERVE_B200_NO_PDL") == nullptr);
  return on;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define SB_PDL_CHECK(expr)                        \
  do {                                            \
    cudaError_t e_ = (expr);                      \
    if (e_ != cudaSuccess) return (int)e_;        \
  } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// The order of additions depends only on blockDim, never on the batch.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (lane < nwarps) ? smem32[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// SMs of the current device (asked of the driver once per device and kept; 148 on a B200).
static inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace sb
