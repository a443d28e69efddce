// Shared helpers of the hand-written sm_100a kernels: element types, error
// reporting, reductions.  Every launcher is an extern "C" function that takes
// raw device pointers and a stream, launches, and returns 0 or an error code
// whose text skyla_error_message() gives; nothing here allocates memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <utility>

namespace skyla {

enum DType : int { kF32 = 0, kBF16 = 1 };

constexpr int kOk = 0;
constexpr int kBadArgument = -1;   // a size or dtype the kernel refuses
constexpr int kLaunchFailed = -2;  // the CUDA runtime refused the launch

inline char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

template <typename... A>
inline int fail(int code, const char* fmt, A... a) {
  snprintf(error_buffer(), 512, fmt, a...);
  return code;
}
inline int fail(int code, const char* msg) {
  snprintf(error_buffer(), 512, "%s", msg);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kLaunchFailed, "%s: %s", what, cudaGetErrorString(e));
  return kOk;
}

// Programmatic dependent launch: a kernel launched through launch_overlapped() may
// start while the kernel before it in the stream is still running.  It must call
// grid_dependency_wait() before it reads anything an earlier kernel wrote and before
// it writes anything at all (an earlier kernel may still be reading it); what it does
// before that (set up barriers, allocate tensor memory, prefetch weights that no
// kernel writes) overlaps with its predecessor.  allow_dependents() lets the next
// kernel be scheduled as soon as every block of this one has got that far.  Without
// the launch attribute both are no-ops.  SKYLA_NO_PDL=1 turns the attribute off.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool overlap_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("SKYLA_NO_PDL");
    on = (e != nullptr && e[0] == '1') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);  // errors are read by check_launch()
}

// The same for a kernel whose blocks form clusters of `cluster_z` along the grid's z axis.
template <typename... KArgs, typename... Args>
inline void launch_overlapped_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, unsigned cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster_z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Sum over the 32 lanes with a fixed butterfly: the same order for every warp
// and every launch, so results do not depend on what else is in the batch.
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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < n_warps; ++i) t += scratch[i];
  return t;
}

}  // namespace skyla

// Calls `BODY` with `T` bound to the C++ type of a dtype code.
#define SKYLA_DISPATCH(code, T, ...)                                       \
  do {                                                                     \
    if ((code) == skyla::kF32) {                                           \
      using T = float;                                                     \
      __VA_ARGS__                                                          \
    } else if ((code) == skyla::kBF16) {                                   \
      using T = __nv_bfloat16;                                             \
      __VA_ARGS__                                                          \
    } else {                                                               \
      return skyla::fail(skyla::kBadArgument, "unknown dtype code %d", (int)(code)); \
    }                                                                      \
  } while (0)

#define SKYLA_EXPORT_ERROR_MESSAGE() \
  extern "C" const char* skyla_error_message() { return skyla::error_buffer(); }
