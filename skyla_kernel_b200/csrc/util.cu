// Utilities that are not part of a model step.
//  * bandwidth probe: a streaming read of a buffer, XOR-folded per thread, with
//    a store that only an impossible value triggers so that the read cannot be
//    elided (skyla-shaders/shaders/bandwidth.comp:10-23); it gives the measured
//    read roofline that the memory-bound kernels are judged against
//    (docs/roadmap.md:46-47,184-195).
//  * normal fill: random weights in place on the device, N(mean, std) from a
//    hash of (seed, element index) by Box-Muller, for models that are too large
//    to draw on the host.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
__global__ void __launch_bounds__(256) bandwidth_kernel(const uint4* __restrict__ src, size_t n_vec,
                                                        uint32_t* __restrict__ sink) {
  uint4 acc = make_uint4(0, 0, 0, 0);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // eight loads of a thread are in flight at a time: the memory's latency is what a stream has to cover
  for (; i + 7 * stride < n_vec; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __ldcs(src + i + k * stride);
#pragma unroll
    for (int k = 0; k < 8; ++k) { acc.x ^= v[k].x; acc.y ^= v[k].y; acc.z ^= v[k].z; acc.w ^= v[k].w; }
  }
  for (; i < n_vec; i += stride) {
    const uint4 v = __ldcs(src + i);
    acc.x ^= v.x; acc.y ^= v.y; acc.z ^= v.z; acc.w ^= v.w;
  }
  const uint32_t f = acc.x ^ acc.y ^ acc.z ^ acc.w;
  if (f == 0x9e3779b1u && sink != nullptr) sink[0] = f;  // all-equal inputs never fold to this
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

template <typename T>
__global__ void __launch_bounds__(256) fill_normal_kernel(T* __restrict__ out, size_t n, float mean,
                                                          float std, uint32_t seed_lo, uint32_t seed_hi) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const uint32_t base = mix32(mix32(seed_lo ^ 0x9e3779b9u) ^ seed_hi);
  for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; 2 * p < n; p += stride) {
    const uint32_t a = mix32(base ^ (uint32_t)p), b = mix32(a ^ (uint32_t)(p >> 32) ^ 0x85ebca6bu);
    const uint32_t c = mix32(b + 0x68e31da4u);
    const float u1 = ((float)(b >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = ((float)(c >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float rad = sqrtf(-2.0f * logf(u1));
    float s, co;
    sincospif(2.0f * u2, &s, &co);
    out[2 * p] = from_float<T>(mean + std * rad * co);
    if (2 * p + 1 < n) out[2 * p + 1] = from_float<T>(mean + std * rad * s);
  }
}
}  // namespace

// Reads `bytes` (a multiple of 16) from `src` once.
extern "C" int skyla_bandwidth_read(const void* src, size_t bytes, int blocks, uint32_t* sink,
                                    cudaStream_t stream) {
  if (bytes % 16 || ((uintptr_t)src) % 16) return fail(kBadArgument, "bandwidth_read: buffer not in 16-byte units");
  if (blocks <= 0) return fail(kBadArgument, "bandwidth_read: no blocks");
  bandwidth_kernel<<<blocks, 256, 0, stream>>>((const uint4*)src, bytes / 16, sink);
  return check_launch("bandwidth_read");
}

extern "C" int skyla_fill_normal(void* out, int dtype, size_t n, float mean, float std, uint64_t seed,
                                 cudaStream_t stream) {
  if (n == 0) return kOk;
  const size_t pairs = (n + 1) / 2;
  const int blocks = (int)((pairs + 255) / 256 < 148 * 16 ? (pairs + 255) / 256 : 148 * 16);
  SKYLA_DISPATCH(dtype, T, {
    fill_normal_kernel<T><<<blocks, 256, 0, stream>>>((T*)out, n, mean, std, (uint32_t)seed,
                                                      (uint32_t)(seed >> 32));
  });
  return check_launch("fill_normal");
}
