// RMSNorm over rows: r = 1/sqrt(mean(x^2)+eps); y = (x*r)*w, all in 32-bit
// (skyla-ref/src/ops.rs:1-16; GPU twin skyla-shaders/shaders/rmsnorm.comp:22-51).
// An optional row list turns it into "gather the wanted rows, then norm", which
// is what the reference does with take_last before the output head
// (skyla-engine/src/graph.rs:219-229).
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

template <typename TI, typename TO>
__global__ void rmsnorm_kernel(const TI* __restrict__ x, int64_t ldx, const int32_t* __restrict__ rows,
                               int width, const float* __restrict__ w, float eps,
                               TO* __restrict__ out, int64_t ldo) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const TI* xr = x + (int64_t)(rows ? rows[r] : r) * ldx;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(xr[i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  TO* o = out + (int64_t)r * ldo;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = from_float<TO>(to_float(xr[i]) * inv * w[i]);
}

// float32 rows whose width is a multiple of 4 and that start on 16 bytes: four elements per load,
// kept in registers between the two passes (up to kKeep loads a thread; wider rows are read again),
// four bfloat16 per store.
constexpr int kKeep = 4;
__global__ void rmsnorm_vec4_kernel(const float* __restrict__ x, int64_t ldx, const int32_t* __restrict__ rows,
                                    int width, const float* __restrict__ w, float eps,
                                    __nv_bfloat16* __restrict__ out, int64_t ldo) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)(rows ? rows[r] : r) * ldx);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const int n4 = width / 4;
  float4 keep[kKeep];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < n4) {
      const float4 v = xr[i];
      keep[j] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  }
  for (int i = threadIdx.x + kKeep * blockDim.x; i < n4; i += blockDim.x) {
    const float4 v = xr[i];
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (int64_t)r * ldo);
  auto put = [&](int i, const float4& v) {
    const float4 g = wr[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * inv * g.x, v.y * inv * g.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * inv * g.z, v.w * inv * g.w);
    o[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  };
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < n4) put(i, keep[j]);
  }
  for (int i = threadIdx.x + kKeep * blockDim.x; i < n4; i += blockDim.x) put(i, xr[i]);
}

extern "C" int skyla_rmsnorm(const void* x, int x_dtype, int64_t ldx, const int32_t* rows,
                             int n_rows, int width, const float* weight, float eps, void* out,
                             int out_dtype, int64_t ldo, cudaStream_t stream) {
  if (n_rows <= 0) return kOk;
  if (width <= 0 || ldx < width || ldo < width)
    return fail(kBadArgument, "rmsnorm: bad width %d or row stride", width);
  // the block size depends on the width only, so a row's sum has one order whatever the batch
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  // the vector kernel adds a row's squares in another order than the scalar one: it serves the
  // 16-bit path only, so that the 32-bit path keeps one order for every way of calling it
  if (x_dtype == kF32 && out_dtype == kBF16 && width % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 &&
      ((uintptr_t)x) % 16 == 0 && ((uintptr_t)weight) % 16 == 0 && ((uintptr_t)out) % 8 == 0) {
    // few threads a row where the row is short, so that every thread has a load or two in flight
    const int vthreads = width >= 4096 ? 256 : 128;
    launch_overlapped(rmsnorm_vec4_kernel, dim3(n_rows), dim3(vthreads), 0, stream, (const float*)x, ldx,
                      rows, width, weight, eps, (__nv_bfloat16*)out, ldo);
    return check_launch("rmsnorm");
  }
  SKYLA_DISPATCH(x_dtype, TI, SKYLA_DISPATCH(out_dtype, TO, {
    launch_overlapped(rmsnorm_kernel<TI, TO>, dim3(n_rows), dim3(threads), 0, stream, (const TI*)x, ldx, rows, width,
                      weight, eps, (TO*)out, ldo);
  }););
  return check_launch("rmsnorm");
}
