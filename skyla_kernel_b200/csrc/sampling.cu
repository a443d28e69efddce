// Next-token choice on the device, one block per row of 32-bit logits.
//   greedy      : argmax; among equal maxima the lowest index (the reference's
//                 host argmax, skyla-ref/src/ops.rs:36-41, meets no exact ties
//                 with real logits)
//   temperature : z = logit / T, optional top-k then top-p filter (the options
//                 of the reference's chat sampler, docs/roadmap.md:282-283),
//                 then one draw from softmax(z) over the kept set.
// The draw is Gumbel-max, argmax_i (z_i - log(-log u_i)), with u_i a hash of
// (seed, request id, step, i): a request's draws depend on nothing else, so
// its tokens do not change with the batch it is in, and the result needs no
// ordered prefix sum.  Filters are thresholds found by bisection on the bit
// pattern of z, with block sums in a fixed order: no atomics, same result on
// every run.
//   top-k : keep z_i >= the k-th largest value (ties at the edge all stay)
//   top-p : with e_i = exp(z_i - max) over the top-k set, keep z_i >= tau, tau
//           the largest value with sum_{z_i >= tau} e_i >= p * sum e_i
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float uniform01(uint32_t seed_lo, uint32_t seed_hi, uint32_t req,
                                           uint32_t step, uint32_t i) {
  uint32_t h = mix32(seed_lo ^ 0x9e3779b9u);
  h = mix32(h ^ seed_hi);
  h = mix32(h ^ req);
  h = mix32(h ^ step);
  h = mix32(h ^ i);
  return ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}
// order-preserving map from float to unsigned
__device__ __forceinline__ uint32_t ordered(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best { float v; int i; };
__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ Best block_argmax(Best b, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
    b = better(b, other);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = b;
  __syncthreads();
  Best r = scratch[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = better(r, scratch[w]);
  return r;
}
__device__ float block_sum_f(float v, float* scratch) { return block_sum(v, scratch); }

// A row in which no logit compares (all NaN) leaves no candidate: the token is then 0, never an
// index outside the vocabulary (the next step would read the embedding table there), and the
// device's error word is raised (code 31) for the host to find.
constexpr int kNoTokenCode = 31;
__device__ __forceinline__ int checked(int token, int vocab, int* error_flag) {
  if (token >= 0 && token < vocab) return token;
  if (error_flag != nullptr) atomicCAS(error_flag, 0, kNoTokenCode);
  return 0;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t ld, int vocab, float temperature, int top_k,
              float top_p, uint32_t seed_lo, uint32_t seed_hi, const int32_t* __restrict__ req_ids,
              const int32_t* __restrict__ steps, int32_t* __restrict__ out, int* error_flag) {
  __shared__ Best bscratch[32];
  __shared__ float fscratch[32];
  const int r = blockIdx.x;
  const float* row = logits + (int64_t)r * ld;
  const int tid = threadIdx.x;

  if (!(temperature > 0.f)) {
    Best b{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += kThreads) b = better(b, Best{row[i], i});
    b = block_argmax(b, bscratch);
    if (tid == 0) out[r] = checked(b.i, vocab, error_flag);
    return;
  }
  uint32_t tau = 0;  // keep ordered(z_i) >= tau
  if (top_k > 0 && top_k < vocab) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = tau | (1u << bit);
      float n = 0.f;  // counts up to 2^24 are exact in 32-bit floating point
      for (int i = tid; i < vocab; i += kThreads) n += ordered(row[i] / temperature) >= cand ? 1.f : 0.f;
      if (block_sum_f(n, fscratch) >= (float)top_k) tau = cand;
    }
  }
  if (top_p < 1.f) {
    Best b{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += kThreads) b = better(b, Best{row[i] / temperature, i});
    const float zmax = block_argmax(b, bscratch).v;
    float s = 0.f;
    for (int i = tid; i < vocab; i += kThreads) {
      const float z = row[i] / temperature;
      if (ordered(z) >= tau) s += expf(z - zmax);
    }
    const float target = top_p * block_sum_f(s, fscratch);
    uint32_t t2 = 0;  // the largest threshold whose kept mass still reaches the target
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = t2 | (1u << bit);
      const uint32_t thr = cand > tau ? cand : tau;
      float part = 0.f;
      for (int i = tid; i < vocab; i += kThreads) {
        const float z = row[i] / temperature;
        if (ordered(z) >= thr) part += expf(z - zmax);
      }
      if (block_sum_f(part, fscratch) >= target) t2 = cand;
    }
    tau = t2 > tau ? t2 : tau;
  }
  Best b{-INFINITY, 0x7fffffff};
  const uint32_t req = (uint32_t)req_ids[r], step = (uint32_t)steps[r];
  for (int i = tid; i < vocab; i += kThreads) {
    const float z = row[i] / temperature;
    if (ordered(z) < tau) continue;
    const float u = uniform01(seed_lo, seed_hi, req, step, (uint32_t)i);
    b = better(b, Best{z - logf(-logf(u)), i});
  }
  b = block_argmax(b, bscratch);
  if (tid == 0) out[r] = checked(b.i, vocab, error_flag);
}
}  // namespace

extern "C" int skyla_sample(const float* logits, int64_t ld, int n_rows, int vocab, float temperature,
                            int top_k, float top_p, uint64_t seed, const int32_t* req_ids,
                            const int32_t* steps, int32_t* out, int* error_flag, cudaStream_t stream) {
  if (n_rows <= 0) return kOk;
  if (vocab <= 0 || ld < vocab) return fail(kBadArgument, "sample: bad vocabulary %d", vocab);
  if (vocab > (1 << 24)) return fail(kBadArgument, "sample: vocabulary %d above 2^24", vocab);
  if (!(top_p > 0.f)) return fail(kBadArgument, "sample: top_p must be in (0, 1]");
  if (temperature > 0.f && (req_ids == nullptr || steps == nullptr))
    return fail(kBadArgument, "sample: a random draw needs request ids and steps");
  sample_kernel<<<n_rows, kThreads, 0, stream>>>(logits, ld, vocab, temperature, top_k, top_p,
                                                (uint32_t)seed, (uint32_t)(seed >> 32), req_ids,
                                                steps, out, error_flag);
  return check_launch("sample");
}
