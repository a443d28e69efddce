// Plain attention over the paged cache, one warp per (token, query head):
//   s_p = dot(q, K[p]) * scale for the positions p this token may see (all
//   p <= its own, or the last `window` of them), softmax with the maximum
//   subtracted, o = sum_p w_p V[p]   (skyla-ref/src/model.rs:149-165,
//   skyla-ref/src/ops.rs:18-26).
// Keys are taken 32 at a time, aligned to absolute positions, with an online
// softmax between groups as in the reference's GPU kernel
// (skyla-shaders/shaders/attention.comp:81-99).  Query head h reads KV head
// h / (nq / nkv).  The same kernel serves prompts and single tokens, so a
// token's result depends only on its own query and its own cache: it is the
// attention of the true 32-bit path and the reference twin of the fast kernels.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 512;
constexpr int kMaxPerLane = kMaxHeadDim / 32;

struct AttnArgs {
  const void* q; int64_t ldq; void* out; int64_t ldo;
  int n_tokens, nq, nkv, hd;
  const void* k_pool; const void* v_pool; const int32_t* page_table; int max_pages, page_size;
  const int32_t* tok_pos; const int32_t* tok_slot;
  float scale; int window;
};

template <typename TA, typename TC>
__global__ void __launch_bounds__(kWarps * 32) attention_plain_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.x * kWarps + warp, t = blockIdx.y;
  if (h >= a.nq) return;
  const int hd = a.hd, kvh = h / (a.nq / a.nkv);
  float* qs = smem + warp * hd;
  const TA* q = (const TA*)a.q + (int64_t)t * a.ldq + (int64_t)h * hd;
  for (int e = lane; e < hd; e += 32) qs[e] = to_float(q[e]);
  __syncwarp();
  const int pos = a.tok_pos[t];
  const int32_t* pages = a.page_table + (int64_t)a.tok_slot[t] * a.max_pages;
  const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;

  float m = -INFINITY, l = 0.f, acc[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) acc[i] = 0.f;
  const int n_per_lane = (hd + 31) / 32;

  for (int p0 = first / 32 * 32; p0 <= pos; p0 += 32) {
    const int p = p0 + lane;
    const bool live = p >= first && p <= pos;
    float s = -INFINITY;
    const TC* vrow = nullptr;
    if (live) {
      const int64_t row = ((int64_t)pages[p / a.page_size] * a.nkv + kvh) * a.page_size + p % a.page_size;
      const TC* k = (const TC*)a.k_pool + row * hd;
      vrow = (const TC*)a.v_pool + row * hd;
      float d = 0.f;
      for (int e = 0; e < hd; ++e) d = fmaf(qs[e], to_float(k[e]), d);
      s = d * a.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));  // at least one key of a group is live
    const float c = expf(m - m_new);            // exp(-inf) = 0 on the first group
    const float w = live ? expf(s - m_new) : 0.f;
    l = l * c + warp_sum(w);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) acc[i] *= c;
    for (int j = 0; j < 32; ++j) {
      const float wj = __shfl_sync(0xffffffffu, w, j);
      const unsigned long long vj = __shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
      if (vj == 0) continue;  // uniform across the warp
      const TC* v = (const TC*)vj;
#pragma unroll
      for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (i < n_per_lane && e < hd) acc[i] = fmaf(wj, to_float(v[e]), acc[i]);
      }
    }
  }
  TA* o = (TA*)a.out + (int64_t)t * a.ldo + (int64_t)h * hd;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    if (i < n_per_lane && e < hd) o[e] = from_float<TA>(acc[i] / l);
  }
}
}  // namespace

extern "C" int skyla_attention_plain(
    const void* q, int act_dtype, int64_t ldq, void* out, int64_t ldo, int n_tokens, int nq, int nkv,
    int hd, const void* k_pool, const void* v_pool, int cache_dtype, const int32_t* page_table,
    int max_pages, int page_size, const int32_t* tok_pos, const int32_t* tok_slot, float scale,
    int window, cudaStream_t stream) {
  if (n_tokens <= 0) return kOk;
  if (hd <= 0 || hd > kMaxHeadDim) return fail(kBadArgument, "attention_plain: head size %d is outside 1..%d", hd, kMaxHeadDim);
  if (nkv <= 0 || nq % nkv) return fail(kBadArgument, "attention_plain: %d query heads do not divide into %d key/value heads", nq, nkv);
  if (n_tokens > 65535) return fail(kBadArgument, "attention_plain: %d tokens exceed the grid", n_tokens);
  AttnArgs a{q, ldq, out, ldo, n_tokens, nq, nkv, hd, k_pool, v_pool, page_table, max_pages,
             page_size, tok_pos, tok_slot, scale, window};
  dim3 grid((nq + kWarps - 1) / kWarps, n_tokens);
  const size_t smem = (size_t)kWarps * hd * sizeof(float);
  SKYLA_DISPATCH(act_dtype, TA, SKYLA_DISPATCH(cache_dtype, TC, {
    attention_plain_kernel<TA, TC><<<grid, kWarps * 32, smem, stream>>>(a);
  }););
  return check_launch("attention_plain");
}
