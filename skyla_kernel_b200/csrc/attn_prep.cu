// Per-head preparation of a step's new tokens, one warp per (token, head):
//   q, k heads: RMSNorm over the head with one [head_dim] weight shared by all
//               heads (skyla-ref/src/ops.rs:8-11, model.rs:138-145), then
//               rotate-half RoPE on the first n_rot elements at the token's
//               absolute position (skyla-ref/src/rope.rs:59-68);
//   q is written back in place, k and v go to the token's place in the paged
//   cache (the reference's qkv_prep does the same into its flat cache,
//   skyla-shaders/shaders/qkv_prep.comp:67-123).
// Norm and rotation are optional (null weight / null table), so a mixer that
// uses neither, or another position encoding applied elsewhere, can share it.
// All arithmetic is 32-bit; cos/sin come from a table built once on the host.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 512;

struct PrepArgs {
  const void* qkv; int64_t ld; int q_off, k_off, v_off;
  void* q_out; int64_t ldq;            // where the prepared queries go (may be the input itself)
  int n_tokens, nq, nkv, hd;
  const float* q_norm; const float* k_norm; float eps;
  const float* cos_t; const float* sin_t; int n_rot;
  const int32_t* tok_pos; const int32_t* tok_slot;
  void* k_pool; void* v_pool; const int32_t* page_table; int max_pages; int page_size;
};

template <typename TI, typename TA, typename TC>
__global__ void __launch_bounds__(kWarps * 32) prep_kernel(PrepArgs a) {
  extern __shared__ float smem[];
  allow_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.x * kWarps + warp;
  const int t = blockIdx.y;
  const int n_heads = a.nq + 2 * a.nkv;
  if (head >= n_heads) return;
  float* u = smem + warp * a.hd;
  const int hd = a.hd;
  const bool is_q = head < a.nq, is_k = !is_q && head < a.nq + a.nkv;
  const int kvh = is_q ? 0 : (is_k ? head - a.nq : head - a.nq - a.nkv);
  const TI* src = (const TI*)a.qkv + (int64_t)t * a.ld +
                  (is_q ? a.q_off + head * hd : (is_k ? a.k_off : a.v_off) + kvh * hd);
  auto load = [&](int e) { return to_float(src[e]); };
  const int pos = a.tok_pos[t];

  TC* dst = nullptr;
  if (!is_q) {
    if (a.k_pool == nullptr) return;  // this run reads another entry's cache
    const int page = a.page_table[(int64_t)a.tok_slot[t] * a.max_pages + pos / a.page_size];
    TC* pool = (TC*)(is_k ? a.k_pool : a.v_pool);
    dst = pool + (((int64_t)page * a.nkv + kvh) * a.page_size + pos % a.page_size) * hd;
  }
  if (!is_q && !is_k) {  // v: a copy
    for (int e = lane; e < hd; e += 32) dst[e] = from_float<TC>(load(e));
    return;
  }
  const float* nw = is_q ? a.q_norm : a.k_norm;
  float ss = 0.f;
  for (int e = lane; e < hd; e += 32) {
    const float v = load(e);
    u[e] = v;
    ss = fmaf(v, v, ss);
  }
  if (nw != nullptr) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hd + a.eps);
    for (int e = lane; e < hd; e += 32) u[e] *= inv * nw[e];
  }
  __syncwarp();
  const int half = a.n_rot / 2;
  for (int e = lane; e < hd; e += 32) {
    float v = u[e];
    if (a.cos_t != nullptr && e < a.n_rot) {
      const int i = e < half ? e : e - half;
      const float c = a.cos_t[(int64_t)pos * half + i], s = a.sin_t[(int64_t)pos * half + i];
      const float x0 = u[i], x1 = u[i + half];
      v = e < half ? x0 * c - x1 * s : x0 * s + x1 * c;
    }
    if (is_q) ((TA*)a.q_out)[(int64_t)t * a.ldq + head * hd + e] = from_float<TA>(v);
    else dst[e] = from_float<TC>(v);
  }
}
// The common case on prompts: bfloat16 in and out, one split, the whole head rotates and its
// size is a multiple of 32.  A lane owns hd/32 consecutive elements, so lanes 0-15 hold the
// first half of the head and lane l+16 holds the rotation partners of lane l: loads and stores
// are contiguous and the partner comes by one shuffle.
constexpr int kHeadsPerWarp = 4;  // a warp finishes this many heads of one token: their loads are in flight together
template <int EPL>  // elements per lane
__global__ void __launch_bounds__(kWarps * 32) prep_bf16_kernel(PrepArgs a) {
  allow_dependents();
  grid_dependency_wait();
  typedef __nv_bfloat16 bf16;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head0 = (blockIdx.x * kWarps + warp) * kHeadsPerWarp, t = blockIdx.y;
  const int hd = a.hd, n_heads = a.nq + 2 * a.nkv;
  if (head0 >= n_heads) return;
  const int pos = a.tok_pos[t];
  const int page = a.k_pool != nullptr
                       ? a.page_table[(int64_t)a.tok_slot[t] * a.max_pages + pos / a.page_size] : 0;
  const bf16* src[kHeadsPerWarp];
  bf16* dst[kHeadsPerWarp];
  int kind[kHeadsPerWarp];  // 0 query, 1 key, 2 value, 3 nothing to do
  bf16 raw[kHeadsPerWarp][EPL];
#pragma unroll
  for (int h = 0; h < kHeadsPerWarp; ++h) {
    const int head = head0 + h;
    const bool is_q = head < a.nq, is_k = !is_q && head < a.nq + a.nkv;
    const int kvh = is_q ? 0 : (is_k ? head - a.nq : head - a.nq - a.nkv);
    kind[h] = head >= n_heads ? 3 : (is_q ? 0 : (a.k_pool == nullptr ? 3 : (is_k ? 1 : 2)));
    src[h] = (const bf16*)a.qkv + (int64_t)t * a.ld +
             (is_q ? a.q_off + head * hd : (is_k ? a.k_off : a.v_off) + kvh * hd) + lane * EPL;
    dst[h] = is_q ? (bf16*)a.q_out + (int64_t)t * a.ldq + head * hd + lane * EPL
                  : (bf16*)(is_k ? a.k_pool : a.v_pool) +
                        (((int64_t)page * a.nkv + kvh) * a.page_size + pos % a.page_size) * hd + lane * EPL;
    if (kind[h] == 3) continue;
    if (EPL == 4) *reinterpret_cast<uint2*>(raw[h]) = *reinterpret_cast<const uint2*>(src[h]);
    else if (EPL == 2) *reinterpret_cast<uint32_t*>(raw[h]) = *reinterpret_cast<const uint32_t*>(src[h]);
    else if (EPL == 8) *reinterpret_cast<uint4*>(raw[h]) = *reinterpret_cast<const uint4*>(src[h]);
    else
#pragma unroll
      for (int i = 0; i < EPL; ++i) raw[h][i] = src[h][i];
  }
  // the rotation of this lane's pairs, the same for every head of the token
  float cs[EPL], sn[EPL];
  if (a.cos_t != nullptr) {
    const int half = hd / 2;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int j = (lane & 15) * EPL + i;  // index of the pair
      cs[i] = a.cos_t[(int64_t)pos * half + j];
      sn[i] = a.sin_t[(int64_t)pos * half + j];
    }
  }
#pragma unroll
  for (int h = 0; h < kHeadsPerWarp; ++h) {
    if (kind[h] == 3) continue;
    if (kind[h] < 2) {
      float u[EPL];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) { u[i] = __bfloat162float(raw[h][i]); ss = fmaf(u[i], u[i], ss); }
      const float* nw = kind[h] == 0 ? a.q_norm : a.k_norm;
      if (nw != nullptr) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hd + a.eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i) u[i] *= inv * nw[lane * EPL + i];
      }
      if (a.cos_t != nullptr) {
        const bool low = lane < 16;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, u[i], 16);
          u[i] = low ? u[i] * cs[i] - other * sn[i] : other * sn[i] + u[i] * cs[i];
        }
      }
#pragma unroll
      for (int i = 0; i < EPL; ++i) raw[h][i] = __float2bfloat16_rn(u[i]);
    }
    if (EPL == 4) *reinterpret_cast<uint2*>(dst[h]) = *reinterpret_cast<uint2*>(raw[h]);
    else if (EPL == 2) *reinterpret_cast<uint32_t*>(dst[h]) = *reinterpret_cast<uint32_t*>(raw[h]);
    else if (EPL == 8) *reinterpret_cast<uint4*>(dst[h]) = *reinterpret_cast<uint4*>(raw[h]);
    else
#pragma unroll
      for (int i = 0; i < EPL; ++i) dst[h][i] = raw[h][i];
  }
}
}  // namespace

// qkv: [tokens][ld]; the prepared queries go to q_out [tokens][ldq] (heads contiguous), which may
// alias the q columns of qkv.
extern "C" int skyla_qk_norm_rope_cache(
    const void* qkv, int in_dtype, int64_t ld, void* q_out,
    int act_dtype, int64_t ldq, int q_off, int k_off, int v_off, int n_tokens, int nq,
    int nkv, int hd, const float* q_norm, const float* k_norm, float eps, const float* cos_t,
    const float* sin_t, int n_rot, const int32_t* tok_pos, const int32_t* tok_slot, void* k_pool,
    void* v_pool, int cache_dtype, const int32_t* page_table, int max_pages, int page_size,
    cudaStream_t stream) {
  if (n_tokens <= 0) return kOk;
  if (hd <= 0 || hd > kMaxHeadDim) return fail(kBadArgument, "qk_norm_rope_cache: head size %d is outside 1..%d", hd, kMaxHeadDim);
  if (n_rot < 0 || n_rot > hd || n_rot % 2) return fail(kBadArgument, "qk_norm_rope_cache: rotary width %d does not fit head size %d", n_rot, hd);
  if (n_tokens > 65535) return fail(kBadArgument, "qk_norm_rope_cache: %d tokens exceed the grid", n_tokens);
  PrepArgs a{qkv, ld, q_off, k_off, v_off, q_out, ldq, n_tokens, nq, nkv, hd, q_norm, k_norm, eps, cos_t, sin_t,
             n_rot, tok_pos, tok_slot, k_pool, v_pool, page_table, max_pages, page_size};
  dim3 grid((nq + 2 * nkv + kWarps - 1) / kWarps, n_tokens);
  const size_t smem = (size_t)kWarps * hd * sizeof(float);
  if (in_dtype == kBF16 && act_dtype == kBF16 && (k_pool == nullptr || cache_dtype == kBF16) && hd % 32 == 0 && hd <= 256 && (cos_t == nullptr || n_rot == hd) &&
      ld % 8 == 0 && ldq % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
      ((uintptr_t)qkv) % 16 == 0 && ((uintptr_t)q_out) % 16 == 0) {
    const dim3 gridf((nq + 2 * nkv + kWarps * kHeadsPerWarp - 1) / (kWarps * kHeadsPerWarp), n_tokens);
    switch (hd / 32) {
      case 1: launch_overlapped(prep_bf16_kernel<1>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      case 2: launch_overlapped(prep_bf16_kernel<2>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      case 3: launch_overlapped(prep_bf16_kernel<3>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      case 4: launch_overlapped(prep_bf16_kernel<4>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      case 5: launch_overlapped(prep_bf16_kernel<5>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      case 6: launch_overlapped(prep_bf16_kernel<6>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      case 7: launch_overlapped(prep_bf16_kernel<7>, gridf, dim3(kWarps * 32), 0, stream, a); break;
      default: launch_overlapped(prep_bf16_kernel<8>, gridf, dim3(kWarps * 32), 0, stream, a); break;
    }
    return check_launch("qk_norm_rope_cache");
  }
  SKYLA_DISPATCH(in_dtype, TI, SKYLA_DISPATCH(act_dtype, TA, SKYLA_DISPATCH(cache_dtype, TC, {
    launch_overlapped(prep_kernel<TI, TA, TC>, grid, dim3(kWarps * 32), smem, stream, a);
  });););
  return check_launch("qk_norm_rope_cache");
}
