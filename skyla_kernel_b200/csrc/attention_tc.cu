// Causal prompt attention over the paged bfloat16 cache on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in TMEM, operands by TMA), for heads of 128 elements.
// It computes what attention_mma.cu's prefill kernel computes (skyla-ref/src/model.rs:149-165:
// softmax(q.k * scale) over the visible positions, times v), with the softmax in 32-bit and
// online across pages of 64 keys (skyla-shaders/shaders/attention.comp:81-99).
//
// A block takes 64 consecutive new tokens of one sequence and TWO query heads that share a
// key/value head: 128 rows.  Per page of the sequence:
//   S[128 x 64]  = Q K^T      8 MMAs (M 128, N 64, K 16): Q from shared memory (loaded once), the
//                             page's K as it lies in the cache (keys are rows: K-major)
//   softmax                   a thread owns a row: it reads its 64 scores from TMEM, masks, keeps the
//                             running reference and sum, and writes P (bfloat16) back over them
//   O[128 x 128] += P V       4 MMAs (M 128, N 128, K 16): P straight from TMEM; the page's V as it lies
//                             in the cache is an "MN-major" operand (keys are the K dimension, a
//                             head's elements contiguous)
// Warp 0 loads (TMA, a ring of four tiles: K and V pages have slots and barriers of their own, so a
// K page's slot is free as soon as Q K^T has read it), warp 1 issues the MMAs, warps 2-5 are the 128
// rows.  S/P is double-buffered, so Q K^T of the next page and P V of the page before run while the
// rows work on this one; O stays in TMEM and is rescaled there only when a score exceeds the
// exponents' reference by more than kSlack (then the rows wait for P V of the page before).  Two
// blocks share an SM (96 KB of shared memory and 256 TMEM columns each): one's waits are the
// other's work.  Every wait is bounded.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "tc_common.cuh"
using namespace skyla;
using namespace skyla::tc;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
typedef __nv_bfloat16 bf16;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kSlack = 8.f;  // log2 units a score may exceed the exponents' reference by before O is rescaled
constexpr int kPage = 64, kHD = 128, kRows = 128;
constexpr int kSlots = 4;                         // tiles (a page of K or a page of V) in flight
constexpr int kQBytes = kRows * kHD * 2;          // [2 halves of the head][128 rows][128 bytes]
constexpr int kPageBytes = kPage * kHD * 2;       // one page of K or of V: [2 halves][64 keys][128 bytes]
constexpr int kThreads = 192;
constexpr int kSmemBytes = 1024 + kQBytes + kSlots * kPageBytes + 256;
constexpr uint32_t kTmemCols = 256;               // S/P twice (64 columns each), then O (128)

// 2^x by the hardware's approximation (x = -inf gives 0): one instruction a score
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct PrefillTcArgs {
  bf16* out; int64_t ldo; int nq, nkv;
  const int32_t* pages; int max_pages;
  const int32_t* tok_pos; const int32_t* tile_seq; const int32_t* tile_tok0; const int32_t* tile_rows;
  float scale; int window; int* error_flag;
};

__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(kThreads, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const PrefillTcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base, ring = base + kQBytes;
  const uint32_t bars = ring + kSlots * kPageBytes;
  const uint32_t q_full = bars;
  // "P written" and "P V done" have a barrier per buffer of S/P, used by even and odd pages in turn.
  // A warp of rows may be a page ahead of another, and a barrier counts arrivals, not who arrives; and
  // a parity wait cannot tell two phases ahead or behind from none.  With a barrier per buffer nobody
  // is ever more than one phase away from it: the rows get page i's scores only after P V of page i-2
  // is through (the tensor pipe runs Q K^T of page i behind it).
  auto o_done = [&](int b) { return bars + 8 + 8u * b; };
  auto p_full = [&](int b) { return bars + 24 + 8u * b; };
  auto s_full = [&](int b) { return bars + 40 + 8u * b; };
  auto t_full = [&](int s) { return bars + 56 + 8u * s; };            // tile ring: K0, V0, K1, V1, ..
  auto t_empty = [&](int s) { return bars + 56 + 8u * (kSlots + s); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // A sequence's later tiles see more keys: they go first, so that the short ones fill the end.  Blocks
  // start in the order of their numbers, so the head pairs are the fast index: all pairs of the longest
  // tile, then all of the next (with the tiles as the fast index every pair's longest tile but the first
  // few started late, and the launch ended with long blocks running alone).
  const int n_pairs = a.nq / 2;
  const int tile = (int)(gridDim.x / n_pairs) - 1 - (int)(blockIdx.x / n_pairs), h0 = 2 * (int)(blockIdx.x % n_pairs);
  const int kvh = h0 / (a.nq / a.nkv);
  const int b = a.tile_seq[tile], tok0 = a.tile_tok0[tile], rows = a.tile_rows[tile];
  const int pos_first = a.tok_pos[tok0], pos_last = pos_first + rows - 1;
  const int tile_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int page_begin = tile_lo / kPage, n_pages = pos_last / kPage + 1 - page_begin;
  const int32_t* seq_pages = a.pages + (int64_t)b * a.max_pages;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kSlots; ++s) { mbar_init(t_full(s), 1); mbar_init(t_empty(s), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full(i), 1);
      mbar_init(p_full(i), 4);  // one arrival per warp of rows
      mbar_init(o_done(i), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_slot;
  const uint32_t tmem_o = tmem + 128;
  allow_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ loader
    if (lane == 0) {
      grid_dependency_wait();  // q, and the new tokens' k and v, are the kernel before's
      mbar_expect_tx(q_full, kQBytes);
      for (int head = 0; head < 2; ++head)
        for (int half = 0; half < 2; ++half)
          tma_load_2d(q_smem + half * (kRows * 128) + head * (kPage * 128), &map_q, q_full,
                      (h0 + head) * kHD + half * 64, tok0);
      uint32_t armed = 0, armed_parity = 0;
      bool ok = true;
      for (int t = 0; t < 2 * n_pages; ++t) {  // tile t: K of page t/2 (even t) or V of it (odd t)
        const int s = t % kSlots;
        const uint32_t round = (uint32_t)(t / kSlots) & 1u;
        if (!mbar_wait(t_empty(s), round ^ 1u, &abort_flag, a.error_flag, 11)) { ok = false; break; }
        const int row = (seq_pages[page_begin + (t >> 1)] * a.nkv + kvh) * kPage;
        mbar_expect_tx(t_full(s), kPageBytes);
        armed |= 1u << s;
        armed_parity = (armed_parity & ~(1u << s)) | (round << s);
        tma_load_3d(ring + s * kPageBytes, (t & 1) ? &map_v : &map_k, t_full(s), 0, row, 0);
      }
      if (!ok) {  // gave up: let the loads in flight land before the block's memory goes away
        const long long t0 = clock64();
        while (!mbar_try_wait(q_full, 0) && clock64() - t0 < kWaitCycles / 16) {}
        for (int s = 0; s < kSlots; ++s)
          if (armed & (1u << s)) {
            const long long t1 = clock64();
            while (!mbar_try_wait(t_full(s), (armed_parity >> s) & 1) && clock64() - t1 < kWaitCycles / 16) {}
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kPage >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
      const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |  // B (the page of V) is MN-major
                                ((uint32_t)(kHD >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
      const uint64_t q_desc0 = umma_desc(q_smem), q_desc1 = umma_desc(q_smem + kRows * 128);
      bool ok = mbar_wait(q_full, 0, &abort_flag, a.error_flag, 12);
      auto issue_qk = [&](int i) -> bool {
        const int t = 2 * i, s = t % kSlots, buf = i & 1;
        if (!mbar_wait(t_full(s), (uint32_t)(t / kSlots) & 1u, &abort_flag, a.error_flag, 13)) return false;
        // S/P buffer `buf` held page i-2: its P V was issued before this, and the pipe keeps the order
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_smem = ring + s * kPageBytes;
        const uint64_t k_desc0 = umma_desc(k_smem), k_desc1 = umma_desc(k_smem + kPage * 128);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + buf * kPage, q_desc0 + 2 * k, k_desc0 + 2 * k, idesc_qk, k ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + buf * kPage, q_desc1 + 2 * k, k_desc1 + 2 * k, idesc_qk, 1u);
        umma_commit(t_empty(s));     // the page's K has been read
        umma_commit(s_full(buf));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int i = 0; i < n_pages && ok; ++i) {
        if (i + 1 < n_pages && !issue_qk(i + 1)) { ok = false; break; }  // runs while the rows work on page i
        const int t = 2 * i + 1, s = t % kSlots, buf = i & 1;
        if (!mbar_wait(t_full(s), (uint32_t)(t / kSlots) & 1u, &abort_flag, a.error_flag, 14)) { ok = false; break; }
        if (!mbar_wait(p_full(buf), (uint32_t)(i >> 1) & 1u, &abort_flag, a.error_flag, 15)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_smem = ring + s * kPageBytes;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 16 keys an instruction: 8 packed columns of P, two 8-key groups of V
          umma_bf16_tmem_a(tmem_o, tmem + buf * kPage + 8 * k, umma_desc_mn(v_smem + k * 2048, kPage * 128, 1024), idesc_pv,
                           (i | k) ? 1u : 0u);
        umma_commit(t_empty(s));     // the page's V has been read
        umma_commit(o_done(buf));
      }
    }
  } else {
    // ------------------------------------------------------------ the rows
    grid_dependency_wait();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;           // the TMEM lane this thread may read
    const int head = row >> 6, tok_r = row & 63;
    const bool valid = tok_r < rows;
    const int hi = valid ? pos_first + tok_r : -1;
    const int lo = a.window > 0 ? max(0, hi - a.window + 1) : 0;
    const int lo_max = a.window > 0 ? max(0, pos_first + 63 - a.window + 1) : 0;  // the lowest key the last row sees
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const float scale_log2 = a.scale * kLog2e;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_pages; ++i) {
      const int buf = i & 1;
      if (!mbar_wait(s_full(buf), (uint32_t)(i >> 1) & 1u, &abort_flag, a.error_flag, 16)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t sr[64];
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 16) tmem_ld16(tmem + t_lane + buf * kPage + c0, sr + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int key0 = (page_begin + i) * kPage;
      const bool whole = key0 + 63 <= pos_first && key0 >= lo_max;  // every row sees the whole page (same for the block)
      // The maximum is taken over the raw scores (the scale is positive) on four chains, and the scale
      // goes into the exponent's one multiply-add: max, fma, ex2, add per score.
      if (!whole) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          if (!(key >= lo && key <= hi)) sr[c] = 0xff800000u;  // -inf: exp2 gives 0
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(sr[c]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(sr[c + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(sr[c + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(sr[c + 3]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      // `m` is the reference of the exponents, not the running maximum: it only moves when a score
      // exceeds it by more than kSlack (then O and l are rescaled); in between, exponents reach up
      // to 2^kSlack, which bfloat16 and the 32-bit sums hold just as well, and O is left alone.
      const bool moves = mx > m + kSlack;  // also the first visible score (m is -inf)
      const float mn = moves ? mx : m;
      const float ref = mn == -INFINITY ? 0.f : mn;
      const float alpha = moves ? fast_exp2(m - ref) : 1.f;
      m = mn;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c]), scale_log2, -ref));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), scale_log2, -ref));
        const float p2 = fast_exp2(fmaf(__uint_as_float(sr[c + 2]), scale_log2, -ref));
        const float p3 = fast_exp2(fmaf(__uint_as_float(sr[c + 3]), scale_log2, -ref));
        sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
        __nv_bfloat162 v01 = __floats2bfloat162_rn(p0, p1), v23 = __floats2bfloat162_rn(p2, p3);
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&v01);
        pk[(c >> 1) + 1] = *reinterpret_cast<uint32_t*>(&v23);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l = l * alpha + sum;
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // the reference moved: rescale this warp's rows of O, once P V of the page before is through
        if (!mbar_wait(o_done(buf ^ 1), (uint32_t)((i - 1) >> 1) & 1u, &abort_flag, a.error_flag, 19)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c0 = 0; c0 < kHD; c0 += 16) {
          uint32_t o[16];
          tmem_ld16(tmem_o + t_lane + c0, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st16(tmem_o + t_lane + c0, o);
        }
      }
      // this row of P over its scores: 64 bfloat16 = 32 columns (keys 2c and 2c+1 in column c)
      tmem_st16(tmem + t_lane + buf * kPage, pk);
      tmem_st16(tmem + t_lane + buf * kPage + 16, pk + 16);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(buf));
    }
    if (ok && mbar_wait(o_done((n_pages - 1) & 1), (uint32_t)((n_pages - 1) >> 1) & 1u, &abort_flag, a.error_flag, 18)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = a.out + (int64_t)(tok0 + tok_r) * a.ldo + (int64_t)(h0 + head) * kHD;
#pragma unroll 1
      for (int c0 = 0; c0 < kHD; c0 += 16) {
        uint32_t o[16];
        tmem_ld16(tmem_o + t_lane + c0, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (valid) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv, __uint_as_float(o[2 * j + 1]) * inv);
            w[j] = *reinterpret_cast<uint32_t*>(&v);
          }
          *reinterpret_cast<uint4*>(dst + c0) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (lane == 0 && !abort_flag) {  // every MMA must be through before the columns are freed
      const long long t0 = clock64();
      while (!mbar_try_wait(o_done((n_pages - 1) & 1), (uint32_t)((n_pages - 1) >> 1) & 1u) && clock64() - t0 < kWaitCycles / 16) {}
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}
}  // namespace

// 1 when this kernel takes the head size and grouping (heads of 128, an even number of query heads per
// key/value head, pages of 64).
extern "C" int skyla_attention_prefill_tc_supports(int hd, int nq, int nkv, int page_size) {
  return hd == kHD && page_size == kPage && nkv > 0 && nq % nkv == 0 && (nq / nkv) % 2 == 0 ? 1 : 0;
}

// Prefill on the tcgen05 path.  map_q: tensor map of q [tokens, nq*128] with boxes of 64 rows x 64 columns;
// map_k, map_v: maps of the pools viewed as [pages*nkv*64, 128] with boxes of 64 rows and both 64-column
// halves (see skyla_tensor_map_bf16 in gemm_tc.cu).  out [tokens, nq*128] bfloat16, rows 16-byte aligned.
extern "C" int skyla_attention_prefill_tc(const void* map_q, const void* map_k, const void* map_v, void* out, int64_t ldo,
                                          int n_tiles, int nq, int nkv, int hd, const int32_t* pages, int max_pages,
                                          int page_size, const int32_t* tok_pos, const int32_t* tile_seq,
                                          const int32_t* tile_tok0, const int32_t* tile_rows, float scale, int window,
                                          int* error_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return kOk;
  if (!skyla_attention_prefill_tc_supports(hd, nq, nkv, page_size))
    return fail(kBadArgument, "attention_prefill_tc: heads of 128, pages of 64 and an even group of query heads only");
  if (map_q == nullptr || map_k == nullptr || map_v == nullptr || out == nullptr || ldo % 8 || ((uintptr_t)out) % 16)
    return fail(kBadArgument, "attention_prefill_tc: missing tensor maps or an output that is not 16-byte aligned");
  if ((int64_t)n_tiles * (nq / 2) >= (1LL << 31)) return fail(kBadArgument, "attention_prefill_tc: too many tiles");
  alignas(64) CUtensorMap mq, mk, mv;
  memcpy(&mq, map_q, sizeof(mq));
  memcpy(&mk, map_k, sizeof(mk));
  memcpy(&mv, map_v, sizeof(mv));
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return fail(kLaunchFailed, "attention_prefill_tc: shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  PrefillTcArgs a{(bf16*)out, ldo, nq, nkv, pages, max_pages, tok_pos, tile_seq, tile_tok0, tile_rows, scale, window, error_flag};
  launch_overlapped(attn_prefill_tc_kernel, dim3(n_tiles * (nq / 2)), dim3(kThreads), (size_t)kSmemBytes, stream, mq, mk, mv, a);
  return check_launch("attention_prefill_tc");
}
