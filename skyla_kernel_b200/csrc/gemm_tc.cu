// Tensor-core matrix product for sm_100a: y = x W^T with bfloat16 operands and
// 32-bit accumulation, x[M,K] (tokens) and W[N,K] (rows are outputs) both
// K-major.  It takes the place of the reference's matvec/matmul shaders
// (skyla-shaders/shaders/matmul.comp:113-185, matvec_q8_0.comp:33-76), including
// their fused epilogues: residual add (ACCUM, skyla-engine/src/graph.rs:110-112)
// and silu(gate)*up (skyla-shaders/shaders/silu_mul.comp:15-24).
//
// The weight is the 128-row operand of tcgen05.mma and the tokens are the N
// operand (16..256 wide), so the same kernel serves a 2,048-token prompt and a
// batch of a few decoded tokens that only has to stream the weight once:
//   warp 0    one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//             of a [128 x 64] weight tile and a [BN x 64] token tile per stage;
//   warp 1    allocates TMEM; one lane issues tcgen05.mma (M=128, N=BN, K=16),
//             accumulating in TMEM, and commits each stage back to the loader;
//   warps 2-5 read the accumulator with tcgen05.ld (lane = output feature,
//             column = token) and write the epilogue.
// grid = (feature tiles, token tiles, K splits).  Every mbarrier wait is bounded:
// on a timeout the CTA records an error code, drains what it started, frees its
// TMEM and returns.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {

enum Mode : int {
  kStoreBf16 = 0,   // y[tok, f] = acc                     (bfloat16)
  kStoreF32 = 1,    // y[tok, f] = acc                     (float)
  kAccumF32 = 2,    // y[tok, f] += acc                    (float: the residual sum)
  kGluBf16 = 3,     // y[tok, f] = silu(gate) * up         (bfloat16; W rows in groups of 128 gate, 128 up)
  kPartialF32 = 4,  // y[split, tok, f] = acc of this K split (float scratch)
  kAccumCluster = 5,  // y[tok, f] += sum over the K splits, which form one thread-block cluster: the
                      // splits' tiles meet in rank 0 through distributed shared memory, in rank order
  kAccumLast = 6,     // y[tok, f] += sum over the K splits: every split leaves its tile in scratch and
                      // counts itself in; the one that counts last adds them up in split order
};

constexpr int BM = 128;  // weight rows per tile
constexpr int BK = 64;   // K elements per stage: one 128-byte swizzle row
constexpr int kThreads = 192;
// Pipeline memory per block: one block per SM with as deep a ring as fits.  (Half of it, so
// that the next product's blocks can move in early, measured slower: 4.4 against 4.0 ms for a
// decode step of the 8B shape at batch 8.)
constexpr int kSmemBudget = 200 * 1024;
constexpr long long kWaitCycles = 2000000000LL;  // about a second

template <int BN, int MODE>
struct Cfg {
  static constexpr int kATiles = MODE == kGluBf16 ? 2 : 1;
  static constexpr int kABytes = kATiles * BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // cluster epilogue: a landing zone of BN x 128 floats that the K splits push their tiles into
  static constexpr int kLandingBytes = MODE == kAccumCluster ? (BN + 8) * BM * 4 : 0;  // ranks x ceil(BN/ranks) columns
  static constexpr int kStagesRaw = (kSmemBudget - kLandingBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kTmemColsRaw = kATiles * BN;
  static constexpr int kTmemCols = kTmemColsRaw < 32 ? 32 : kTmemColsRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/ + kLandingBytes;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
  static_assert(kStages >= 2, "pipeline depth");
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false on a timeout or when another role of this CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* error_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      if (error_flag != nullptr) atomicCAS(error_flag, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle:
// 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version of sm_100
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}

// "Make the residual stream whole": x[r] += sum_s part[s][r], rows 0..M-1, width H.
// A side job for warps that would otherwise idle; it runs after the dependency wait.
struct FoldJob {
  float* x; int64_t ldx; const float* part; int n_splits; int64_t split_stride, ldp; int M, H;
};

// The token operand made inside the kernel instead of loaded: rmsnorm(x + sum_s part[s]).
// RMSNorm is x * r * w with one scalar r per row, and a row's scalar commutes with
// the product, so the operand is bf16((x + sum part) * w) and r = 1/sqrt(mean(.^2) + eps)
// is applied to the accumulator (or, for K-split partial output, handed on as the
// split's share of the row's sum of squares in ssq_out[split][row]).
struct NormSource {
  const float* x; int64_t ldx; const float* part; int n_splits; int64_t split_stride, ldp;
  const float* w; float eps; float* ssq_out;
};

struct GemmArgs {
  void* y;
  int64_t ldy;            // elements between token rows of y
  int64_t split_stride;   // elements between K splits of y (partial mode)
  int M, N, K;            // tokens, output features (after gating), reduction length
  int k_blocks_per_split;
  int* error_flag;
  FoldJob fold;           // fold.x == nullptr: none
  NormSource norm;        // used by the NORMB kernels only
  float* scratch;         // kAccumLast: [splits][M][N] tiles of the K splits
  int* counters;          // kAccumLast: one per output tile, zero between launches
};

template <int BN, int MODE, bool NORMB>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const GemmArgs a) {
  using C = Cfg<BN, MODE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;
  __shared__ int last_split;                 // kAccumLast: this block counted in last
  __shared__ float row_ssq[NORMB ? BN : 1];  // sum of squares of each token row over this block's K range
  __shared__ float warp_ssq[NORMB ? 4 : 1][NORMB ? BN : 1];

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + C::kStages * C::kStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  const uint32_t tmem_full_bar = bars + 8u * (2 * C::kStages);
  const uint32_t landing = bars + 256u;  // [source rank][owned token][128 features] floats (cluster epilogue)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f_tile = blockIdx.x, t_tile = blockIdx.y, split = blockIdx.z;
  const int total_kb = (a.K + BK - 1) / BK;
  const int kb0 = split * a.k_blocks_per_split;
  const int n_kb = min(a.k_blocks_per_split, total_kb - kb0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), NORMB ? 2 : 1);  // the loader, and with NORMB the warp that makes the stage's token tile
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  allow_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t armed = 0, armed_parity = 0;  // per stage: a load is in flight, and its phase
      // Weights are written by no kernel: the first stages' weight tiles are requested
      // before this grid waits for its predecessor, the token tiles after.
      const int n_pre = min(n_kb, C::kStages);
      constexpr uint32_t kTxBytes = NORMB ? C::kABytes : C::kStageBytes;
      for (int kb = 0; kb < n_pre; ++kb) {
        mbar_expect_tx(full_bar(kb), kTxBytes);
        tma_load_2d(base + kb * C::kStageBytes, &map_w, full_bar(kb), (kb0 + kb) * BK, f_tile * BM * C::kATiles);
        armed |= 1u << kb;
      }
      if (!NORMB) {
        grid_dependency_wait();
        for (int kb = 0; kb < n_pre; ++kb)
          tma_load_2d(base + kb * C::kStageBytes + C::kABytes, &map_x, full_bar(kb), (kb0 + kb) * BK, t_tile * BN);
      }
      int kb = n_pre;
      for (; kb < n_kb; ++kb) {
        const int s = kb % C::kStages;
        const uint32_t phase = (kb / C::kStages) & 1;
        if (!mbar_wait(empty_bar(s), phase ^ 1, &abort_flag, a.error_flag, 1)) break;
        const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kABytes;
        mbar_expect_tx(full_bar(s), kTxBytes);
        tma_load_2d(sa, &map_w, full_bar(s), (kb0 + kb) * BK, f_tile * BM * C::kATiles);
        if (!NORMB) tma_load_2d(sb, &map_x, full_bar(s), (kb0 + kb) * BK, t_tile * BN);
        armed |= 1u << s;
        armed_parity = (armed_parity & ~(1u << s)) | (phase << s);
      }
      if (kb < n_kb) {
        // gave up: let the loads already issued land before the CTA's memory goes away
        for (int s = 0; s < C::kStages; ++s)
          if (armed & (1u << s)) {
            const long long t0 = clock64();
            while (!mbar_try_wait(full_bar(s), (armed_parity >> s) & 1) && clock64() - t0 < kWaitCycles) {}
          }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=bf16, both K-major, N=BN, M=128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      for (int kb = 0; kb < n_kb; ++kb) {
        const int s = kb % C::kStages;
        const uint32_t phase = (kb / C::kStages) & 1;
        if (!mbar_wait(full_bar(s), phase, &abort_flag, a.error_flag, 2)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kABytes;
        const uint64_t da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          if (MODE == kGluBf16)  // the up rows: the next 128 rows of the tile, into the next BN columns
            umma_bf16(tmem_base + BN, umma_desc(sa + BM * BK * 2) + 2 * k, db + 2 * k, idesc, acc);
        }
        umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
      }
      umma_commit(tmem_full_bar);   // always: the teardown waits for it
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    grid_dependency_wait();                      // the epilogue reads and writes what earlier kernels touch
    const int quad = warp & 3;                   // the TMEM lanes this warp may read
    const int f = f_tile * BM + quad * 32 + lane;  // output feature of this thread
    const int et = threadIdx.x - 64;             // 0..127 among the four epilogue warps
    uint32_t my_rank = 0, n_ranks = 1;
    if (MODE == kAccumCluster) {
      asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(my_rank));
      asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n_ranks));
    }
    if (a.fold.x != nullptr && f_tile == 0 && t_tile == 0) {
      // side job while the main loop runs: this split's share of the columns of x
      const int per = (a.fold.H + (int)gridDim.z - 1) / (int)gridDim.z;
      const int c0 = split * per, c1 = min(a.fold.H, c0 + per);
      for (int r = 0; r < a.fold.M; ++r)
        for (int c = c0 + et; c < c1; c += 128) {
          float v = a.fold.x[(int64_t)r * a.fold.ldx + c];
          for (int sp = 0; sp < a.fold.n_splits; ++sp)
            v += a.fold.part[(int64_t)sp * a.fold.split_stride + (int64_t)r * a.fold.ldp + c];
          a.fold.x[(int64_t)r * a.fold.ldx + c] = v;
        }
    }
    if (NORMB) {
      // Make the token tiles (BN = 16): each of the four warps takes every fourth stage, so four
      // stages' loads are in flight at once.  Lane l handles chunk l%8 (8 elements) of rows
      // l/8, l/8+4, l/8+8, l/8+12.
      static_assert(!NORMB || BN == 16, "the in-kernel norm is written for token tiles of 16");
      // No more producing warps than stages: a warp that has finished block kb then knows that
      // block kb - stages has been consumed, so the stage of its next block, kb + producers, is
      // at most one phase behind -- the most a parity wait can tell apart.
      constexpr int kProducers = C::kStages < 4 ? C::kStages : 4;
      const int ew = warp - 2, chunk = lane & 7;
      float ssq[4] = {0.f, 0.f, 0.f, 0.f};
      for (int kb = ew; kb < n_kb && ew < kProducers; kb += kProducers) {
        const int s = kb % C::kStages;
        const uint32_t phase = (kb / C::kStages) & 1;
        if (!mbar_wait(empty_bar(s), phase ^ 1, &abort_flag, a.error_flag, 4)) break;
        const int k = (kb0 + kb) * BK + chunk * 8;
        uint8_t* sb = smem_raw + (base - smem_u32(smem_raw)) + s * C::kStageBytes + C::kABytes;
        float4 v0[4], v1[4];
        bool live[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // all loads first
          const int tok = t_tile * BN + (lane >> 3) + 4 * i;
          live[i] = tok < a.M && k < a.K;
          v0[i] = v1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (live[i]) {
            const float* xp = a.norm.x + (int64_t)tok * a.norm.ldx + k;
            v0[i] = *reinterpret_cast<const float4*>(xp);
            v1[i] = *reinterpret_cast<const float4*>(xp + 4);
          }
        }
        float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
        if (k < a.K) {
          w0 = *reinterpret_cast<const float4*>(a.norm.w + k);
          w1 = *reinterpret_cast<const float4*>(a.norm.w + k + 4);
        }
        for (int sp = 0; sp < a.norm.n_splits; ++sp)  // pending partial sums, if any (ascending order)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (live[i]) {
              const int tok = t_tile * BN + (lane >> 3) + 4 * i;
              const float* pp = a.norm.part + (int64_t)sp * a.norm.split_stride + (int64_t)tok * a.norm.ldp + k;
              const float4 p0 = *reinterpret_cast<const float4*>(pp), p1 = *reinterpret_cast<const float4*>(pp + 4);
              v0[i].x += p0.x; v0[i].y += p0.y; v0[i].z += p0.z; v0[i].w += p0.w;
              v1[i].x += p1.x; v1[i].y += p1.y; v1[i].z += p1.z; v1[i].w += p1.w;
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = (lane >> 3) + 4 * i;
          ssq[i] += v0[i].x * v0[i].x + v0[i].y * v0[i].y + v0[i].z * v0[i].z + v0[i].w * v0[i].w +
                    v1[i].x * v1[i].x + v1[i].y * v1[i].y + v1[i].z * v1[i].z + v1[i].w * v1[i].w;
          __nv_bfloat162 b0 = __floats2bfloat162_rn(v0[i].x * w0.x, v0[i].y * w0.y);
          __nv_bfloat162 b1 = __floats2bfloat162_rn(v0[i].z * w0.z, v0[i].w * w0.w);
          __nv_bfloat162 b2 = __floats2bfloat162_rn(v1[i].x * w1.x, v1[i].y * w1.y);
          __nv_bfloat162 b3 = __floats2bfloat162_rn(v1[i].z * w1.z, v1[i].w * w1.w);
          // the layout TMA's 128-byte swizzle would have written: chunk ^ (row mod 8)
          *reinterpret_cast<uint4*>(sb + r * 128 + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1),
                         *reinterpret_cast<uint32_t*>(&b2), *reinterpret_cast<uint32_t*>(&b3));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
      }
      // whole rows: a row's 8 chunks sit in consecutive lanes; then the four warps, in order
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = ssq[i];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (chunk == 0) warp_ssq[ew][(lane >> 3) + 4 * i] = v;
      }
      asm volatile("barrier.sync 1, 128;" ::: "memory");  // the four epilogue warps
      if (et < BN) row_ssq[et] = warp_ssq[0][et] + warp_ssq[1][et] + warp_ssq[2][et] + warp_ssq[3][et];
      asm volatile("barrier.sync 1, 128;" ::: "memory");
      if (a.norm.ssq_out != nullptr && f_tile == 0 && et < BN && t_tile * BN + et < a.M)
        a.norm.ssq_out[(int64_t)split * a.M + t_tile * BN + et] = row_ssq[et];
    }
    if (n_kb > 0 && mbar_wait(tmem_full_bar, 0, &abort_flag, a.error_flag, 3)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
      const int tok0 = t_tile * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (tok0 + c0 >= a.M) break;  // uniform for the warp
        uint32_t r[16], u[16];
        tmem_ld16(taddr + c0, r);
        if (MODE == kGluBf16) tmem_ld16(taddr + BN + c0, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (f < a.N) {
          float old[16];
          if (MODE == kAccumF32) {  // all loads first: they do not wait for one another
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = tok0 + c0 + j;
              old[j] = tok < a.M ? ((const float*)a.y)[(int64_t)tok * a.ldy + f] : 0.f;
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok >= a.M) break;
            float v = __uint_as_float(r[j]);
            float inv = 1.f;
            if (NORMB && MODE != kPartialF32) {  // one block sees the whole row: apply the norm's scalar here
              inv = 1.0f / sqrtf(row_ssq[c0 + j] / (float)a.K + a.norm.eps);
              v *= inv;
            }
            if (MODE == kStoreBf16) {
              ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + f] = __float2bfloat16_rn(v);
            } else if (MODE == kStoreF32) {
              ((float*)a.y)[(int64_t)tok * a.ldy + f] = v;
            } else if (MODE == kAccumF32) {
              ((float*)a.y)[(int64_t)tok * a.ldy + f] = old[j] + v;
            } else if (MODE == kAccumCluster) {
              // token column c0+j belongs to rank (c0+j) % n_ranks: push this split's value into
              // that block's landing zone, slot [my rank][(c0+j) / n_ranks][feature]
              const uint32_t col = (uint32_t)(c0 + j);
              const uint32_t local = landing + 4u * ((my_rank * ((BN + n_ranks - 1) / n_ranks) + col / n_ranks) * BM +
                                                     quad * 32 + lane);
              uint32_t remote;
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(col % n_ranks));
              asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
            } else if (MODE == kGluBf16) {
              const float up = __uint_as_float(u[j]) * inv;
              ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + f] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * up);
            } else if (MODE == kAccumLast) {
              a.scratch[((int64_t)split * a.M + tok) * a.N + f] = v;
            } else {
              ((float*)a.y)[(int64_t)split * a.split_stride + (int64_t)tok * a.ldy + f] = v;
            }
          }
        }
      }
    }
    if (MODE == kAccumLast) {
      // count this split in; whoever counts last has every split's tile in reach and adds them up
      __threadfence();
      asm volatile("barrier.sync 1, 128;" ::: "memory");
      if (et == 0) {
        const int tile_id = f_tile * (int)gridDim.y + t_tile;
        const int before = atomicAdd(&a.counters[tile_id], 1);
        last_split = before == (int)gridDim.z - 1;
        if (last_split) a.counters[tile_id] = 0;  // ready for the next launch
      }
      asm volatile("barrier.sync 1, 128;" ::: "memory");
      if (last_split && f < a.N && !abort_flag) {
        __threadfence();
        const int tok0 = t_tile * BN;
        const int n_tok = min(BN, a.M - tok0);
        for (int j0 = 0; j0 < n_tok; j0 += 8) {
          float sum[8], old[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            sum[j] = 0.f;
            old[j] = j0 + j < n_tok ? ((const float*)a.y)[(int64_t)(tok0 + j0 + j) * a.ldy + f] : 0.f;
          }
          for (int sp = 0; sp < (int)gridDim.z; ++sp)
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (j0 + j < n_tok) sum[j] += __ldcg(&a.scratch[((int64_t)sp * a.M + tok0 + j0 + j) * a.N + f]);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j0 + j < n_tok) ((float*)a.y)[(int64_t)(tok0 + j0 + j) * a.ldy + f] = old[j] + sum[j];
        }
      }
    }
  }
  if (MODE == kAccumCluster) {
    // All splits have pushed their tiles; each block now owns the token columns c with
    // c % n_ranks == its rank, adds the splits' values in rank order and updates y.
    uint32_t rank, n_ranks;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n_ranks));
    const int f = f_tile * BM + (warp & 3) * 32 + lane;
    const int tok0 = t_tile * BN;
    const int n_tok = min(BN, a.M - tok0);
    constexpr int kMaxOwned = BN;  // with one rank a block owns every column
    const int per_rank = (BN + (int)n_ranks - 1) / (int)n_ranks;
    float old[kMaxOwned > 16 ? 16 : kMaxOwned];
    const bool worker = warp >= 2 && f < a.N;
    if (worker) {  // the old values do not depend on the peers: fetch them while waiting
#pragma unroll
      for (int i = 0; i < (kMaxOwned > 16 ? 16 : kMaxOwned); ++i) {
        const int col = i * (int)n_ranks + (int)rank;
        old[i] = (i < per_rank && col < n_tok) ? ((const float*)a.y)[(int64_t)(tok0 + col) * a.ldy + f] : 0.f;
      }
    }
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
    if (worker && !abort_flag) {
      const float* land = reinterpret_cast<const float*>(smem_raw + (landing - smem_u32(smem_raw)));
#pragma unroll
      for (int i = 0; i < (kMaxOwned > 16 ? 16 : kMaxOwned); ++i) {
        const int col = i * (int)n_ranks + (int)rank;
        if (i >= per_rank || col >= n_tok) continue;
        float sum = 0.f;
        for (uint32_t src = 0; src < n_ranks; ++src) sum += land[((int)src * per_rank + i) * BM + (warp & 3) * 32 + lane];
        ((float*)a.y)[(int64_t)(tok0 + col) * a.ldy + f] = old[i] + sum;
      }
      for (int i = 16; i < per_rank; ++i) {  // a block that owns more than 16 columns (few splits, wide tile)
        const int col = i * (int)n_ranks + (int)rank;
        if (col >= n_tok) break;
        float sum = 0.f;
        for (uint32_t src = 0; src < n_ranks; ++src) sum += land[((int)src * per_rank + i) * BM + (warp & 3) * 32 + lane];
        float* p = (float*)a.y + (int64_t)(tok0 + col) * a.ldy + f;
        *p += sum;
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (lane == 0 && n_kb > 0) {  // the accumulator must be idle before its columns are freed
      const long long t0 = clock64();
      while (!mbar_try_wait(tmem_full_bar, 0) && clock64() - t0 < kWaitCycles) {}
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ persistent, for prompts
// Many tokens: the kernel is bound by the tensor cores, so the epilogue must not cost
// tensor time.  One block per SM walks the output tiles (tile = blockIdx.x, += gridDim.x;
// tiles of one weight tile are neighbours, so concurrent blocks share it through L2).  TMEM
// holds two accumulators: while the four epilogue warps drain tile i, the MMA warp already
// works on tile i+1.  The TMA ring runs on across tile boundaries.
template <int BN, int MODE>
struct PCfg {
  static constexpr int kATiles = MODE == kGluBf16 ? 2 : 1;
  static constexpr int kABytes = kATiles * BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kSmemBudget / kStageBytes;
  static constexpr int kAccCols = kATiles * BN;
  static constexpr int kTmemCols = 2 * kAccCols;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols >= 32, "TMEM columns");
  static_assert(kStages >= 2 && kStages <= 12, "pipeline depth");
};

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          const GemmArgs a, int n_f_tiles, int n_t_tiles) {
  using C = PCfg<BN, MODE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + C::kStages * C::kStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * C::kStages + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * C::kStages + 2 + b); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (a.K + BK - 1) / BK;
  const int n_tiles = n_f_tiles * n_t_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  allow_dependents();

  if (warp == 0) {
    if (lane == 0) {
      grid_dependency_wait();
      uint32_t armed = 0, armed_parity = 0;
      int kbg = 0;  // K blocks loaded so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int f_tile = tile / n_t_tiles, t_tile = tile % n_t_tiles;
        for (int kb = 0; kb < total_kb; ++kb, ++kbg) {
          const int s = kbg % C::kStages;
          const uint32_t phase = (kbg / C::kStages) & 1;
          if (!mbar_wait(empty_bar(s), phase ^ 1, &abort_flag, a.error_flag, 1)) { ok = false; break; }
          const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kABytes;
          mbar_expect_tx(full_bar(s), C::kStageBytes);
          tma_load_2d(sa, &map_w, full_bar(s), kb * BK, f_tile * BM * C::kATiles);
          tma_load_2d(sb, &map_x, full_bar(s), kb * BK, t_tile * BN);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (phase << s);
        }
      }
      if (!ok)  // gave up: let the loads already issued land before the block's memory goes away
        for (int s = 0; s < C::kStages; ++s)
          if (armed & (1u << s)) {
            const long long t0 = clock64();
            while (!mbar_try_wait(full_bar(s), (armed_parity >> s) & 1) && clock64() - t0 < kWaitCycles) {}
          }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      int kbg = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!mbar_wait(acc_empty_bar(buf), ((it >> 1) & 1) ^ 1, &abort_flag, a.error_flag, 5)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_base + buf * C::kAccCols;
        for (int kb = 0; kb < total_kb; ++kb, ++kbg) {
          const int s = kbg % C::kStages;
          const uint32_t phase = (kbg / C::kStages) & 1;
          if (!mbar_wait(full_bar(s), phase, &abort_flag, a.error_flag, 2)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kABytes;
          const uint64_t da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            umma_bf16(d, da + 2 * k, db + 2 * k, idesc, acc);
            if (MODE == kGluBf16) umma_bf16(d + BN, umma_desc(sa + BM * BK * 2) + 2 * k, db + 2 * k, idesc, acc);
          }
          umma_commit(empty_bar(s));
        }
        umma_commit(acc_full_bar(buf));
      }
    }
  } else {
    grid_dependency_wait();
    const int quad = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      const int f_tile = tile / n_t_tiles, t_tile = tile % n_t_tiles, buf = it & 1;
      if (!mbar_wait(acc_full_bar(buf), (it >> 1) & 1, &abort_flag, a.error_flag, 3)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int f = f_tile * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + buf * C::kAccCols + ((uint32_t)(quad * 32) << 16);
      const int tok0 = t_tile * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (tok0 + c0 >= a.M) break;
        uint32_t r[16], u[16];
        tmem_ld16(taddr + c0, r);
        if (MODE == kGluBf16) tmem_ld16(taddr + BN + c0, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (f < a.N) {
          float old[16];
          if (MODE == kAccumF32) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = tok0 + c0 + j;
              old[j] = tok < a.M ? ((const float*)a.y)[(int64_t)tok * a.ldy + f] : 0.f;
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok >= a.M) break;
            const float v = __uint_as_float(r[j]);
            if (MODE == kStoreBf16) {
              ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + f] = __float2bfloat16_rn(v);
            } else if (MODE == kStoreF32) {
              ((float*)a.y)[(int64_t)tok * a.ldy + f] = v;
            } else if (MODE == kAccumF32) {
              ((float*)a.y)[(int64_t)tok * a.ldy + f] = old[j] + v;
            } else {
              const float up = __uint_as_float(u[j]);
              ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + f] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * up);
            }
          }
        }
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(buf));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (lane == 0) {  // every accumulator must be idle before its columns are freed
      const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
      for (int b = 0; b < 2; ++b) {
        const int uses = (my_tiles + 1 - b) / 2;  // tiles that used accumulator b
        if (uses > 0) {
          const long long t0 = clock64();
          while (!mbar_try_wait(acc_full_bar(b), (uses - 1) & 1) && clock64() - t0 < kWaitCycles) {}
        }
      }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

template <int BN, int MODE>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, int n_f, int n_t, cudaStream_t stream) {
  using C = PCfg<BN, MODE>;
  static bool configured = false;
  static int n_sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc: cannot reserve %d bytes of shared memory: %s",
                                      C::kSmemBytes, cudaGetErrorString(e));
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 148;
    configured = true;
  }
  const int tiles = n_f * n_t;
  launch_overlapped(gemm_tc_persistent_kernel<BN, MODE>, dim3(tiles < n_sms ? tiles : n_sms), dim3(kThreads),
                    C::kSmemBytes, stream, mw, mx, a, n_f, n_t);
  return check_launch("gemm_tc_persistent");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

template <int BN, int MODE, bool NORMB = false>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, dim3 grid, cudaStream_t stream) {
  using C = Cfg<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE, NORMB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc: cannot reserve %d bytes of shared memory: %s",
                                      C::kSmemBytes, cudaGetErrorString(e));
    configured = true;
  }
  if (MODE == kAccumCluster)
    launch_overlapped_cluster(gemm_tc_kernel<BN, MODE, NORMB>, grid, dim3(kThreads), C::kSmemBytes, stream, grid.z, mw, mx, a);
  else
    launch_overlapped(gemm_tc_kernel<BN, MODE, NORMB>, grid, dim3(kThreads), C::kSmemBytes, stream, mw, mx, a);
  return check_launch("gemm_tc");
}

template <int MODE>
int launch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, dim3 grid, cudaStream_t s) {
  switch (bn) {
    case 16: return launch<16, MODE>(mw, mx, a, grid, s);
    case 32: return launch<32, MODE>(mw, mx, a, grid, s);
    case 64: return launch<64, MODE>(mw, mx, a, grid, s);
    case 128: return launch<128, MODE>(mw, mx, a, grid, s);
    case 256: return launch<256, MODE>(mw, mx, a, grid, s);
  }
  return fail(kBadArgument, "gemm_tc: no kernel for a token tile of %d", bn);
}
}  // namespace

// Fills a 128-byte tensor map for a row-major bfloat16 matrix [rows, cols] with
// `ld` elements between rows; boxes are [box_rows x 64 columns], 128-byte swizzle.
extern "C" int skyla_tensor_map_bf16(void* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                                     uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(kLaunchFailed, "tensor map: the driver does not offer cuTensorMapEncodeTiled");
  if (((uintptr_t)ptr) % 16 || (ld * 2) % 16) return fail(kBadArgument, "tensor map: base or row stride is not a multiple of 16 bytes");
  if (box_rows == 0 || box_rows > 256) return fail(kBadArgument, "tensor map: box of %u rows", box_rows);
  alignas(64) CUtensorMap m;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kLaunchFailed, "tensor map: cuTensorMapEncodeTiled failed with %d", (int)r);
  memcpy(out, &m, sizeof(m));
  return kOk;
}

extern "C" int skyla_gemm_tc_stages(int bn, int mode) {
  if (mode == kGluBf16) return bn == 16 ? Cfg<16, kGluBf16>::kStages : bn == 32 ? Cfg<32, kGluBf16>::kStages
                             : bn == 64 ? Cfg<64, kGluBf16>::kStages : bn == 128 ? Cfg<128, kGluBf16>::kStages
                             : Cfg<256, kGluBf16>::kStages;
  return bn == 16 ? Cfg<16, 0>::kStages : bn == 32 ? Cfg<32, 0>::kStages : bn == 64 ? Cfg<64, 0>::kStages
       : bn == 128 ? Cfg<128, 0>::kStages : Cfg<256, 0>::kStages;
}

// map_w: weight [rows, K] with boxes of 128 rows (256 in gated mode); map_x: tokens [M, K] with boxes of bn rows.
// fold_x (may be null): a residual stream [M, fold_h] to which fold_part [fold_splits][M][fold_h]
// is added on the side, after this kernel's dependency wait.
extern "C" int skyla_gemm_tc(const void* map_w, const void* map_x, void* y, int64_t ldy, int64_t split_stride,
                             int M, int N, int K, int bn, int mode, int splits, int* error_flag,
                             float* fold_x, int64_t fold_ldx, const float* fold_part, int fold_splits,
                             int64_t fold_split_stride, int64_t fold_ldp, int fold_h, float* scratch, int* counters,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || K % 8) return fail(kBadArgument, "gemm_tc: K=%d must be a positive multiple of 8", K);
  if (mode < 0 || mode > 6) return fail(kBadArgument, "gemm_tc: unknown epilogue %d", mode);
  if (splits < 1 || (splits > 1 && mode != kPartialF32 && mode != kAccumCluster && mode != kAccumLast))
    return fail(kBadArgument, "gemm_tc: %d K splits need the partial, the cluster or the last-arriver epilogue", splits);
  if (mode == kAccumLast && (scratch == nullptr || counters == nullptr || bn > 64))
    return fail(kBadArgument, "gemm_tc: the last-arriver epilogue needs scratch, counters and at most 64 tokens per tile");
  if (mode == kAccumCluster && (splits > 8 || bn > 64))
    return fail(kBadArgument, "gemm_tc: the cluster epilogue takes at most 8 K splits and 64 tokens per tile");
  const int total_kb = (K + BK - 1) / BK;
  const int per = (total_kb + splits - 1) / splits;
  if ((splits - 1) * per >= total_kb) return fail(kBadArgument, "gemm_tc: %d K splits leave one empty (K=%d)", splits, K);
  alignas(64) CUtensorMap mw, mx;
  memcpy(&mw, map_w, sizeof(mw));
  memcpy(&mx, map_x, sizeof(mx));
  GemmArgs a{y, ldy, split_stride, M, N, K, per, error_flag,
             FoldJob{fold_x, fold_ldx, fold_part, fold_splits, fold_split_stride, fold_ldp, M, fold_h}, NormSource{},
             scratch, counters};
  dim3 grid((N + BM - 1) / BM, (M + bn - 1) / bn, splits);
  if (grid.y > 65535 || grid.z > 65535) return fail(kBadArgument, "gemm_tc: grid too large");
  if (splits == 1 && mode <= kGluBf16 && ((mode == kGluBf16 && bn == 128) || (mode != kGluBf16 && bn == 256))) {
    // many tokens: the persistent kernel with two accumulators
    const int n_f = (int)grid.x, n_t = (int)grid.y;
    switch (mode) {
      case kStoreBf16: return launch_persistent<256, kStoreBf16>(mw, mx, a, n_f, n_t, stream);
      case kStoreF32: return launch_persistent<256, kStoreF32>(mw, mx, a, n_f, n_t, stream);
      case kAccumF32: return launch_persistent<256, kAccumF32>(mw, mx, a, n_f, n_t, stream);
      default: return launch_persistent<128, kGluBf16>(mw, mx, a, n_f, n_t, stream);
    }
  }
  switch (mode) {
    case kStoreBf16: return launch_bn<kStoreBf16>(bn, mw, mx, a, grid, stream);
    case kStoreF32: return launch_bn<kStoreF32>(bn, mw, mx, a, grid, stream);
    case kAccumF32: return launch_bn<kAccumF32>(bn, mw, mx, a, grid, stream);
    case kGluBf16: return launch_bn<kGluBf16>(bn, mw, mx, a, grid, stream);
    case kAccumCluster:
      switch (bn) {
        case 16: return launch<16, kAccumCluster>(mw, mx, a, grid, stream);
        case 32: return launch<32, kAccumCluster>(mw, mx, a, grid, stream);
        default: return launch<64, kAccumCluster>(mw, mx, a, grid, stream);
      }
    case kAccumLast:
      switch (bn) {
        case 16: return launch<16, kAccumLast>(mw, mx, a, grid, stream);
        case 32: return launch<32, kAccumLast>(mw, mx, a, grid, stream);
        default: return launch<64, kAccumLast>(mw, mx, a, grid, stream);
      }
    default: return launch_bn<kPartialF32>(bn, mw, mx, a, grid, stream);
  }
}

// The same product with the token operand made in the kernel: rmsnorm(x + sum_s part[s]) * w.
// x [M, K] float, part [n_part][M][K] float or null, w [K] float.  Modes: gated (bf16 out),
// store bf16/f32 (one K split only: the norm's scalar is applied in the epilogue), or partial
// with ssq_out [splits][M] receiving each split's share of the rows' sums of squares.
// Token tiles of 16, 32 or 64; x is not changed.
extern "C" int skyla_gemm_tc_norm(const void* map_w, const float* x, int64_t ldx, const float* part, int n_part,
                                  int64_t part_split_stride, int64_t ldp, const float* w, float eps, float* ssq_out,
                                  void* y, int64_t ldy, int64_t split_stride, int M, int N, int K, int bn, int mode,
                                  int splits, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || K % 8) return fail(kBadArgument, "gemm_tc_norm: K=%d must be a positive multiple of 8", K);
  if (bn != 16 || M > 16) return fail(kBadArgument, "gemm_tc_norm: at most 16 tokens (token tile 16), got %d", M);
  if (ldx % 4 || ldp % 4 || part_split_stride % 4 || ((uintptr_t)x) % 16 || ((uintptr_t)part) % 16 || ((uintptr_t)w) % 16)
    return fail(kBadArgument, "gemm_tc_norm: x, the partial sums and the weight must be 16-byte aligned");
  if (mode == kPartialF32 ? ssq_out == nullptr : splits != 1)
    return fail(kBadArgument, "gemm_tc_norm: K splits go with the partial epilogue and a place for the sums of squares");
  if (mode != kPartialF32 && mode != kGluBf16 && mode != kStoreBf16 && mode != kStoreF32)
    return fail(kBadArgument, "gemm_tc_norm: epilogue %d is not offered", mode);
  const int total_kb = (K + BK - 1) / BK;
  const int per = (total_kb + splits - 1) / splits;
  if (splits < 1 || (splits - 1) * per >= total_kb) return fail(kBadArgument, "gemm_tc_norm: %d K splits leave one empty (K=%d)", splits, K);
  alignas(64) CUtensorMap mw;
  memcpy(&mw, map_w, sizeof(mw));
  GemmArgs a{y, ldy, split_stride, M, N, K, per, error_flag, FoldJob{},
             NormSource{x, ldx, part, part ? n_part : 0, part_split_stride, ldp, w, eps, ssq_out}, nullptr, nullptr};
  dim3 grid((N + BM - 1) / BM, (M + bn - 1) / bn, splits);
#define SKYLA_NORM_LAUNCH(MODE_) return launch<16, MODE_, true>(mw, mw, a, grid, stream);
  switch (mode) {
    case kPartialF32: SKYLA_NORM_LAUNCH(kPartialF32)
    case kGluBf16: SKYLA_NORM_LAUNCH(kGluBf16)
    case kStoreBf16: SKYLA_NORM_LAUNCH(kStoreBf16)
    default: SKYLA_NORM_LAUNCH(kStoreF32)
  }
#undef SKYLA_NORM_LAUNCH
}
