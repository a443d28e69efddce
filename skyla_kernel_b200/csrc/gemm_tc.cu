// Tensor-core matrix product for sm_100a: y = x W^T with bfloat16 operands and
// 32-bit accumulation, x[M,K] (tokens) and W[N,K] (rows are outputs) both
// K-major.  It takes the place of the reference's matvec/matmul shaders
// (skyla-shaders/shaders/matmul.comp:113-185, matvec_q8_0.comp:33-76), including
// their fused epilogues: residual add (ACCUM, skyla-engine/src/graph.rs:110-112)
// and silu(gate)*up (skyla-shaders/shaders/silu_mul.comp:15-24).
//
// The weight is the 128-row operand of tcgen05.mma and the tokens are the N
// operand (16..256 wide): a batch of decoded tokens only has to stream the weight
// once (prompts of more than 128 tokens have a kernel of their own, gemm_prompt.cu):
//   warp 0    one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//             of a [128 x 64] weight tile and a [BN x 64] token tile per stage;
//   warp 1    allocates TMEM; one lane issues tcgen05.mma (M=128, N=BN, K=16),
//             accumulating in TMEM, and commits each stage back to the loader;
//   warps 2-5 read the accumulator with tcgen05.ld (lane = output feature,
//             column = token) and write the epilogue.
// Two kernels: gemm_tc_rows_kernel (up to 128 tokens: every SM streams its share of the
// weight; see there) and gemm_tc_kernel (grid = feature tiles x token tiles, whole K in a
// block: what the other does not take from 17 tokens on).  Every mbarrier wait is bounded: on a timeout the
// CTA records an error code, drains what it started, frees its TMEM and returns.
#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "tc_common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
using namespace skyla::tc;

enum Mode : int {
  kStoreBf16 = 0,   // y[tok, f] = acc                     (bfloat16)
  kStoreF32 = 1,    // y[tok, f] = acc                     (float)
  kAccumF32 = 2,    // y[tok, f] += acc                    (float: the residual sum)
  kGluBf16 = 3,     // y[tok, f] = silu(gate) * up         (bfloat16; W = N gate rows, then the N up rows)
};

constexpr int BM = 128;  // weight rows per tile
constexpr int BK = 64;   // K elements per stage: one 128-byte swizzle row
constexpr int kThreads = 192;
// Pipeline memory per block: one block per SM with as deep a ring as fits.  (Half of it, so
// that the next product's blocks can move in early, measured slower: 4.4 against 4.0 ms for a
// decode step of the 8B shape at batch 8.)
constexpr int kSmemBudget = 200 * 1024;

template <int BN, int MODE>
struct Cfg {
  static constexpr int kATiles = MODE == kGluBf16 ? 2 : 1;
  static constexpr int kABytes = kATiles * BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kTmemColsRaw = kATiles * BN;
  static constexpr int kTmemCols = kTmemColsRaw < 32 ? 32 : kTmemColsRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
  static_assert(kStages >= 2, "pipeline depth");
};

// "Norm ahead": the product that writes the residual stream last (y += x W^T) also leaves, for the
// RMSNorm that reads it next, the rows times that norm's weight in bfloat16 (the next product's
// token operand) and each block's share of the rows' sums of squares (ssq_part[block * M + tok]).
struct NormAhead { const float* w; __nv_bfloat16* xw; int64_t ldxw; float* ssq_part; };
// The other side: the token operand came without its norm's scalar; the rows' sums of squares lie in
// `n_parts` shares (ssq_part[p * M + tok]) and the result is multiplied by 1/sqrt(sum / width + eps).
struct ScaleIn { const float* ssq_part; int n_parts; float eps; int width; };

struct GemmArgs {
  void* y;
  int64_t ldy;            // elements between token rows of y
  int M, N, K;            // tokens, output features (after gating), reduction length
  int k_blocks_per_split; // weight-streaming kernel: the K blocks of each split of a cluster
  int* error_flag;
  NormAhead ahead;        // weight-streaming kernel, accumulate epilogue: ahead.xw == nullptr: none
  ScaleIn scale;          // weight-streaming kernel: scale.ssq_part == nullptr: none
};

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const GemmArgs a) {
  using C = Cfg<BN, MODE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + C::kStages * C::kStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  const uint32_t tmem_full_bar = bars + 8u * (2 * C::kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f_tile = blockIdx.x, t_tile = blockIdx.y;
  const int n_kb = (a.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
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
      constexpr uint32_t kTxBytes = C::kStageBytes;
      for (int kb = 0; kb < n_pre; ++kb) {
        mbar_expect_tx(full_bar(kb), kTxBytes);
        tma_load_2d(base + kb * C::kStageBytes, &map_w, full_bar(kb), kb * BK, f_tile * BM);
        if (MODE == kGluBf16)  // the up rows of the same outputs follow the a.N gate rows
          tma_load_2d(base + kb * C::kStageBytes + BM * BK * 2, &map_w, full_bar(kb), kb * BK, a.N + f_tile * BM);
        armed |= 1u << kb;
      }
      grid_dependency_wait();
      for (int kb = 0; kb < n_pre; ++kb)
        tma_load_2d(base + kb * C::kStageBytes + C::kABytes, &map_x, full_bar(kb), kb * BK, t_tile * BN);
      int kb = n_pre;
      for (; kb < n_kb; ++kb) {
        const int s = kb % C::kStages;
        const uint32_t phase = (kb / C::kStages) & 1;
        if (!mbar_wait(empty_bar(s), phase ^ 1, &abort_flag, a.error_flag, 1)) break;
        const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kABytes;
        mbar_expect_tx(full_bar(s), kTxBytes);
        tma_load_2d(sa, &map_w, full_bar(s), kb * BK, f_tile * BM);
        if (MODE == kGluBf16) tma_load_2d(sa + BM * BK * 2, &map_w, full_bar(s), kb * BK, a.N + f_tile * BM);
        tma_load_2d(sb, &map_x, full_bar(s), kb * BK, t_tile * BN);
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

// ------------------------------------------------------------------ few tokens: weight streaming
// A few decoded tokens: the product has to stream the weight once, at the memory's speed, and
// little else.  What that takes on this machine (all measured):
//   * a TMA tensor load occupies the SM's TMA unit for about 0.16 us whatever its size, so a
//     box has to carry tens of KB: one box brings `kkb` K blocks of a tile (a 3-D tensor map
//     whose outermost dimension is the K block), and so does the token operand's box;
//   * a tcgen05.mma of 16 tokens takes about 50 cycles whatever its shape, so an instruction
//     should cover 64 or more useful weight rows;
//   * every SM has to stream.  The tile height R (a multiple of 8, at most 128) and the number
//     of K splits are chosen by the host so that tiles x splits fills the SMs.  The MMA still
//     reads 128 rows: the rows past R hold whatever lies behind the tile in shared memory and
//     feed accumulator lanes that nobody reads.
//   * stacking: with tiles of R <= 64 rows the MMA's 128 rows take `kstack` = 128 / R K blocks
//     at once: the box of kstack K blocks lies in shared memory as kstack tiles of R rows one
//     after the other, which is a 128-row operand whose row group q holds K block q; the token
//     operand's box likewise is a (kstack x BN)-row operand.  One MMA then computes all pairs
//     (row group q, token group q'); the kstack diagonal blocks are the wanted partial products
//     (the others are never read), and the epilogue adds them up through shared memory.  So a
//     block covers its whole K with K/64/kstack x 4 instructions and needs no K split.
// K splits (without stacking) form a thread-block cluster: each pushes its tile into the landing
// zones of the blocks that own the token columns, one cluster barrier, the owners add up in rank order.
constexpr int kRowsMaxStages = 24;
// Ring + landing zone + barriers of one block: one block per SM.  (Half of it, so that the next
// product's blocks move in beside this one's and fill their rings early, measured slower for every
// product of the 8B shape: 27.2 against 22.3 us for the down product, 38.4 against 34.4 gated.)
// Asking the L2 for the next product's first boxes (cp.async.bulk.prefetch.tensor) once a block's own
// loads are issued also measured slower: a decode step of the 8B shape took 4.09, 4.18, 4.25 ms with
// 64, 128, 256 KB per block against 4.07 without.
// Running the four products between two attention kernels (O, gate/up, down, the next QKV) as the
// phases of ONE launch, a grid-wide barrier between them and the loader running on into the next
// phase's weights, was built and measured too: 93 against 80 us per layer.  A phase's end costs the
// same as a launch's (the epilogue's stores have to be visible before the barrier: 3 to 5 us, and the
// barrier 2.4), and the 192 KB ring is full again 3.7 us after a phase's last box was asked for, so the
// memory idles through most of that just the same.
constexpr int kRowsSmemBytes = 212 * 1024;
constexpr int kRowsMaxSplits = 8;

struct RowsArgs {
  int rows_per_block;   // R
  int n_stages;         // ring depth chosen by the host
  int kkb;              // K blocks per stage and per TMA box; 1: the tensor maps are 2-D
  int kstack;           // K blocks that one MMA takes at once, stacked along its rows (see below); divides kkb
  int tmem_cols;        // accumulator columns to allocate: a power of two >= 32
  int landing_bytes;    // behind the ring: the cluster's landing zone, at least the 16 KB the MMA may over-read
};


// KIND: kPlain (whole K in one block, one K block an MMA), kCluster (the K splits of a tile form a thread-block
// cluster of gridDim.z blocks) or kStacked (whole K, several K blocks stacked into one MMA).  Kernels of their
// own, so that the kernels of a decode step, which run one after the other with cold instruction caches, carry
// one epilogue each: with the cluster's epilogue inside, every launch of a step took 1.7 us longer although
// nothing of it ran.
enum RowsKind : int { kPlain = 0, kCluster = 1, kStacked = 2 };
template <int BN, int MODE, int KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmArgs a, const RowsArgs ra) {
  constexpr int kATiles = MODE == kGluBf16 ? 2 : 1;
  constexpr int kBBytes = BN * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;
  __shared__ float row_ssq[BN];  // the rows' sums of squares, handed in as shares
  __shared__ float row_inv[BN];  // 1/sqrt(mean square + eps) of the rows (not where the K splits of a cluster meet)

  const int n_stages = ra.n_stages, kkb = ra.kkb;
  const int a_tile = ra.rows_per_block * BK * 2;  // R rows of 128 bytes: a multiple of 1024
  const uint32_t stage_bytes = (uint32_t)(kkb * (kATiles * a_tile + kBBytes));
  const uint32_t bars = (smem_u32(smem_raw) + 15u) & ~15u;                       // barriers first
  const uint32_t base = (bars + 8u * (2 * kRowsMaxStages + 3) + 1023u) & ~1023u;  // then the ring
  const uint32_t landing = base + (uint32_t)n_stages * stage_bytes;               // then the landing zone
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kRowsMaxStages + s); };
  const uint32_t tmem_full_bar = bars + 8u * (2 * kRowsMaxStages);
  const uint32_t land_bar = bars + 8u * (2 * kRowsMaxStages + 1);  // the peers' tiles have landed (K splits as a cluster)
  const uint32_t sent_bar = bars + 8u * (2 * kRowsMaxStages + 2);  // the peers have taken what this block sent them

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.x * ra.rows_per_block;  // first output feature of this block
  const int split = blockIdx.z;
  constexpr bool clustered = KIND == kCluster;
  constexpr bool stacked = KIND == kStacked;
  const int total_kb = (a.K + BK - 1) / BK;
  const int kb0 = split * a.k_blocks_per_split;
  const int n_kb = max(0, min(a.k_blocks_per_split, total_kb - kb0));
  const int n_st = (n_kb + kkb - 1) / kkb;  // stages' worth of K blocks
  // every block walks its stages from a start of its own (and wraps): at any moment the blocks
  // read different lines of the token rows, which they all share, not all the same L2 line
  const int st_start = n_st > 0 ? (int)(((unsigned)blockIdx.x * 5u) % (unsigned)n_st) : 0;
  auto st_of = [&](int i) { int t = i + st_start; return t >= n_st ? t - n_st : t; };
  const uint32_t tx_bytes = (uint32_t)(kkb * kATiles * a_tile) + (uint32_t)(kkb * kBBytes);

  auto load_weights = [&](int i, int s) {
    const uint32_t sa = base + s * stage_bytes;
    const int kb = kb0 + st_of(i) * kkb;
    mbar_expect_tx(full_bar(s), tx_bytes);
    if (kkb == 1) {
      tma_load_2d(sa, &map_w, full_bar(s), kb * BK, f0);
      if (MODE == kGluBf16) tma_load_2d(sa + a_tile, &map_w, full_bar(s), kb * BK, a.N + f0);
    } else {
      tma_load_3d(sa, &map_w, full_bar(s), 0, f0, kb);
      if (MODE == kGluBf16) tma_load_3d(sa + kkb * a_tile, &map_w, full_bar(s), 0, a.N + f0, kb);
    }
  };
  const int n_pre = min(n_st, n_stages);  // stages that are filled before anything is consumed
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    mbar_init(land_bar, 1);
    if (clustered) {  // one arrival from every peer that this block sends tokens to (rank r owns ceil(M / ranks) tokens from r * that on)
      uint32_t ranks;
      asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(ranks));
      const int per = (a.M + (int)ranks - 1) / (int)ranks;
      const int owners = (a.M + per - 1) / per;  // ranks that own tokens: the first ones
      uint32_t rank;
      asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
      const int n_dst = owners - ((int)rank < owners ? 1 : 0);
      mbar_init(sent_bar, n_dst > 0 ? n_dst : 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // weights are written by no kernel: this thread, which is the loader, asks for the ring's first
    // filling at once, while the other warps allocate TMEM and the block meets (0.35 us earlier)
    for (int i = 0; i < n_pre; ++i) load_weights(i, i);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)ra.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  allow_dependents();
  // K splits as a cluster: nobody may send into a peer's landing zone before that peer's barrier exists.
  // Every thread arrives here (it costs nothing); who sends waits for the others just before sending.
  if (clustered) asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  bool met_cluster = false;  // this thread has waited for that first meeting

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      auto load_tokens = [&](int i, int s) {
        const uint32_t sb = base + s * stage_bytes + kkb * kATiles * a_tile;
        const int kb = kb0 + st_of(i) * kkb;
        if (kkb == 1) tma_load_2d(sb, &map_x, full_bar(s), kb * BK, 0);
        else tma_load_3d(sb, &map_x, full_bar(s), 0, 0, kb);
      };
      // (the ring's first filling of weights was asked for during the set-up)
      grid_dependency_wait();
      for (int i = 0; i < n_pre; ++i) load_tokens(i, i);
      int i = n_pre, s = 0;
      uint32_t phase = 1;
      for (; i < n_st; ++i) {
        if (!mbar_wait(empty_bar(s), phase ^ 1, &abort_flag, a.error_flag, 1)) break;
        load_weights(i, s);
        load_tokens(i, s);
        if (++s == n_stages) { s = 0; phase ^= 1; }
      }
      if (i < n_st) {  // gave up: let the loads in flight land before the block's memory goes away
        for (int j = max(0, i - n_stages); j < i; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar(j % n_stages), (j / n_stages) & 1) && clock64() - t0 < kWaitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const int kstack = stacked ? ra.kstack : 1;
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((kstack * BN) >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      int s = 0;
      uint32_t phase = 0, started = 0;
      for (int i = 0; i < n_st; ++i) {
        if (!mbar_wait(full_bar(s), phase, &abort_flag, a.error_flag, 2)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = base + s * stage_bytes, sb = sa + kkb * kATiles * a_tile;
        // K blocks past the end of K hold zeros (the loads fill them)
        for (int j = 0; j < kkb; j += kstack) {
          const uint64_t da = umma_desc(sa + j * a_tile), db = umma_desc(sb + j * kBBytes);
          const uint64_t du = umma_desc(sa + (kkb + j) * a_tile);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, started);
            if (MODE == kGluBf16) umma_bf16(tmem_base + BN, du + 2 * k, db + 2 * k, idesc, started);
            started = 1u;
          }
        }
        umma_commit(empty_bar(s));
        if (++s == n_stages) { s = 0; phase ^= 1; }
      }
      umma_commit(tmem_full_bar);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    grid_dependency_wait();
    const int quad = warp & 3;
    const int r_local = quad * 32 + lane;  // row of the tile that this thread's TMEM lane holds
    const int f = f0 + r_local;
    const bool mine = r_local < ra.rows_per_block && f < a.N;
    const int et = threadIdx.x - 64;
    uint32_t my_rank = 0, n_ranks = 1;
    if (clustered) {
      asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(my_rank));
      asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n_ranks));
    }
    const bool scale_in = a.scale.ssq_part != nullptr;
    if (scale_in) {  // while the main loop runs: add up the shares of the rows' sums of squares
      if (et < BN) {
        float v = 0.f;
        if (et < a.M)
          for (int p = 0; p < a.scale.n_parts; ++p) v += a.scale.ssq_part[(int64_t)p * a.M + et];
        row_ssq[et] = v;
      }
      asm volatile("barrier.sync 1, 128;" ::: "memory");
    }
    const bool scaled = scale_in;
    const float norm_width = (float)a.scale.width;
    const float norm_eps = a.scale.eps;
    // The epilogue below runs once per block with one warp per scheduler: nothing hides an
    // instruction's latency there, so whatever can be done while the main loop runs is done here
    // (the rows' scalars: 1.6 to 1.0 us for the q/k/v product's epilogue).  (Running the token loops
    // without their early exit, so that the tokens' chains interleave, measured slower for 8 tokens.)
    if (scaled) {
      if (et < BN) row_inv[et] = 1.0f / sqrtf(row_ssq[et] / norm_width + norm_eps);
      asm volatile("barrier.sync 1, 128;" ::: "memory");
    }
    const bool ahead = MODE == kAccumF32 && a.ahead.xw != nullptr;
    const int kstack = stacked ? ra.kstack : 1, R = ra.rows_per_block;
    float* red = reinterpret_cast<float*>(smem_raw + (landing - smem_u32(smem_raw)));
    float* sqbuf = red + (stacked ? kstack * BN * R : 0);  // [tok][row of the tile]: squares of the new x
    bool ssq_in_warp = false;
    // the old values of y do not depend on the product: fetch them while the main loop runs
    float old_pre[4] = {0.f, 0.f, 0.f, 0.f}, wn_pre[4] = {0.f, 0.f, 0.f, 0.f}, old16[16];
    if (MODE == kAccumF32 && stacked) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int idx = et + 128 * n;
        const int tok = idx / R, ff = f0 + idx - tok * R;
        if (idx < a.M * R && ff < a.N) {
          old_pre[n] = ((const float*)a.y)[(int64_t)tok * a.ldy + ff];
          if (ahead) wn_pre[n] = a.ahead.w[ff];
        }
      }
    }
    if (MODE == kAccumF32 && !stacked && !clustered && mine) {
#pragma unroll
      for (int j = 0; j < 16; ++j) old16[j] = j < a.M ? ((const float*)a.y)[(int64_t)j * a.ldy + f] : 0.f;
    }
    // K splits as a cluster: rank r owns the tokens [r * per, r * per + per) of the tile (see below)
    const int per = (a.M + (int)n_ranks - 1) / (int)n_ranks;
    const int my_n = max(0, min(per, a.M - (int)my_rank * per));
    constexpr uint32_t kRowBytes = BM * 4;  // a token's 128 features of the tile
    // ... and in the owner a warp takes every fourth token and a lane four neighbouring features of the tile
    const int f4 = f0 + 4 * lane;
    const bool mine4 = 4 * lane < ra.rows_per_block && f4 < a.N;  // (rows and N are multiples of 4 here)
    float4 old4[4];
    float4 w_next4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (clustered) {  // what does not depend on the product is fetched while the main loop runs
      if (et == 0 && my_n > 0) mbar_expect_tx(land_bar, (n_ranks - 1) * (uint32_t)my_n * kRowBytes);
      if (ahead && mine4) w_next4 = *reinterpret_cast<const float4*>(a.ahead.w + f4);
      if (MODE == kAccumF32) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = quad + 4 * j;
          old4[j] = (mine4 && i < my_n) ? *reinterpret_cast<const float4*>((const float*)a.y + (int64_t)((int)my_rank * per + i) * a.ldy + f4)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
    const bool ok = n_kb > 0 && mbar_wait(tmem_full_bar, 0, &abort_flag, a.error_flag, 3);
    if (ok) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
    if (clustered) {
      // The K splits of a tile form a cluster.  Rank r owns the tokens [r * per, r * per + per): every
      // split writes its accumulator, token by token, into shared memory of its own (the ring, idle by
      // now), one region per owner, and sends each region to its owner's landing zone with ONE bulk
      // copy through distributed shared memory (cp.async.bulk.shared::cluster), which the owner's
      // barrier counts in.  (Element-wise remote stores, tried first, take 70 ns each and cannot be
      // overlapped: 4.4 us for 64 tokens, more than streaming the block's weights.)  The owner then
      // adds the splits' values in rank order: one order whatever the batch.
      const bool warp_reads = ok && quad * 32 < R;  // uniform for the warp
      // Token col lies at slot col of the travelling regions (owner col / per, place col % per: the regions
      // follow one another); this block's own tokens stay there and are read from there.  The epilogue runs
      // with one warp per scheduler, where every instruction costs its latency, so it is kept to one store per
      // element at a constant offset: columns past the last token are written too (nobody reads them).
      const uint32_t travel = base + 4u * (uint32_t)r_local;
      // (Compact code matters as much as short code here: a kernel of a decode step starts with cold
      // instruction caches, and every line of straight-line code is a miss of its own.  So: loops.)
#pragma unroll 1
      for (int c0 = 0; c0 < BN && warp_reads; c0 += 16) {
        if (c0 >= a.M) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const uint32_t at = travel + (uint32_t)c0 * kRowBytes;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(at + (uint32_t)j * kRowBytes), "r"(r[j]) : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes, as the bulk copies will read them
      asm volatile("barrier.sync 1, 128;" ::: "memory");
      // every peer's barrier exists from here on.  (Whole warps wait together: one lane of a warp waiting
      // for the cluster alone is held until the rest of its warp waits too.)
      asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
      met_cluster = true;
      if (et == 0) {
        for (uint32_t d = 1; ok && d < n_ranks; ++d) {
          const uint32_t dst = (my_rank + d) % n_ranks;
          const int dst_n = max(0, min(per, a.M - (int)dst * per));
          if (dst_n == 0) continue;
          uint32_t remote_zone, remote_bar;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_zone) : "r"(landing + my_rank * (uint32_t)per * kRowBytes), "r"(dst));
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(land_bar), "r"(dst));
          asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(remote_zone), "r"(base + dst * (uint32_t)per * kRowBytes), "r"((uint32_t)dst_n * kRowBytes), "r"(remote_bar)
                       : "memory");
        }
      }
      bool landed = ok;
      if (landed && my_n > 0 && n_ranks > 1) landed = mbar_wait(land_bar, 0, &abort_flag, a.error_flag, 7);
      if (et == 32 && landed && my_n > 0) {  // what the peers sent has arrived: they may leave
        // (relaxed: nothing this thread wrote has to be seen by them, only the copies' end, which the barrier
        // that let it pass has vouched for; with release semantics each arrival costs 0.35 us)
        for (uint32_t d = 1; d < n_ranks; ++d) {
          uint32_t remote_bar;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(sent_bar), "r"((my_rank + d) % n_ranks));
          asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
        }
      }
      // The owner adds the splits' values in rank order: a warp per token (every fourth), a lane per four
      // neighbouring features, so that a token's share of a row's sum of squares (norm ahead) is a butterfly in
      // the warp.  Kept small: this code runs once per block from cold instruction caches.
      const uint32_t rank_stride = (uint32_t)per * kRowBytes;
      const uint32_t zone = landing + 16u * (uint32_t)lane;                    // [source rank][owned token][feature]
      const uint32_t own = base + my_rank * rank_stride + 16u * (uint32_t)lane;  // this block's own share of its tokens
      const bool live = landed && mine4;
#pragma unroll 1
      for (int j = 0; quad + 4 * j < my_n; ++j) {
        const int i = quad + 4 * j, col = (int)my_rank * per + i;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
          for (uint32_t src = 0; src < n_ranks; ++src) {
            float4 v;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                         : "r"((src == my_rank ? own : zone + src * rank_stride) + (uint32_t)i * kRowBytes));
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
          }
          if (scaled) { const float r = row_inv[col]; sum.x *= r; sum.y *= r; sum.z *= r; sum.w *= r; }
        }
        float sq = 0.f;
        if (live) {
          if (MODE == kStoreBf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
            *reinterpret_cast<uint2*>((__nv_bfloat16*)a.y + (int64_t)col * a.ldy + f4) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          } else if (MODE == kStoreF32) {
            *reinterpret_cast<float4*>((float*)a.y + (int64_t)col * a.ldy + f4) = sum;
          } else {
            float* p = (float*)a.y + (int64_t)col * a.ldy + f4;
            const float4 before = j == 0 ? old4[0] : j == 1 ? old4[1] : j == 2 ? old4[2] : j == 3 ? old4[3] : *reinterpret_cast<const float4*>(p);
            const float4 nv = make_float4(before.x + sum.x, before.y + sum.y, before.z + sum.z, before.w + sum.w);
            *reinterpret_cast<float4*>(p) = nv;
            if (ahead) {
              __nv_bfloat162 lo = __floats2bfloat162_rn(nv.x * w_next4.x, nv.y * w_next4.y);
              __nv_bfloat162 hi = __floats2bfloat162_rn(nv.z * w_next4.z, nv.w * w_next4.w);
              *reinterpret_cast<uint2*>(a.ahead.xw + (int64_t)col * a.ahead.ldxw + f4) =
                  make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
              sq = nv.x * nv.x + nv.y * nv.y + nv.z * nv.z + nv.w * nv.w;
            }
          }
        }
        if (ahead) {  // uniform for the block: this tile's share of the token's sum of squares, in one fixed order
          sq += __shfl_xor_sync(0xffffffffu, sq, 16);
          sq += __shfl_xor_sync(0xffffffffu, sq, 8);
          sq += __shfl_xor_sync(0xffffffffu, sq, 4);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          if (lane == 0 && landed) a.ahead.ssq_part[(int64_t)blockIdx.x * a.M + col] = sq;
        }
      }
    } else if (stacked) {
      // lane L of the accumulator is row L % R of K-block group L / R; its partial products are the
      // columns [q*BN, q*BN + BN) of its own group q.  red[(q*BN + tok)*R + r], then a sum over q.
      if (ok) {
        const int L = quad * 32 + lane;
        const int q_mine = L / R, r_mine = L - q_mine * R;
        const int q_lo = (quad * 32) / R, q_hi = min(kstack - 1, (quad * 32 + 31) / R);  // uniform for the warp
        for (int q = q_lo; q <= q_hi; ++q) {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            if (c0 >= a.M) break;
            uint32_t r[16];
            tmem_ld16(taddr + q * BN + c0, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (q == q_mine) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + j < a.M) red[(q * BN + c0 + j) * R + r_mine] = __uint_as_float(r[j]);
            }
          }
        }
      }
      asm volatile("barrier.sync 1, 128;" ::: "memory");
      const float inv_R = 1.0f / (float)R;
      // tiles of 32 whole rows: a warp's 32 items are one token's row, so its share of the row's sum of
      // squares is a butterfly in the warp (the same order as below) and needs neither memory nor a barrier
      ssq_in_warp = ahead && R == 32 && f0 + 32 <= a.N;
      for (int idx = et; ok && idx < a.M * R; idx += 128) {
        // idx / R without the integer division: (idx + 0.5) / R is at least 1 / (2 R) away from an integer
        const int tok = (int)(((float)idx + 0.5f) * inv_R), rr = idx - tok * R;
        const int ff = f0 + rr;
        if (ff >= a.N) {
          if (ahead) sqbuf[idx] = 0.f;
          continue;
        }
        float v = 0.f;
        for (int q = 0; q < kstack; ++q) v += red[(q * BN + tok) * R + rr];
        if (scaled) v *= row_inv[tok];
        if (MODE == kStoreBf16) ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + ff] = __float2bfloat16_rn(v);
        else if (MODE == kStoreF32) ((float*)a.y)[(int64_t)tok * a.ldy + ff] = v;
        else if (MODE == kAccumF32) {
          float* p = (float*)a.y + (int64_t)tok * a.ldy + ff;
          const int n = (idx - et) >> 7;  // which of this thread's items
          const float nv = (n == 0 ? old_pre[0] : n == 1 ? old_pre[1] : n == 2 ? old_pre[2] : n == 3 ? old_pre[3] : *p) + v;
          *p = nv;
          if (ahead) {
            const float wn = n == 0 ? wn_pre[0] : n == 1 ? wn_pre[1] : n == 2 ? wn_pre[2] : n == 3 ? wn_pre[3] : a.ahead.w[ff];
            a.ahead.xw[(int64_t)tok * a.ahead.ldxw + ff] = __float2bfloat16_rn(nv * wn);
            if (ssq_in_warp) {
              float sq = nv * nv;
              sq += __shfl_xor_sync(0xffffffffu, sq, 16);
              sq += __shfl_xor_sync(0xffffffffu, sq, 8);
              sq += __shfl_xor_sync(0xffffffffu, sq, 4);
              sq += __shfl_xor_sync(0xffffffffu, sq, 2);
              sq += __shfl_xor_sync(0xffffffffu, sq, 1);
              if (lane == 0) a.ahead.ssq_part[(int64_t)blockIdx.x * a.M + tok] = sq;
            } else {
              sqbuf[idx] = nv * nv;
            }
          }
        }
      }
    }
    const bool warp_has_rows = ok && !stacked && !clustered && quad * 32 < R;  // uniform for the warp
#pragma unroll 1
    for (int c0 = 0; c0 < BN && warp_has_rows; c0 += 16) {
      if (c0 >= a.M) break;
      uint32_t r[16], u[16];
      tmem_ld16(taddr + c0, r);
      if (MODE == kGluBf16) tmem_ld16(taddr + BN + c0, u);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (!mine) {
        if (ahead && r_local < R)
          for (int j = 0; j < 16 && c0 + j < a.M; ++j) sqbuf[(c0 + j) * R + r_local] = 0.f;
        continue;
      }
      float old[16];
      if (MODE == kAccumF32) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          old[j] = c0 == 0 ? old16[j] : (c0 + j < a.M ? ((const float*)a.y)[(int64_t)(c0 + j) * a.ldy + f] : 0.f);
      }
      const float w_next = ahead ? a.ahead.w[f] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int tok = c0 + j;
        if (tok >= a.M) break;
        const float inv = scaled ? row_inv[tok] : 1.f;
        const float v = __uint_as_float(r[j]) * inv;
        if (MODE == kStoreBf16) {
          ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + f] = __float2bfloat16_rn(v);
        } else if (MODE == kStoreF32) {
          ((float*)a.y)[(int64_t)tok * a.ldy + f] = v;
        } else if (MODE == kAccumF32) {
          const float nv = old[j] + v;
          ((float*)a.y)[(int64_t)tok * a.ldy + f] = nv;
          if (ahead) {
            a.ahead.xw[(int64_t)tok * a.ahead.ldxw + f] = __float2bfloat16_rn(nv * w_next);
            sqbuf[tok * R + r_local] = nv * nv;
          }
        } else {
          const float up = __uint_as_float(u[j]) * inv;
          // silu with the fast exponential and division: their error (a few 2^-22) is far below the
          // bfloat16 rounding that follows, and the exact ones are most of this loop's time
          ((__nv_bfloat16*)a.y)[(int64_t)tok * a.ldy + f] = __float2bfloat16_rn(__fdividef(v, 1.0f + __expf(-v)) * up);
        }
      }
    }
    if (ahead && !ssq_in_warp && !clustered) {  // this block's share of the new rows' sums of squares, added up in a fixed order
      asm volatile("barrier.sync 1, 128;" ::: "memory");
      // a warp per token: lanes take the rows 32 apart, then a butterfly (one order whatever the batch)
      for (int tok = warp - 2; ok && tok < a.M; tok += 4) {
        float v = 0.f;
        for (int rr = lane; rr < R; rr += 32) v += sqbuf[tok * R + rr];
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        if (lane == 0) a.ahead.ssq_part[(int64_t)blockIdx.x * a.M + tok] = v;
      }
    }
  }
  if (clustered) {
    // A block's shared memory has to outlive the copies that read it: it leaves when every peer it sent to has
    // told it so (the copies INTO this block were over when its own barrier let it go on).  A peer that gave up
    // never tells; the wait is bounded like every other.
    if (!met_cluster) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    if (threadIdx.x == 64) {
      uint32_t rank, ranks;
      asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
      asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(ranks));
      const int per = (a.M + (int)ranks - 1) / (int)ranks;
      const int owners = (a.M + per - 1) / per;
      if (owners - ((int)rank < owners ? 1 : 0) > 0 && !abort_flag) mbar_wait(sent_bar, 0, &abort_flag, a.error_flag, 8);
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)ra.tmem_cols) : "memory");
  }
}

template <int BN, int MODE>
int launch_rows(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, int rows_per_block, int kkb, int kstack,
                int splits, cudaStream_t stream) {
  constexpr int kATiles = MODE == kGluBf16 ? 2 : 1;
  RowsArgs ra;
  ra.rows_per_block = rows_per_block;
  ra.kkb = kkb;
  ra.kstack = kstack;
  int cols = kATiles * kstack * BN;
  ra.tmem_cols = 32;
  while (ra.tmem_cols < cols) ra.tmem_cols *= 2;
  const int stage = kkb * (kATiles * rows_per_block * BK * 2 + BN * BK * 2);
  // behind the ring: the landing zone of the cluster epilogue or the stacked epilogue's sums, which
  // also is the room that the MMA, reading 128 rows whatever R is, may run into
  // [source rank][owned token][128 features], and four tokens' room behind it: the owner reads four at a time
  int landing = splits > 1 ? ((BN + splits - 1) / splits * splits + 4) * BM * 4 : 0;
  if (kstack > 1) landing = kstack * BN * rows_per_block * 4;
  if (a.ahead.xw != nullptr && splits == 1) landing += BN * rows_per_block * 4;  // the squares of the new rows (a cluster's owners add them up in their warps)
  const int over_read = (BM - kstack * rows_per_block) * BK * 2;
  ra.landing_bytes = landing > over_read ? landing : over_read;
  const int fixed = 16 + 8 * (2 * kRowsMaxStages + 3) + 1024 + ra.landing_bytes;
  ra.n_stages = (kRowsSmemBytes - fixed) / stage;
  if (ra.n_stages > kRowsMaxStages) ra.n_stages = kRowsMaxStages;
  if (ra.n_stages < 2) return fail(kBadArgument, "gemm_tc_rows: stages of %d bytes do not fit twice", stage);
  if (splits > 1 && ra.n_stages * stage < landing)  // the splits' tiles wait in the idle ring for their bulk copies
    return fail(kBadArgument, "gemm_tc_rows: a ring of %d bytes is too small for the K splits' tiles", ra.n_stages * stage);
  const int smem = fixed + ra.n_stages * stage;
  const dim3 grid((a.N + rows_per_block - 1) / rows_per_block, 1, splits);
  constexpr int M2 = MODE == kGluBf16 ? kStoreBf16 : MODE;  // (no gated instance of the cluster and stacked kernels is built)
  if (splits > 1) {
    if (MODE == kGluBf16) return fail(kBadArgument, "gemm_tc_rows: the gated product takes one K split");
    // the owners of a cluster write four neighbouring outputs of a token at once
    const int ybytes = MODE == kStoreBf16 ? 2 : 4;
    if (a.N % 4 || a.ldy % 4 || ((uintptr_t)a.y) % (4 * ybytes) ||
        (a.ahead.xw != nullptr && (a.ahead.ldxw % 4 || ((uintptr_t)a.ahead.xw) % 8 || ((uintptr_t)a.ahead.w) % 16)))
      return fail(kBadArgument, "gemm_tc_rows: K splits want the outputs in fours: N=%d, rows of y and of the norm-ahead "
                  "buffer in multiples of 4 elements, 16-byte aligned (8 for bfloat16)", a.N);
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_rows_kernel<BN, M2, kCluster>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kRowsSmemBytes);
      if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc_rows: cannot reserve shared memory: %s", cudaGetErrorString(e));
      configured = true;
    }
    launch_overlapped_cluster(gemm_tc_rows_kernel<BN, M2, kCluster>, grid, dim3(kThreads), (size_t)smem, stream,
                              (unsigned)splits, mw, mx, a, ra);
  } else if (kstack > 1) {
    if (MODE == kGluBf16) return fail(kBadArgument, "gemm_tc_rows: the gated product does not stack K blocks");
    if (BN > 64) return fail(kBadArgument, "gemm_tc_rows: K blocks are stacked for token tiles up to 64");
    constexpr int BS = BN > 64 ? 64 : BN;  // (no stacked kernel is built for the widest tile)
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_rows_kernel<BS, M2, kStacked>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kRowsSmemBytes);
      if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc_rows: cannot reserve shared memory: %s", cudaGetErrorString(e));
      configured = true;
    }
    launch_overlapped(gemm_tc_rows_kernel<BS, M2, kStacked>, grid, dim3(kThreads), (size_t)smem, stream, mw, mx, a, ra);
  } else {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_rows_kernel<BN, MODE, kPlain>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kRowsSmemBytes);
      if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc_rows: cannot reserve shared memory: %s", cudaGetErrorString(e));
      configured = true;
    }
    launch_overlapped(gemm_tc_rows_kernel<BN, MODE, kPlain>, grid, dim3(kThreads), (size_t)smem, stream, mw, mx, a, ra);
  }
  return check_launch("gemm_tc_rows");
}

template <int BN, int MODE>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, dim3 grid, cudaStream_t stream) {
  using C = Cfg<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc: cannot reserve %d bytes of shared memory: %s",
                                      C::kSmemBytes, cudaGetErrorString(e));
    configured = true;
  }
  launch_overlapped(gemm_tc_kernel<BN, MODE>, grid, dim3(kThreads), C::kSmemBytes, stream, mw, mx, a);
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
// box_kblocks > 1: a 3-D map (64 columns, rows, K blocks of 64 columns) whose boxes bring
// box_kblocks K blocks of box_rows rows, one after the other in shared memory; cols must be a
// multiple of 64 (a column past the end would be read from the next row, not filled with zero).
extern "C" int skyla_tensor_map_bf16(void* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                                     uint32_t box_rows, uint32_t box_kblocks) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(kLaunchFailed, "tensor map: the driver does not offer cuTensorMapEncodeTiled");
  if (((uintptr_t)ptr) % 16 || (ld * 2) % 16) return fail(kBadArgument, "tensor map: base or row stride is not a multiple of 16 bytes");
  if (box_rows == 0 || box_rows > 256) return fail(kBadArgument, "tensor map: box of %u rows", box_rows);
  alignas(64) CUtensorMap m;
  if (box_kblocks > 1) {
    if (cols % BK || box_kblocks > 256) return fail(kBadArgument, "tensor map: %u K blocks per box need columns in multiples of 64", box_kblocks);
    const cuuint64_t dims3[3] = {BK, rows, cols / BK};
    const cuuint64_t strides3[2] = {ld * 2, BK * 2};
    const cuuint32_t box3[3] = {BK, box_rows, box_kblocks};
    const cuuint32_t estr3[3] = {1, 1, 1};
    CUresult r3 = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims3, strides3, box3, estr3,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r3 != CUDA_SUCCESS) return fail(kLaunchFailed, "tensor map: cuTensorMapEncodeTiled (3-D) failed with %d", (int)r3);
    memcpy(out, &m, sizeof(m));
    return kOk;
  }
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

// How many clusters of `cluster` blocks of the weight-streaming kernel the current device holds at a time
// (one block per SM, clusters inside a GPC): a product whose tiles x K splits exceed it runs in two waves.
// Returns the count, or a negative error code.
extern "C" int skyla_gemm_tc_rows_max_clusters(int cluster) {
  if (cluster < 1 || cluster > kRowsMaxSplits) return fail(kBadArgument, "gemm_tc_rows: clusters of %d blocks", cluster);
  auto kernel = gemm_tc_rows_kernel<64, kAccumF32, kCluster>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRowsSmemBytes);
  if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc_rows: cannot reserve shared memory: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1024, 1, cluster);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kRowsSmemBytes - 4096;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
  if (e != cudaSuccess) return fail(kLaunchFailed, "gemm_tc_rows: cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(e));
  return n;
}

extern "C" int skyla_gemm_tc_stages(int bn, int mode) {
  if (mode == kGluBf16) return bn == 16 ? Cfg<16, kGluBf16>::kStages : bn == 32 ? Cfg<32, kGluBf16>::kStages
                             : bn == 64 ? Cfg<64, kGluBf16>::kStages : bn == 128 ? Cfg<128, kGluBf16>::kStages
                             : Cfg<256, kGluBf16>::kStages;
  return bn == 16 ? Cfg<16, 0>::kStages : bn == 32 ? Cfg<32, 0>::kStages : bn == 64 ? Cfg<64, 0>::kStages
       : bn == 128 ? Cfg<128, 0>::kStages : Cfg<256, 0>::kStages;
}

// map_w: weight [rows, K] with boxes of 128 rows (a gated weight: the N gate rows, then the N up rows);
// map_x: tokens [M, K] with boxes of bn rows.  Whole K in every block: the products of 17 to 128 tokens of
// weights whose K is too short (or whose width too odd) for the weight-streaming kernel.
extern "C" int skyla_gemm_tc(const void* map_w, const void* map_x, void* y, int64_t ldy, int M, int N, int K, int bn,
                             int mode, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || K % 8) return fail(kBadArgument, "gemm_tc: K=%d must be a positive multiple of 8", K);
  if (mode < 0 || mode > kGluBf16) return fail(kBadArgument, "gemm_tc: unknown epilogue %d", mode);
  alignas(64) CUtensorMap mw, mx;
  memcpy(&mw, map_w, sizeof(mw));
  memcpy(&mx, map_x, sizeof(mx));
  GemmArgs a{y, ldy, M, N, K, (K + BK - 1) / BK, error_flag};
  dim3 grid((N + BM - 1) / BM, (M + bn - 1) / bn, 1);
  if (grid.y > 65535) return fail(kBadArgument, "gemm_tc: grid too large");
  switch (mode) {
    case kStoreBf16: return launch_bn<kStoreBf16>(bn, mw, mx, a, grid, stream);
    case kStoreF32: return launch_bn<kStoreF32>(bn, mw, mx, a, grid, stream);
    case kAccumF32: return launch_bn<kAccumF32>(bn, mw, mx, a, grid, stream);
    default: return launch_bn<kGluBf16>(bn, mw, mx, a, grid, stream);
  }
}

// Few tokens (at most 64): blocks of `rows_per_block` weight rows (a multiple of 8, at most 128), K cut
// into `splits` (at most 8) that meet in a thread-block cluster.  map_w has boxes of rows_per_block rows
// and `kkb` K blocks (kkb > 1: a 3-D map, see skyla_tensor_map_bf16), of which one MMA takes `kstack` at
// once (stacked along its rows; one split then).  x comes by map_x (bf16 [M, K], boxes of bn rows
// and kkb K blocks).
// Modes: store bf16 / f32, accumulate into f32 y, gated (bf16, one split).
// ahead_*: with the accumulate epilogue, also leave bf16(y_new * ahead_w) in ahead_xw [M, N] and this
// launch's blocks' shares of the new rows' sums of squares in ahead_ssq [blocks, M].
// scale_*: the result is multiplied by 1/sqrt(sum_p scale_ssq[p, tok] / K + scale_eps).
extern "C" int skyla_gemm_tc_rows(const void* map_w, const void* map_x, void* y, int64_t ldy, int M, int N, int K, int bn,
                                  int mode, int rows_per_block, int kkb, int kstack, int splits, int* error_flag,
                                  const float* ahead_w, void* ahead_xw, int64_t ahead_ldxw, float* ahead_ssq,
                                  const float* scale_ssq, int scale_parts, float scale_eps, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || K % 8) return fail(kBadArgument, "gemm_tc_rows: K=%d must be a positive multiple of 8", K);
  if (rows_per_block < 8 || rows_per_block > BM || rows_per_block % 8)
    return fail(kBadArgument, "gemm_tc_rows: %d rows per block (a multiple of 8 up to 128)", rows_per_block);
  if (M > bn || (bn != 16 && bn != 32 && bn != 64 && bn != 128)) return fail(kBadArgument, "gemm_tc_rows: %d tokens in a tile of %d", M, bn);
  if (mode != kStoreBf16 && mode != kStoreF32 && mode != kAccumF32 && mode != kGluBf16)
    return fail(kBadArgument, "gemm_tc_rows: epilogue %d is not offered", mode);
  if (kkb < 1 || kkb > 16 || (kkb > 1 && K % BK))
    return fail(kBadArgument, "gemm_tc_rows: %d K blocks per box need 1..16 and K=%d a multiple of 64", kkb, K);
  if (kstack < 1 || kkb % kstack || kstack * rows_per_block > BM || kstack * bn > 256 ||
      (kstack > 1 && (splits != 1 || mode == kGluBf16)))
    return fail(kBadArgument, "gemm_tc_rows: stacking %d K blocks needs kstack | kkb, kstack * rows <= 128, kstack * tile <= 256, "
                "one split and no gating", kstack);
  const int total_kb = (K + BK - 1) / BK;
  if (splits < 1 || splits > kRowsMaxSplits || splits > total_kb || (mode == kGluBf16 && splits != 1))
    return fail(kBadArgument, "gemm_tc_rows: %d K splits (1..8, one for the gated product)", splits);
  if (map_w == nullptr || map_x == nullptr) return fail(kBadArgument, "gemm_tc_rows: both operands come by tensor maps");
  alignas(64) CUtensorMap mw, mx;
  memcpy(&mw, map_w, sizeof(mw));
  memcpy(&mx, map_x, sizeof(mx));
  int kps = (total_kb + splits - 1) / splits;
  kps = (kps + kkb - 1) / kkb * kkb;  // whole boxes per split
  if ((splits - 1) * kps >= total_kb) return fail(kBadArgument, "gemm_tc_rows: %d splits leave one without K blocks", splits);
  GemmArgs a{y, ldy, M, N, K, kps, error_flag};
  if (ahead_xw != nullptr) {
    if (mode != kAccumF32 || ahead_w == nullptr || ahead_ssq == nullptr)
      return fail(kBadArgument, "gemm_tc_rows: norm-ahead goes with the accumulate epilogue, a norm weight and room for the sums");
    a.ahead = NormAhead{ahead_w, (__nv_bfloat16*)ahead_xw, ahead_ldxw, ahead_ssq};
  }
  if (scale_ssq != nullptr) {
    if (scale_parts < 1) return fail(kBadArgument, "gemm_tc_rows: handed-in sums of squares come in one share at least");
    a.scale = ScaleIn{scale_ssq, scale_parts, scale_eps, K};
  }
#define SKYLA_ROWS_BN(MODE_)                                                                          \
  switch (bn) {                                                                                       \
    case 16: return launch_rows<16, MODE_>(mw, mx, a, rows_per_block, kkb, kstack, splits, stream);   \
    case 32: return launch_rows<32, MODE_>(mw, mx, a, rows_per_block, kkb, kstack, splits, stream);   \
    case 64: return launch_rows<64, MODE_>(mw, mx, a, rows_per_block, kkb, kstack, splits, stream);   \
    default: return launch_rows<128, MODE_>(mw, mx, a, rows_per_block, kkb, kstack, splits, stream);  \
  }
  switch (mode) {
    case kStoreBf16: SKYLA_ROWS_BN(kStoreBf16)
    case kStoreF32: SKYLA_ROWS_BN(kStoreF32)
    case kAccumF32: SKYLA_ROWS_BN(kAccumF32)
    default: SKYLA_ROWS_BN(kGluBf16)
  }
#undef SKYLA_ROWS_BN
}
