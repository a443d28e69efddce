// Tensor-core matrix product for prompts on sm_100a: y = x W^T, x[M,K] tokens and W[N,K]
// (rows are outputs) both bfloat16 and K-major, 32-bit accumulation in TMEM.
//
// Here the TOKENS are the 128-row operand of tcgen05.mma and 256 outputs are its N, so a
// thread of the epilogue owns one token's row of the tile.  What the reference does in passes
// of their own over a prompt's activations (skyla-engine/src/graph.rs:96-130: rms_norm, matmul,
// qkv_prep, matmul with ACCUM, rms_norm, matmul, silu_mul, matmul with ACCUM) is then per-row
// arithmetic on an accumulator that is already in registers:
//   * "scale in": the token operand came as bf16(x * norm weight); the row's 1/sqrt(mean(x^2)+eps)
//     is applied to the accumulator (RMSNorm is a row scalar times a column weight, and the
//     scalar commutes with the product; skyla-ref/src/ops.rs:8-11);
//   * the residual add goes out as TMA reduce-adds from shared memory (the tile never has to be
//     read back), 128 tokens x 32 outputs at a time;
//   * "norm ahead": the product that adds into the residual stream also leaves bf16(x_new * w_next)
//     and its tile's share of the rows' sums of squares for the norm that reads x next;
//   * silu(gate) * up of a gated weight (skyla-shaders/shaders/silu_mul.comp:15-24);
//   * the per-head q/k RMSNorm, the rotation at the token's position and the write of k and v
//     into the paged cache (skyla-shaders/shaders/qkv_prep.comp:67-123), when a head's columns
//     lie within one tile (head sizes 32, 64, 128, 256).
//
// One block per SM walks the output tiles (tiles of one weight tile are neighbours, so blocks
// that run together share it through L2).  Where the tiles are at most half the SMs (a prompt of
// a few hundred tokens), each is cut along K into up to four equal runs of K blocks, one run per
// block: a block whose run starts inside a tile leaves its accumulator in scratch (a "share")
// and raises a flag; the block that has the tile's first K blocks adds the shares into its own
// accumulator in block order and runs the epilogue.  The sum order is fixed by the shapes alone.
// Roles:
//   warp 0    one lane issues TMA loads of a [128 tokens x 64] and two [128 outputs x 64] boxes
//             a stage (a gated weight: 128 gate rows and the 128 up rows that go with them);
//   warp 1    allocates TMEM (two accumulators of 256 columns); one lane issues tcgen05.mma
//             (M=128, N=256, K=16) and commits each stage back to the loader;
//   warps 2-5 drain accumulator i (tcgen05.ld: lane = token, column = output) while the MMA
//             warp fills accumulator i+1.
// Every mbarrier wait is bounded: on a timeout the block records an error code, lets the loads
// it issued land, frees its TMEM and returns.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "tc_common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
using namespace skyla::tc;

enum Mode : int {
  kStoreBf16 = 0,  // y[tok, f] = acc                  (bfloat16)
  kStoreF32 = 1,   // y[tok, f] = acc                  (float)
  kAccumF32 = 2,   // y[tok, f] += acc                 (float: the residual sum), optionally "norm ahead"
  kGluBf16 = 3,    // y[tok, f] = silu(gate) * up      (bfloat16; W = N gate rows, then the N up rows)
  kQkvPrep = 4,    // heads of q, k, v: norm, rotation, q to y (bfloat16), k and v into the cache
};

constexpr int BT = 128;  // tokens per tile: the MMA's M
constexpr int BF = 256;  // accumulator columns per tile: the MMA's N
constexpr int BK = 64;   // K elements per stage: one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr int kXBytes = BT * BK * 2, kWBytes = BF * BK * 2;
constexpr int kStageBytes = kXBytes + kWBytes;  // 48 KB
constexpr int kStages = 4;
constexpr int kOutCols = 32;                  // outputs per TMA store of the epilogue: 128 bytes of floats
constexpr int kOutBytes = BT * kOutCols * 4;  // 16 KB, twice: one is filled while the other is read
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kOutBytes + 1024 /*align*/ + 256 /*barriers*/;
static_assert(kSmemBytes <= 227 * 1024, "shared memory of a block");
constexpr int kTmemCols = 2 * BF;

struct ScaleIn { const float* ssq_part; int n_parts; float eps; int width; };           // ssq_part[p * M + tok]
struct NormAhead { const float* w; __nv_bfloat16* xw; int64_t ldxw; float* ssq_part; };  // ssq_part[f_tile * M + tok]
struct QkvPrep {
  int nq, nkv, hd;
  const float* q_norm; const float* k_norm; float eps;  // null: that head kind is not normed
  const float* cos_t; const float* sin_t;               // [positions][hd / 2]; null: no rotation
  const int32_t* tok_pos; const int32_t* tok_slot;
  __nv_bfloat16* k_pool; __nv_bfloat16* v_pool;          // [page][kv head][page_size][hd]
  const int32_t* page_table; int max_pages; int page_size;
};
struct PromptArgs {
  void* y; int64_t ldy;  // kQkvPrep: the prepared queries [M, nq * hd]
  int M, N, K;           // tokens, outputs (after gating), reduction length
  int vec;               // rows of y (and of ahead.xw) start on 16 bytes: whole chunks go as vectors
  int y_tma;             // kAccumF32: the kernel got a tensor map of y and adds by TMA reduce
  float* share;          // [block][BF / 4][BT rows][4] accumulators of tiles that are cut along K; null: none are
  int* share_flags;      // [block]: 1 while that block's share waits to be taken; zero between launches
  int* error_flag;
  ScaleIn scale;         // scale.ssq_part == nullptr: none
  NormAhead ahead;       // ahead.xw == nullptr: none
  QkvPrep prep;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
// 16 consecutive outputs of one token: as two 16-byte vectors where the row allows, else one by one
__device__ __forceinline__ void store16_bf16(__nv_bfloat16* dst, const float* v, int n, bool vec) {
  if (vec && n == 16) {
    uint4 lo, hi;
    lo.x = pack_bf16(v[0], v[1]); lo.y = pack_bf16(v[2], v[3]); lo.z = pack_bf16(v[4], v[5]); lo.w = pack_bf16(v[6], v[7]);
    hi.x = pack_bf16(v[8], v[9]); hi.y = pack_bf16(v[10], v[11]); hi.z = pack_bf16(v[12], v[13]); hi.w = pack_bf16(v[14], v[15]);
    reinterpret_cast<uint4*>(dst)[0] = lo;
    reinterpret_cast<uint4*>(dst)[1] = hi;
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (j < n) dst[j] = __float2bfloat16_rn(v[j]);
  }
}
__device__ __forceinline__ void store16_f32(float* dst, const float* v, int n, bool vec) {
  if (vec && n == 16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (j < n) dst[j] = v[j];
  }
}
__device__ __forceinline__ void load16_f32(const float* src, float* v, int n, bool vec) {
  if (vec && n == 16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 t = reinterpret_cast<const float4*>(src)[q];
      v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = j < n ? src[j] : 0.f;
  }
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- which work a block does, computed alike by its three roles: whole tiles (tile = blockIdx.x +
// i * gridDim.x), or, where the tiles are cut along K, one run of units (unit = one K block of one tile)
struct Plan {
  int total_kb, n_whole;
  long long u, u_end, units;
};
struct Segment { int tile, kb0, kb1; };

__device__ __forceinline__ Plan make_plan(const PromptArgs& a, int n_tiles, int total_kb) {
  Plan p;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  p.total_kb = total_kb;
  if (a.share == nullptr) {
    p.n_whole = b < n_tiles ? (n_tiles - b + G - 1) / G : 0;
    p.units = p.u = p.u_end = 0;
  } else {
    p.n_whole = 0;
    p.units = (long long)n_tiles * total_kb;
    p.u = p.units * b / G;
    p.u_end = p.units * (b + 1) / G;
  }
  return p;
}
__device__ __forceinline__ bool next_segment(Plan& p, int& i, Segment& s) {
  if (i < p.n_whole) {
    s.tile = (int)blockIdx.x + i * (int)gridDim.x;
    s.kb0 = 0;
    s.kb1 = p.total_kb;
    ++i;
    return true;
  }
  if (p.u >= p.u_end) return false;
  s.tile = (int)(p.u / p.total_kb);
  s.kb0 = (int)(p.u % p.total_kb);
  const long long left = p.u_end - p.u;
  s.kb1 = (long long)(p.total_kb - s.kb0) <= left ? p.total_kb : s.kb0 + (int)left;
  p.u += s.kb1 - s.kb0;
  ++i;
  return true;
}

// ---- the epilogues: one thread, one token's row of the tile.  tcgen05.ld is a warp's business:
// every lane runs every load; only what touches global memory looks at `valid`.

template <int MODE>
__device__ __forceinline__ void drain_plain(const PromptArgs& a, uint32_t taddr, int tok, bool valid, int f0, float s) {
  const bool vec = a.vec != 0;
  const int width = MODE == kGluBf16 ? BF / 2 : BF;
  float old_next[16];
  if (MODE == kAccumF32) {
    const int n = min(16, a.N - f0);
    if (valid && n > 0) load16_f32((const float*)a.y + (int64_t)tok * a.ldy + f0, old_next, n, vec);
  }
  float ssq = 0.f;
#pragma unroll 1
  for (int c0 = 0; c0 < width; c0 += 16) {
    const int f = f0 + c0;
    if (f >= a.N) break;  // the same for the whole warp
    const int n = min(16, a.N - f);
    uint32_t r[16], u[16];
    __syncwarp();
    tmem_ld16(taddr + c0, r);
    if (MODE == kGluBf16) tmem_ld16(taddr + BF / 2 + c0, u);
    float old[16];
    if (MODE == kAccumF32) {
#pragma unroll
      for (int j = 0; j < 16; ++j) old[j] = old_next[j];
      const int fn = f + 16, nn = min(16, a.N - fn);  // the next chunk's old values are asked for now
      if (valid && c0 + 16 < width && nn > 0) load16_f32((const float*)a.y + (int64_t)tok * a.ldy + fn, old_next, nn, vec);
    }
    tmem_wait_ld();
    float v[16];
    if (!valid) {
      // a row beyond the last token: nothing to write
    } else if (MODE == kGluBf16) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float g = __uint_as_float(r[j]) * s, up = __uint_as_float(u[j]) * s;
        v[j] = g / (1.0f + expf(-g)) * up;
      }
      store16_bf16((__nv_bfloat16*)a.y + (int64_t)tok * a.ldy + f, v, n, vec);
    } else if (MODE == kStoreBf16) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) * s;
      store16_bf16((__nv_bfloat16*)a.y + (int64_t)tok * a.ldy + f, v, n, vec);
    } else if (MODE == kStoreF32) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) * s;
      store16_f32((float*)a.y + (int64_t)tok * a.ldy + f, v, n, vec);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = old[j] + __uint_as_float(r[j]) * s;
      store16_f32((float*)a.y + (int64_t)tok * a.ldy + f, v, n, vec);
      if (a.ahead.xw != nullptr) {
        float w[16];
        load16_f32(a.ahead.w + f, w, n, vec);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j < n) ssq = fmaf(v[j], v[j], ssq);
          w[j] *= v[j];
        }
        store16_bf16(a.ahead.xw + (int64_t)tok * a.ahead.ldxw + f, w, n, vec);
      }
    }
  }
  if (MODE == kAccumF32 && a.ahead.xw != nullptr && valid) a.ahead.ssq_part[(int64_t)(f0 / BF) * a.M + tok] = ssq;
}

// y += acc without reading y: 32 outputs of the tile's 128 tokens at a time are laid out in shared
// memory the way a 128-byte-swizzled tensor map expects them (row r's 16-byte piece c at
// r * 128 + ((c ^ (r & 7)) * 16): the threads of a warp, one row each, hit different banks) and one
// thread sends them off as a TMA reduce-add, which clips what lies beyond the matrix.  Two buffers
// take turns; `n_sent` counts the sends of this block so that the turns go on across tiles.
__device__ __forceinline__ void drain_reduce(const PromptArgs& a, const CUtensorMap* map_y, uint32_t taddr, uint32_t out_smem,
                                             int row, int tok0, int f0, float s, bool sender, int& n_sent) {
#pragma unroll 1
  for (int c0 = 0; c0 < BF; c0 += kOutCols) {
    if (f0 + c0 >= a.N) break;  // the same for all four warps
    const uint32_t buf = out_smem + (uint32_t)(n_sent & 1) * kOutBytes;
    // the send that read this buffer last (two sends ago) must be done with it
    if (sender) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    asm volatile("barrier.sync 1, 128;" ::: "memory");
    uint32_t r[32];
    tmem_ld16(taddr + c0, r);
    tmem_ld16(taddr + c0 + 16, r + 16);
    tmem_wait_ld();
    const uint32_t row_smem = buf + (uint32_t)row * 128u;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                   ::"r"(row_smem + (uint32_t)((c ^ (row & 7)) << 4)), "f"(__uint_as_float(r[4 * c]) * s),
                     "f"(__uint_as_float(r[4 * c + 1]) * s), "f"(__uint_as_float(r[4 * c + 2]) * s),
                     "f"(__uint_as_float(r[4 * c + 3]) * s) : "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the TMA unit reads what the threads wrote
    asm volatile("barrier.sync 1, 128;" ::: "memory");
    if (sender) {
      asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                   ::"l"(map_y), "r"(buf), "r"(f0 + c0), "r"(tok0) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    ++n_sent;
  }
}

// The heads whose columns this tile holds: q and k heads are normed over the head and rotated
// (pairs (i, i + hd/2): out_i = x_i cos - x_{i+hd/2} sin, out_{i+hd/2} = x_i sin + x_{i+hd/2} cos,
// skyla-ref/src/rope.rs:59-68), q goes to y, k and v to the token's place in the cache.
__device__ __forceinline__ void drain_qkv(const PromptArgs& a, uint32_t taddr, int tok, bool valid, int f0, float s) {
  const QkvPrep& p = a.prep;
  const int hd = p.hd, half = hd >> 1, n_heads = p.nq + 2 * p.nkv;
  int pos = 0;
  int64_t cache_row = 0;  // (page * nkv) * page_size + place in the page, to which kv_head * page_size is added
  if (valid) {
    pos = p.tok_pos[tok];
    if (p.k_pool != nullptr) {
      const int page = p.page_table[(int64_t)p.tok_slot[tok] * p.max_pages + pos / p.page_size];
      cache_row = (int64_t)page * p.nkv * p.page_size + pos % p.page_size;
    }
  }
  for (int c_head = 0; c_head < BF; c_head += hd) {
    const int head = (f0 + c_head) / hd;
    if (head >= n_heads) break;
    const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
    const int kvh = is_q ? 0 : (is_k ? head - p.nq : head - p.nq - p.nkv);
    __nv_bfloat16* dst = nullptr;
    if (valid) {
      if (is_q) dst = (__nv_bfloat16*)a.y + (int64_t)tok * a.ldy + (int64_t)head * hd;
      else if (p.k_pool != nullptr) dst = (is_k ? p.k_pool : p.v_pool) + (cache_row + (int64_t)kvh * p.page_size) * hd;
    }
    const float* nw = is_q ? p.q_norm : (is_k ? p.k_norm : nullptr);
    const uint32_t t0 = taddr + c_head;
    float rs = s;  // the row's scalar, times the head's once it is known
    if (nw != nullptr) {
      float ssq = 0.f;
#pragma unroll 1
      for (int c = 0; c < hd; c += 16) {
        uint32_t r[16];
        __syncwarp();
        tmem_ld16(t0 + c, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) { const float v = __uint_as_float(r[j]) * s; ssq = fmaf(v, v, ssq); }
      }
      rs = s * (1.0f / sqrtf(ssq / (float)hd + p.eps));
    }
    const bool rotate = (is_q || is_k) && p.cos_t != nullptr;
    if (!rotate) {
#pragma unroll 1
      for (int c = 0; c < hd; c += 16) {
        uint32_t r[16];
        __syncwarp();
        tmem_ld16(t0 + c, r);
        tmem_wait_ld();
        if (dst != nullptr) {
          float v[16];
          if (nw != nullptr) load16_f32(nw + c, v, 16, true);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) * rs * (nw != nullptr ? v[j] : 1.0f);
          store16_bf16(dst + c, v, 16, true);
        }
      }
      continue;
    }
#pragma unroll 1
    for (int c = 0; c < half; c += 16) {
      uint32_t lo[16], hi[16];
      __syncwarp();
      tmem_ld16(t0 + c, lo);
      tmem_ld16(t0 + half + c, hi);
      tmem_wait_ld();
      if (dst != nullptr) {
        float x0[16], x1[16], cs[16], sn[16];
        if (nw != nullptr) {
          load16_f32(nw + c, x0, 16, true);
          load16_f32(nw + half + c, x1, 16, true);
        }
        load16_f32(p.cos_t + (int64_t)pos * half + c, cs, 16, true);
        load16_f32(p.sin_t + (int64_t)pos * half + c, sn, 16, true);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float a0 = __uint_as_float(lo[j]) * rs * (nw != nullptr ? x0[j] : 1.0f);
          const float a1 = __uint_as_float(hi[j]) * rs * (nw != nullptr ? x1[j] : 1.0f);
          x0[j] = a0 * cs[j] - a1 * sn[j];
          x1[j] = a0 * sn[j] + a1 * cs[j];
        }
        store16_bf16(dst + c, x0, 16, true);
        store16_bf16(dst + half + c, x1, 16, true);
      }
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_prompt_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_y, const PromptArgs a, int n_t_tiles, int n_f_tiles) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t out_smem = base + kStages * kStageBytes;  // the epilogue's two buffers for TMA stores
  const uint32_t bars = out_smem + 2 * kOutBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * kStages + 2 + b); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (a.K + BK - 1) / BK;
  const int n_tiles = n_f_tiles * n_t_tiles;
  constexpr int kTileOutputs = MODE == kGluBf16 ? BF / 2 : BF;  // outputs a tile covers

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
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
                 ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)kTmemCols) : "memory");
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
      int kbg = 0;  // K blocks loaded so far, over all segments
      bool ok = true;
      Plan plan = make_plan(a, n_tiles, total_kb);
      Segment sg;
      for (int i = 0; ok && next_segment(plan, i, sg);) {
        const int f_tile = sg.tile / n_t_tiles, t_tile = sg.tile % n_t_tiles;
        const int row0 = f_tile * kTileOutputs;
        const int row1 = MODE == kGluBf16 ? a.N + row0 : row0 + BF / 2;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++kbg) {
          const int s = kbg % kStages;
          const uint32_t phase = (kbg / kStages) & 1;
          if (!mbar_wait(empty_bar(s), phase ^ 1, &abort_flag, a.error_flag, 1)) { ok = false; break; }
          const uint32_t sx = base + s * kStageBytes, sw = sx + kXBytes;
          mbar_expect_tx(full_bar(s), kStageBytes);
          tma_load_2d(sx, &map_x, full_bar(s), kb * BK, t_tile * BT);
          tma_load_2d(sw, &map_w, full_bar(s), kb * BK, row0);
          tma_load_2d(sw + kWBytes / 2, &map_w, full_bar(s), kb * BK, row1);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (phase << s);
        }
      }
      if (!ok)  // gave up: let the loads already issued land before the block's memory goes away
        for (int s = 0; s < kStages; ++s)
          if (armed & (1u << s)) {
            const long long t0 = clock64();
            while (!mbar_try_wait(full_bar(s), (armed_parity >> s) & 1) && clock64() - t0 < kWaitCycles) {}
          }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BF >> 3) << 17) |
                             ((uint32_t)(BT >> 4) << 24);
      int kbg = 0;
      bool ok = true;
      Plan plan = make_plan(a, n_tiles, total_kb);
      Segment sg;
      for (int i = 0; ok && next_segment(plan, i, sg);) {
        const int it = i - 1, buf = it & 1;
        // the epilogue must have drained this accumulator (two segments ago)
        if (!mbar_wait(acc_empty_bar(buf), ((it >> 1) & 1) ^ 1, &abort_flag, a.error_flag, 5)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_base + buf * BF;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++kbg) {
          const int s = kbg % kStages;
          const uint32_t phase = (kbg / kStages) & 1;
          if (!mbar_wait(full_bar(s), phase, &abort_flag, a.error_flag, 2)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sx = base + s * kStageBytes, sw = sx + kXBytes;
          const uint64_t dx = umma_desc(sx), dw = umma_desc(sw);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_bf16(d, dx + 2 * k, dw + 2 * k, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(s));
        }
        umma_commit(acc_full_bar(buf));
      }
    }
  } else {
    grid_dependency_wait();
    const int quad = warp & 3, row = quad * 32 + lane;
    const bool by_tma = MODE == kAccumF32 && a.y_tma != 0;
    const bool sender = warp == 2 && lane == 0;
    const int G = (int)gridDim.x, me = (int)blockIdx.x;
    constexpr int kShareVecs = BT * BF / 4;  // a share: [4 columns][row] as float4, a warp's 32 rows 512 bytes in a row
    int n_sent = 0;
    Plan plan = make_plan(a, n_tiles, total_kb);
    const long long units = plan.units;
    Segment sg;
    for (int i = 0; next_segment(plan, i, sg);) {
      const int it = i - 1, buf = it & 1;
      const int f_tile = sg.tile / n_t_tiles, t_tile = sg.tile % n_t_tiles;
      const int tok = t_tile * BT + row;
      const bool valid = tok < a.M;
      const bool gives = sg.kb0 > 0;                        // another block has the tile's first K blocks
      const bool takes = sg.kb0 == 0 && sg.kb1 < total_kb;  // this block finishes the tile from others' shares
      float s = 1.0f;
      if (a.scale.ssq_part != nullptr && valid && !gives) {  // while the tile's products run
        float v = 0.f;
        for (int p = 0; p < a.scale.n_parts; ++p) v += a.scale.ssq_part[(int64_t)p * a.M + tok];
        s = 1.0f / sqrtf(v / (float)a.scale.width + a.scale.eps);
      }
      int n_parts = 0;
      if (takes) {  // the blocks after this one whose runs begin inside this tile
        const long long tile_end = (long long)(sg.tile + 1) * total_kb;
        while (me + 1 + n_parts < G && units * (me + 1 + n_parts) / G < tile_end) ++n_parts;
      }
      if (!mbar_wait(acc_full_bar(buf), (it >> 1) & 1, &abort_flag, a.error_flag, 3)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + buf * BF + ((uint32_t)(quad * 32) << 16);
      if (gives) {
        // leave the accumulator for the block that has the tile's first K blocks
        float4* sh = (float4*)a.share + (int64_t)me * kShareVecs + row;
#pragma unroll 1
        for (int c0 = 0; c0 < BF; c0 += 64) {
          uint32_t r[64];
          __syncwarp();
#pragma unroll
          for (int g = 0; g < 4; ++g) tmem_ld16(taddr + c0 + 16 * g, r + 16 * g);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            __stcg(sh + (int64_t)(c0 / 4 + j) * BT, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
        }
        __threadfence();
        asm volatile("barrier.sync 1, 128;" ::: "memory");
        if (sender) atomicExch(a.share_flags + me, 1);
      } else {
        if (takes) {
          if (sender) {
            for (int q = 0; q < n_parts && !abort_flag; ++q) {
              const volatile int* flag = a.share_flags + me + 1 + q;
              const long long t0 = clock64();
              while (*flag == 0) {
                if (clock64() - t0 > kWaitCycles) {
                  abort_flag = 1;
                  if (a.error_flag != nullptr) atomicCAS(a.error_flag, 0, 6);
                  break;
                }
              }
            }
            __threadfence();
          }
          asm volatile("barrier.sync 1, 128;" ::: "memory");
          if (abort_flag) break;  // the same for all four warps: written before the barrier
          // add the shares into the accumulator where it lies, in block order; 64 columns' loads are
          // in flight together (taken one by one with the epilogue's steps they cost a trip to L2 each)
          const float4* sh = (const float4*)a.share + (int64_t)(me + 1) * kShareVecs + row;
#pragma unroll 1
          for (int c0 = 0; c0 < BF; c0 += 64) {
#pragma unroll 1
            for (int q = 0; q < n_parts; ++q) {
              float4 v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __ldcg(sh + (int64_t)q * kShareVecs + (int64_t)(c0 / 4 + j) * BT);
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint32_t r[16];
                __syncwarp();
                tmem_ld16(taddr + c0 + 16 * g, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v[4 * g + j].x);
                  r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v[4 * g + j].y);
                  r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v[4 * g + j].z);
                  r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v[4 * g + j].w);
                }
                tmem_st16(taddr + c0 + 16 * g, r);
              }
              asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
          }
          // the shares are read: their flags go back to zero for the next launch
          asm volatile("barrier.sync 1, 128;" ::: "memory");
          if (sender)
            for (int q = 0; q < n_parts; ++q) a.share_flags[me + 1 + q] = 0;
        }
        if (MODE == kQkvPrep) drain_qkv(a, taddr, tok, valid, f_tile * kTileOutputs, s);
        else if (by_tma) drain_reduce(a, &map_y, taddr, out_smem, row, t_tile * BT, f_tile * kTileOutputs, s, sender, n_sent);
        else drain_plain<MODE>(a, taddr, tok, valid, f_tile * kTileOutputs, s);
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(buf));
    }
    if (by_tma && sender) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the buffers go away with the block
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (lane == 0) {  // every accumulator must be idle before its columns are freed
      Plan plan = make_plan(a, n_tiles, total_kb);
      Segment sg;
      int my_segments = 0;
      while (next_segment(plan, my_segments, sg)) {}
      for (int b = 0; b < 2; ++b) {
        const int uses = (my_segments + 1 - b) / 2;  // segments that used accumulator b
        if (uses > 0) {
          const long long t0 = clock64();
          while (!mbar_try_wait(acc_full_bar(b), (uses - 1) & 1) && clock64() - t0 < kWaitCycles) {}
        }
      }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
  }
}

// Whether `tiles` tiles of `total_kb` K blocks are cut along K, and over how many blocks: where the
// tiles are at most half the SMs, every tile is cut into the same number of runs, at most four (the
// tile's owner reads the other runs' accumulators through its one SM: about 3 us each) of at least
// 8 K blocks.  0: whole tiles.  (Cutting only a last, partial round of many tiles measured slower
// than leaving it: 63 against 57 us for 256 tiles of 64 K blocks.)
int cut_blocks(long long tiles, long long total_kb, int n_sms) {
  if (tiles <= 0 || tiles * 2 > n_sms) return 0;
  long long runs = n_sms / tiles;
  if (runs > 4) runs = 4;
  if (runs > total_kb / 8) runs = total_kb / 8;
  return runs < 2 ? 0 : (int)(tiles * runs);
}

template <int MODE>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& my, const PromptArgs& a, int share_blocks,
           cudaStream_t stream) {
  static bool configured = false;
  static int n_sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_prompt_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess)
      return fail(kLaunchFailed, "gemm_prompt: cannot reserve %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(e));
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 148;
    configured = true;
  }
  const int per_tile = MODE == kGluBf16 ? BF / 2 : BF;
  const int n_f = (a.N + per_tile - 1) / per_tile, n_t = (a.M + BT - 1) / BT;
  const long long tiles = (long long)n_f * n_t;
  if (tiles > 0x7fffffffLL) return fail(kBadArgument, "gemm_prompt: too many tiles");
  PromptArgs b = a;
  const int cut = b.share != nullptr ? cut_blocks(tiles, (a.K + BK - 1) / BK, n_sms < share_blocks ? n_sms : share_blocks) : 0;
  if (cut == 0) b.share = nullptr;
  const unsigned grid = cut > 0 ? (unsigned)cut : (unsigned)(tiles < n_sms ? tiles : n_sms);
  launch_overlapped(gemm_prompt_kernel<MODE>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, stream, mx, mw, my, b, n_t, n_f);
  return check_launch("gemm_prompt");
}
}  // namespace

// Over how many blocks a product of these sizes is cut along K on a device of n_sms SMs (0: whole tiles).
extern "C" int skyla_gemm_prompt_cut_blocks(int M, int N, int K, int gated, int n_sms) {
  const long long n_f = (N + (gated ? BF / 2 : BF) - 1) / (gated ? BF / 2 : BF), n_t = (M + BT - 1) / BT;
  return n_sms > 0 ? cut_blocks(n_f * n_t, (K + BK - 1) / BK, n_sms) : 0;
}

// How many shares of a row's sum of squares the "norm ahead" of a product with N outputs leaves.
extern "C" int skyla_gemm_prompt_ahead_parts(int N) { return (N + BF - 1) / BF; }

// A tensor map of a float matrix y [rows, cols] (ld elements between rows, a multiple of 4; base on
// 16 bytes) for the accumulate epilogue: boxes of 128 rows x 32 columns, 128-byte swizzle.
extern "C" int skyla_output_map_f32(void* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(kLaunchFailed, "tensor map: the driver does not offer cuTensorMapEncodeTiled");
  if (((uintptr_t)ptr) % 16 || (ld * 4) % 16) return fail(kBadArgument, "tensor map: base or row stride is not a multiple of 16 bytes");
  alignas(64) CUtensorMap m;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 4};
  const cuuint32_t box[2] = {kOutCols, BT};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kLaunchFailed, "tensor map: cuTensorMapEncodeTiled failed with %d", (int)r);
  memcpy(out, &m, sizeof(m));
  return kOk;
}

// map_x: tokens [M, K], map_w: weight [N (2N gated), K], both bfloat16 with boxes of 128 rows x 64.
// map_y (or null; mode 2 without norm-ahead): y as skyla_output_map_f32 describes it; the sums are
//   then added by TMA reduce instead of read, added and written by the threads.
// mode 0..3: y [M, N] (ldy elements between rows) as the mode says.
// mode 4: the weight's rows are nq query heads, nkv key heads, nkv value heads of hd (32, 64, 128 or
//   256) each; y [M, nq * hd] bfloat16 receives the prepared queries, the pools the keys and values;
//   q_norm / k_norm [hd] or null; cos_t / sin_t [positions][hd / 2] or both null (the whole head rotates).
// scale_ssq (or null): the result is multiplied by 1/sqrt(sum_p scale_ssq[p * M + tok] / K + scale_eps).
// share, share_flags (or null): scratch of share_blocks x 128 x 256 floats and as many flags (zero between
//   launches), with which few tiles are cut along K over up to share_blocks blocks.
// ahead_xw (or null; mode 2): also leave bf16(y_new * ahead_w) in ahead_xw [M, N] and each tile's share
//   of the rows' sums of squares in ahead_ssq [skyla_gemm_prompt_ahead_parts(N)][M].
extern "C" int skyla_gemm_prompt(const void* map_x, const void* map_w, const void* map_y, void* y, int64_t ldy, int M, int N, int K, int mode,
                                 int* error_flag, const float* scale_ssq, int scale_parts, float scale_eps,
                                 const float* ahead_w, void* ahead_xw, int64_t ahead_ldxw, float* ahead_ssq,
                                 int nq, int nkv, int hd, const float* q_norm, const float* k_norm, float qk_eps,
                                 const float* cos_t, const float* sin_t, const int32_t* tok_pos, const int32_t* tok_slot,
                                 void* k_pool, void* v_pool, const int32_t* page_table, int max_pages, int page_size,
                                 float* share, int* share_flags, int share_blocks, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || K % 8) return fail(kBadArgument, "gemm_prompt: K=%d must be a positive multiple of 8", K);
  if (mode < 0 || mode > kQkvPrep) return fail(kBadArgument, "gemm_prompt: unknown epilogue %d", mode);
  alignas(64) CUtensorMap mx, mw, my;
  memcpy(&mx, map_x, sizeof(mx));
  memcpy(&mw, map_w, sizeof(mw));
  if (map_y != nullptr) memcpy(&my, map_y, sizeof(my));
  else memcpy(&my, map_x, sizeof(my));  // not used; a valid map all the same
  PromptArgs a{};
  a.y = y; a.ldy = ldy; a.M = M; a.N = N; a.K = K; a.error_flag = error_flag;
  if (share != nullptr && share_flags != nullptr && share_blocks > 1) { a.share = share; a.share_flags = share_flags; }
  const int per16 = (mode == kStoreF32 || mode == kAccumF32) ? 4 : 8;  // elements of y in 16 bytes
  a.vec = ((uintptr_t)y % 16 == 0 && ldy % per16 == 0) ? 1 : 0;
  if (scale_ssq != nullptr) {
    if (scale_parts < 1) return fail(kBadArgument, "gemm_prompt: scale-in without shares");
    a.scale = ScaleIn{scale_ssq, scale_parts, scale_eps, K};
  }
  if (map_y != nullptr) {
    if (mode != kAccumF32 || ahead_xw != nullptr)
      return fail(kBadArgument, "gemm_prompt: a tensor map of y goes with the plain accumulate epilogue only");
    a.y_tma = 1;
  }
  if (ahead_xw != nullptr) {
    if (mode != kAccumF32 || ahead_w == nullptr || ahead_ssq == nullptr)
      return fail(kBadArgument, "gemm_prompt: norm-ahead goes with the accumulate epilogue, a weight and a place for the shares");
    // vectors are used for y, the norm weight and xw alike, or for none of them
    if ((uintptr_t)ahead_xw % 16 || ahead_ldxw % 8 || (uintptr_t)ahead_w % 16) a.vec = 0;
    a.ahead = NormAhead{ahead_w, (__nv_bfloat16*)ahead_xw, ahead_ldxw, ahead_ssq};
  }
  if (mode == kQkvPrep) {
    if (hd != 32 && hd != 64 && hd != 128 && hd != 256)
      return fail(kBadArgument, "gemm_prompt: the q/k/v epilogue takes head sizes 32, 64, 128 and 256, not %d", hd);
    if (nq < 1 || nkv < 0 || (int64_t)(nq + 2 * nkv) * hd != N)
      return fail(kBadArgument, "gemm_prompt: %d + 2 x %d heads of %d are not the %d outputs", nq, nkv, hd, N);
    if ((cos_t == nullptr) != (sin_t == nullptr)) return fail(kBadArgument, "gemm_prompt: cos and sin tables go together");
    if (tok_pos == nullptr || (nkv > 0 && k_pool != nullptr && (v_pool == nullptr || tok_slot == nullptr || page_table == nullptr || page_size < 1)))
      return fail(kBadArgument, "gemm_prompt: the q/k/v epilogue needs positions and, with a cache, slots and a page table");
    if ((uintptr_t)y % 16 || ldy % 8 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)cos_t % 16 || (uintptr_t)sin_t % 16 ||
        (uintptr_t)q_norm % 16 || (uintptr_t)k_norm % 16)
      return fail(kBadArgument, "gemm_prompt: the q/k/v epilogue writes 16-byte vectors: unaligned queries, pools, tables or norm weights");
    a.prep = QkvPrep{nq, nkv, hd, q_norm, k_norm, qk_eps, cos_t, sin_t, tok_pos, tok_slot,
                     (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_table, max_pages, page_size};
  }
  switch (mode) {
    case kStoreBf16: return launch<kStoreBf16>(mx, mw, my, a, share_blocks, stream);
    case kStoreF32: return launch<kStoreF32>(mx, mw, my, a, share_blocks, stream);
    case kAccumF32: return launch<kAccumF32>(mx, mw, my, a, share_blocks, stream);
    case kGluBf16: return launch<kGluBf16>(mx, mw, my, a, share_blocks, stream);
    default: return launch<kQkvPrep>(mx, mw, my, a, share_blocks, stream);
  }
}
