// Tensor-core attention over the paged bfloat16 cache, for prompts and for single
// decoded tokens.  It computes what the plain kernel computes
// (skyla-ref/src/model.rs:149-165): softmax(q.k * scale) over the visible
// positions, times v, with the softmax in 32-bit and online across blocks of keys
// (skyla-shaders/shaders/attention.comp:81-99).
//
// A warp owns a tile of 16 query rows and walks the cache 16 keys at a time:
//   S = Q K^T   mma.sync m16n8k16 (bf16 in, f32 out); K rows come straight from
//               global memory as 16-byte loads into B fragments.  The order of a
//               head's elements inside a 32-wide block is permuted the same way
//               in the Q and the K fragments, which a dot product does not notice.
//   P = exp2(S*scale*log2e - max), running max/sum per row in 32-bit
//   O += P V    P re-packed from the S accumulators as the A operand; V rows also
//               come from global memory as contiguous 16..32-byte pieces, with the
//               output columns permuted so that each thread's piece is contiguous;
//               the permutation is undone when O is written.
// A block stages whole cache pages (64 positions of one key/value head, contiguous
// in the pool) in shared memory with cp.async, several pages deep, with the 16-byte
// chunks of a row swizzled (or the rows padded) so that the fragment reads spread
// over the banks; the warps read their fragments from there, 16 bytes at a time.
//
// Decode: the 16 rows of a tile are the query heads that share a key/value head (grouped-query
// attention), so the cache is read once for all of them, as the reference does with N_REP
// (attention.comp:60-79).  The pages of all (sequence, key/value head) pairs of the step are laid end
// to end and dealt to the CTAs in equal runs (see kPlanInts), so that every CTA reads the same amount
// whatever the lengths are; a CTA's four warps take 16 of a page's 64 positions each and are merged in
// shared memory; the pieces of a pair that different CTAs read are merged, in the order of the
// positions, by the CTA that finishes last (skyla-shaders/shaders/attention_merge.comp:17-41 is the
// reference's merge, a pass of its own).
// Prefill: one CTA per (64 new tokens of one sequence, query head), a warp per 16
// tokens, causal by row.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
typedef __nv_bfloat16 bf16;
constexpr float kLog2e = 1.4426950408889634f;

template <int HD>
struct Shape {
  static constexpr int KB32 = HD / 32;
  static constexpr bool TAIL16 = (HD % 32) == 16;
  static constexpr int NQ = KB32 * 4 + (TAIL16 ? 2 : 0);  // 32-bit registers of a row's fragment
  static constexpr int NV = HD / 16;                      // registers of a thread's piece of a V row
  static constexpr int NT = HD / 8;                       // 8-wide output column tiles
  static_assert(HD % 16 == 0 && HD >= 16, "head size in steps of 16");
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory rows of 128 or 256 bytes are not padded; their 16-byte chunks are
// XOR-swizzled so that the eight threads of a quarter warp hit eight different bank
// groups.  K rows: chunk ^ 4*(row & 1).  V rows: chunk ^ a value that depends on which
// thread of a quad reads the row.  Other head sizes use rows padded by 16 bytes.
template <int HD>
struct Swz {
  static constexpr bool kOn = HD % 64 == 0;
  static constexpr int RS = kOn ? HD : HD + 8;  // row stride in elements
  __device__ static __forceinline__ int k(int row) { return kOn ? ((row & 1) << 2) : 0; }
  __device__ static __forceinline__ int v(int row) {
    const int q = (row >> 1) & 3;  // rows 2t, 2t+1, 8+2t, 9+2t are read by thread t of a quad
    return !kOn ? 0 : (HD == 64 ? 2 * q : ((q & 1) | ((q & 2) << 1)));
  }
};

// A row's fragment: thread t of a quad takes elements 32*kb + 8t .. +7 of each
// 32-wide block (and 4t .. +3 of a trailing 16-wide one).  `x` is the XOR applied
// to the 16-byte chunk index (0 for rows in global memory).
template <int HD>
__device__ __forceinline__ void load_row(const bf16* __restrict__ row, int t, uint32_t (&out)[Shape<HD>::NQ], int x = 0) {
  using S = Shape<HD>;
#pragma unroll
  for (int kb = 0; kb < S::KB32; ++kb) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + 8 * ((4 * kb + t) ^ x));
    out[4 * kb] = v.x; out[4 * kb + 1] = v.y; out[4 * kb + 2] = v.z; out[4 * kb + 3] = v.w;
  }
  if (S::TAIL16) {
    const uint2 v = *reinterpret_cast<const uint2*>(row + 32 * S::KB32 + 4 * t);
    out[4 * S::KB32] = v.x; out[4 * S::KB32 + 1] = v.y;
  }
}
// A thread's piece of a V row: columns g*HD/8 .. (g+1)*HD/8 - 1.
template <int HD>
__device__ __forceinline__ void load_v(const bf16* __restrict__ row, int g, uint32_t (&out)[Shape<HD>::NV], int x = 0) {
  constexpr int NV = Shape<HD>::NV;
  if (NV % 4 == 0) {
#pragma unroll
    for (int i = 0; i < NV / 4; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(row + 8 * ((g * (NV / 4) + i) ^ x));
      out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
  } else if (NV % 2 == 0) {
    const bf16* p = row + g * (HD / 8);
#pragma unroll
    for (int i = 0; i < NV / 2; ++i) {
      const uint2 v = reinterpret_cast<const uint2*>(p)[i];
      out[2 * i] = v.x; out[2 * i + 1] = v.y;
    }
  } else {
    const bf16* p = row + g * (HD / 8);
#pragma unroll
    for (int i = 0; i < NV; ++i) out[i] = reinterpret_cast<const uint32_t*>(p)[i];
  }
}

template <int HD>
struct RowState {
  float m[2], l[2];                 // running maximum (log2 units) and this thread's share of the sum
  float o[Shape<HD>::NT][4];        // output accumulators, columns permuted
  __device__ __forceinline__ void init() {
    m[0] = m[1] = -INFINITY; l[0] = l[1] = 0.f;
#pragma unroll
    for (int n = 0; n < Shape<HD>::NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  }
};

// 16 keys starting at absolute position key0; k16/v16 point at their rows for one
// key/value head, staged in shared memory.  Rows g and g+8 of the tile see positions lo..hi.
// MASKED = false: every row sees all 16 keys (the caller has checked), so no position is compared.
template <int HD, bool MASKED = true>
__device__ __forceinline__ void attend16(const uint32_t (&qa)[Shape<HD>::NQ], const uint32_t (&qb)[Shape<HD>::NQ],
                                         const bf16* __restrict__ k16, const bf16* __restrict__ v16, int key0,
                                         int lo0, int hi0, int lo1, int hi1, float scale_log2, RowState<HD>& st,
                                         int g, int t) {
  using S = Shape<HD>;
  uint32_t kf[2][S::NQ], vf[4][S::NV];
  constexpr int RS = Swz<HD>::RS;  // k16/v16 are staged rows in shared memory
  load_row<HD>(k16 + (size_t)g * RS, t, kf[0], Swz<HD>::k(g));
  load_row<HD>(k16 + (size_t)(8 + g) * RS, t, kf[1], Swz<HD>::k(8 + g));
  load_v<HD>(v16 + (size_t)(2 * t) * RS, g, vf[0], Swz<HD>::v(2 * t));
  load_v<HD>(v16 + (size_t)(2 * t + 1) * RS, g, vf[1], Swz<HD>::v(2 * t + 1));
  load_v<HD>(v16 + (size_t)(8 + 2 * t) * RS, g, vf[2], Swz<HD>::v(8 + 2 * t));
  load_v<HD>(v16 + (size_t)(8 + 2 * t + 1) * RS, g, vf[3], Swz<HD>::v(8 + 2 * t + 1));

  float s[2][4];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kb = 0; kb < S::KB32; ++kb) {
      mma_bf16(s[j], qa[4 * kb], qb[4 * kb], qa[4 * kb + 1], qb[4 * kb + 1], kf[j][4 * kb], kf[j][4 * kb + 1]);
      mma_bf16(s[j], qa[4 * kb + 2], qb[4 * kb + 2], qa[4 * kb + 3], qb[4 * kb + 3], kf[j][4 * kb + 2], kf[j][4 * kb + 3]);
    }
    if (S::TAIL16)
      mma_bf16(s[j], qa[4 * S::KB32], qb[4 * S::KB32], qa[4 * S::KB32 + 1], qb[4 * S::KB32 + 1],
               kf[j][4 * S::KB32], kf[j][4 * S::KB32 + 1]);
  }
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (MASKED) {
      const int p = key0 + 8 * j + 2 * t;
      s[j][0] = (p >= lo0 && p <= hi0) ? s[j][0] * scale_log2 : -INFINITY;
      s[j][1] = (p + 1 >= lo0 && p + 1 <= hi0) ? s[j][1] * scale_log2 : -INFINITY;
      s[j][2] = (p >= lo1 && p <= hi1) ? s[j][2] * scale_log2 : -INFINITY;
      s[j][3] = (p + 1 >= lo1 && p + 1 <= hi1) ? s[j][3] * scale_log2 : -INFINITY;
    } else {
      s[j][0] *= scale_log2; s[j][1] *= scale_log2; s[j][2] *= scale_log2; s[j][3] *= scale_log2;
    }
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
  const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
  const float al0 = exp2f(st.m[0] - ref0), al1 = exp2f(st.m[1] - ref1);
  st.m[0] = mn0; st.m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    s[j][0] = exp2f(s[j][0] - ref0); s[j][1] = exp2f(s[j][1] - ref0);
    s[j][2] = exp2f(s[j][2] - ref1); s[j][3] = exp2f(s[j][3] - ref1);
    sum0 += s[j][0] + s[j][1];
    sum1 += s[j][2] + s[j][3];
  }
  st.l[0] = st.l[0] * al0 + sum0;
  st.l[1] = st.l[1] * al1 + sum1;
  const uint32_t a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
  const uint32_t a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
  // the running maxima rarely move once a few hundred keys are in: then every factor is exactly 1
  // and the accumulators need no rescaling (the same bits either way; uniform for the warp)
  if (__any_sync(0xffffffffu, (al0 != 1.f) | (al1 != 1.f))) {
#pragma unroll
    for (int n = 0; n < S::NT; ++n) {
      st.o[n][0] *= al0; st.o[n][1] *= al0; st.o[n][2] *= al1; st.o[n][3] *= al1;
    }
  }
#pragma unroll
  for (int n = 0; n < S::NT; ++n) {
    const uint32_t sel = (n & 1) ? 0x7632u : 0x5410u;
    const uint32_t b0 = __byte_perm(vf[0][n >> 1], vf[1][n >> 1], sel);
    const uint32_t b1 = __byte_perm(vf[2][n >> 1], vf[3][n >> 1], sel);
    mma_bf16(st.o[n], a0, a1, a2, a3, b0, b1);
  }
}

// Accumulator (n, i) of thread (g, t) holds row g + 8*(i>>1), column:
template <int HD>
__device__ __forceinline__ int out_col(int n, int i, int t) { return (2 * t + (i & 1)) * (HD / 8) + n; }

// A thread's accumulators of one row are HD/4 consecutive columns starting at t*HD/4: as float4
// "units" they are stored to shared memory with the unit index XOR-swizzled (head sizes 64 and
// 128), so that the eight lanes of a quarter warp -- two rows, four t -- hit eight bank groups.
template <int HD>
__device__ __forceinline__ int out_unit_xor(int row, int t) {
  return !Swz<HD>::kOn ? 0 : (HD == 128 ? t + 4 * (row & 1) : (t >> 1) + 2 * (row & 1));
}
// Position of column c of row r in a staged [16][HD] float tile.
template <int HD>
__device__ __forceinline__ int staged_index(int r, int c) {
  const int t = c / (HD / 4);
  return r * HD + 4 * ((c >> 2) ^ out_unit_xor<HD>(r, t)) + (c & 3);
}
// Store rows g (half 0) and g+8 (half 1) of the accumulators, scaled, into a staged tile.
template <int HD>
__device__ __forceinline__ void stage_rows(float* tile, const float (&o)[Shape<HD>::NT][4], int g, int t,
                                           bool row0, bool row1, float s0, float s1) {
  constexpr int NT = Shape<HD>::NT;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (!(half ? row1 : row0)) continue;
    const int r = g + 8 * half;
    const float sc = half ? s1 : s0;
#pragma unroll
    for (int b = 0; b < 2; ++b)       // columns (2t+b)*NT + n
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        const int c = (2 * t + b) * NT + n;
        if (NT % 4 == 0) {
          if (n % 4 == 0)
            *reinterpret_cast<float4*>(tile + staged_index<HD>(r, c)) =
                make_float4(o[n][2 * half + b] * sc, o[n + 1][2 * half + b] * sc, o[n + 2][2 * half + b] * sc,
                            o[n + 3][2 * half + b] * sc);
        } else {
          tile[staged_index<HD>(r, c)] = o[n][2 * half + b] * sc;
          tile[staged_index<HD>(r, c + 1)] = o[n + 1][2 * half + b] * sc;
        }
      }
  }
}
// The same rows straight to global memory as bfloat16 (row pointers at column 0 of the head).
template <int HD>
__device__ __forceinline__ void store_rows_bf16(bf16* p0, bf16* p1, const float (&o)[Shape<HD>::NT][4], int t,
                                                float s0, float s1) {
  constexpr int NT = Shape<HD>::NT;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    bf16* p = half ? p1 : p0;
    if (p == nullptr) continue;
    const float sc = half ? s1 : s0;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      bf16* q = p + (2 * t + b) * NT;
      if (NT % 8 == 0) {
#pragma unroll
        for (int n = 0; n < NT; n += 8) {
          uint4 v;
          v.x = pack_bf16(o[n][2 * half + b] * sc, o[n + 1][2 * half + b] * sc);
          v.y = pack_bf16(o[n + 2][2 * half + b] * sc, o[n + 3][2 * half + b] * sc);
          v.z = pack_bf16(o[n + 4][2 * half + b] * sc, o[n + 5][2 * half + b] * sc);
          v.w = pack_bf16(o[n + 6][2 * half + b] * sc, o[n + 7][2 * half + b] * sc);
          *reinterpret_cast<uint4*>(q + n) = v;
        }
      } else {
#pragma unroll
        for (int n = 0; n < NT; n += 2)
          *reinterpret_cast<uint32_t*>(q + n) = pack_bf16(o[n][2 * half + b] * sc, o[n + 1][2 * half + b] * sc);
      }
    }
  }
}

struct PagedKV {
  const bf16* k; const bf16* v; const int32_t* pages; int max_pages, page_size, nkv;
};

// ---- staging of cache pages in shared memory
constexpr int kPage = 64;     // positions per staged page: the cache's page size
template <int HD>
struct Stage {
  static constexpr int RS = Swz<HD>::RS;
  static constexpr int kElems = 2 * kPage * RS;        // K page then V page
  static constexpr int kPageBytes = kElems * (int)sizeof(bf16);
  // decode: four warps work on one page at a time; two blocks share an SM, so that one block's
  // start and end (no loads in flight) hide behind the other's loop: as many pages as about
  // 96 KB hold (3..6)
  static constexpr int kDecodeRaw = (96 * 1024) / kPageBytes;
  static constexpr int kDecodeStages = kDecodeRaw >= 6 ? 6 : (kDecodeRaw < 3 ? 3 : kDecodeRaw);
  // prefill: bound by latency on the compute side, so warps count: two pages deep leaves room for
  // three blocks (twelve warps, all the registers) per SM; 211 against 226 us for 2048 tokens
  static constexpr int kPrefillStages = 2;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NT threads (tid 0..NT-1) copy one page (64 rows of HD elements, contiguous in the pool) of K and of V.
template <int HD, int NT>
__device__ __forceinline__ void stage_page(bf16* stage, const bf16* __restrict__ kg, const bf16* __restrict__ vg, int tid) {
  constexpr int RS = Stage<HD>::RS, CPR = HD / 8;  // 16-byte chunks per row
  bf16* sk = stage;
  bf16* sv = stage + kPage * RS;
  for (int c = tid; c < kPage * CPR; c += NT) {
    const int row = c / CPR, chunk = c % CPR;
    cp_async16(sk + row * RS + 8 * (chunk ^ Swz<HD>::k(row)), kg + row * HD + 8 * chunk);
    cp_async16(sv + row * RS + 8 * (chunk ^ Swz<HD>::v(row)), vg + row * HD + 8 * chunk);
  }
}

// ------------------------------------------------------------------------ decode
// The new token's q, k and v made inside the decode kernel instead of by a kernel before it:
// `qkv` holds the rows [tokens][ld] of the QKV product in 32-bit; every
// block finishes the q heads of its group (row scalar, per-head RMSNorm, rotation), and the
// block whose pages end at the token's own position also finishes k and v, writes them to
// the cache and patches them into the page it has staged.
struct FusedPrep {
  const float* qkv; int64_t ld; int q_off, k_off, v_off;
  const float* q_norm; const float* k_norm; float eps; const float* cos_t; const float* sin_t; int n_rot;
  bf16* k_pool; bf16* v_pool; int n_tokens;
};

// How a decode step's pages are dealt to the blocks.  The items of a step are its (sequence, key/value
// head) pairs, item = sequence * nkv + head, each with the pages of its sequence that the window still
// sees.  A block takes a run of consecutive pages of consecutive items: a run may end one item and begin
// the next.  Row j of the plan says where block j starts: (sequence, head, page of that item, pages of the
// run, position of that sequence's new token, first block and number of pieces of that item, 0).  After
// the rows the plan holds (first block, pieces) of every item: the blocks that read one item are
// consecutive.  Who cuts the runs is free in how: a host that knows the positions may give every item
// equal pieces, or lay all pages end to end and cut them evenly (attn_decode_plan_kernel does the
// latter); the kernel only follows the rows.
// The piece of an item that block j reads has the slot j + item for its partial result, which no other
// piece has (from one piece to the next, j or the item grows); the pieces of one item lie in consecutive
// slots.
constexpr int kPlanInts = 8;

struct DecodeArgs {
  const bf16* q; int64_t ldq; float* part;
  int nq, nkv; PagedKV kv; const int32_t* tok_pos; float scale; int window;
  FusedPrep prep;  // prep.qkv == nullptr: q comes prepared in `q`, k and v are in the cache
  const int32_t* plan;   // [blocks][kPlanInts]
  const int32_t* items;  // [items][2]: first block, pieces
  // if set: the part of an item that finishes last merges the parts itself and writes the heads' rows
  // here (an item that is one part is written straight away); else every part leaves its partial result,
  // `meta` gets (first slot, parts) of every item, and attn_merge_kernel follows in a launch of its own
  bf16* out; int64_t ldo;
  // one zeroed counter per item for "who finishes last"; the last arriver puts it back to
  // zero.  They belong to whoever launches (an engine's kernel state): launches that share them must not
  // overlap on the device
  int* counters;
  int32_t* meta;
};

constexpr int kDecodeWarps = 4;

template <int HD>
__global__ void __launch_bounds__(kDecodeWarps * 32, 2) attn_decode_kernel(DecodeArgs a) {
  using S = Shape<HD>;
  constexpr int RS = Stage<HD>::RS, kStages = Stage<HD>::kDecodeStages, NW = kDecodeWarps;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* stages = reinterpret_cast<bf16*>(smem_raw);
  float* smem = reinterpret_cast<float*>(smem_raw);  // after the loop: [NW][16 rows][HD], [NW][16] m, [NW][16] l
  __shared__ int merges;
  allow_dependents();
  // What the kernel before this one wrote: the unfinished q, k, v (fused) or q and the new
  // token's row of the cache (not fused).  Positions, page lists, the plan and the pages of earlier
  // tokens are older than that, so the fused kernel starts fetching pages right away.
  const bool fused = a.prep.qkv != nullptr;
  bool waited = !fused;
  if (!fused) grid_dependency_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int G = a.nq / a.nkv;
  const int4 row0v = reinterpret_cast<const int4*>(a.plan)[2 * blockIdx.x];
  const int4 row1v = reinterpret_cast<const int4*>(a.plan)[2 * blockIdx.x + 1];
  int b = row0v.x, kvh = row0v.y, page0 = row0v.z, left = row0v.w;
  int pos = row1v.x, j_first = row1v.y, n_parts = row1v.z;
  const float scale_log2 = a.scale * kLog2e;
  // after the page stages: [G+2][HD] bf16 finished heads (q heads, then k, then v), [NW][HD] float scratch
  bf16* fresh = stages + (size_t)kStages * Stage<HD>::kElems;
  constexpr int kAhead = kStages - 1;

  while (left > 0) {  // one piece after the other
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int item_pages = pos / kPage + 1 - first / kPage;
    const int n_pages = min(left, item_pages - page0);
    const int page_begin = first / kPage + page0;
    const int32_t* seq_pages = a.kv.pages + (int64_t)b * a.kv.max_pages;

    auto issue = [&](int i) {
      if (i < n_pages) {
        const size_t row0 = ((size_t)seq_pages[page_begin + i] * a.kv.nkv + kvh) * kPage;
        stage_page<HD, NW * 32>(stages + (size_t)(i % kStages) * Stage<HD>::kElems, a.kv.k + row0 * HD, a.kv.v + row0 * HD,
                                threadIdx.x);
      }
      cp_async_commit();  // an empty group keeps the count the same for every thread
    };
#pragma unroll
    for (int i = 0; i < kAhead; ++i) issue(i);
    if (!waited) {
      grid_dependency_wait();
      waited = true;
    }

    uint32_t qa[S::NQ], qb[S::NQ];
#pragma unroll
    for (int i = 0; i < S::NQ; ++i) qa[i] = qb[i] = 0u;
    const bool owner = fused && page0 + n_pages == item_pages;  // this part ends at the new token
    if (fused) {
      float* uu = reinterpret_cast<float*>(fresh + (size_t)(G + 2) * HD) + (size_t)warp * HD;
      const FusedPrep& p = a.prep;
      for (int job = warp; job < G + 2; job += NW) {  // q heads of the group, then k, then v
        if (job >= G && !owner) continue;
        const bool is_q = job < G, is_k = job == G;
        const float* src = p.qkv + (int64_t)b * p.ld +
                           (is_q ? p.q_off + (kvh * G + job) * HD : (is_k ? p.k_off : p.v_off) + kvh * HD);
        float ss = 0.f;
        for (int e = lane; e < HD; e += 32) {
          const float v = src[e];
          uu[e] = v;
          ss = fmaf(v, v, ss);
        }
        const float* nw = is_q ? p.q_norm : (is_k ? p.k_norm : nullptr);
        if (nw != nullptr) {
          ss = warp_sum(ss);
          const float inv = 1.0f / sqrtf(ss / (float)HD + p.eps);
          for (int e = lane; e < HD; e += 32) uu[e] *= inv * nw[e];
        }
        __syncwarp();
        const int half = p.n_rot / 2;
        bf16* dst = fresh + (size_t)job * HD;
        for (int e = lane; e < HD; e += 32) {
          float v = uu[e];
          if ((is_q || is_k) && p.cos_t != nullptr && e < p.n_rot) {
            const int i = e < half ? e : e - half;
            const float c = p.cos_t[(int64_t)pos * half + i], sn = p.sin_t[(int64_t)pos * half + i];
            const float x0 = uu[i], x1 = uu[i + half];
            v = e < half ? x0 * c - x1 * sn : x0 * sn + x1 * c;
          }
          dst[e] = __float2bfloat16_rn(v);
        }
        __syncwarp();
        if (!is_q) {  // the token's place in the cache, for the steps to come
          const size_t row = ((size_t)seq_pages[pos / kPage] * a.kv.nkv + kvh) * kPage + pos % kPage;
          bf16* pool = is_k ? p.k_pool : p.v_pool;
          for (int e = lane; e < HD; e += 32) pool[row * HD + e] = dst[e];
        }
      }
      __syncthreads();
      if (g < G) load_row<HD>(fresh + (size_t)g * HD, t, qa);
      if (g + 8 < G) load_row<HD>(fresh + (size_t)(g + 8) * HD, t, qb);
    } else {
      const bf16* qrow = a.q + (int64_t)b * a.ldq + (int64_t)kvh * G * HD;
      if (g < G) load_row<HD>(qrow + g * HD, t, qa);
      if (g + 8 < G) load_row<HD>(qrow + (g + 8) * HD, t, qb);
    }
    const int hi0 = g < G ? pos : -1, hi1 = g + 8 < G ? pos : -1;

    RowState<HD> st;
    st.init();
    for (int pg = 0; pg < n_pages; ++pg) {
      issue(pg + kAhead);  // into the stage that the round before this one read
      cp_async_wait<kAhead>();
      __syncthreads();
      if (owner && pg == n_pages - 1) {
        // the staged copy of the token's page was read before k and v were written: put them in
        bf16* page = stages + (size_t)(pg % kStages) * Stage<HD>::kElems;
        const int r = pos % kPage;
        for (int c = threadIdx.x; c < 2 * (HD / 8); c += NW * 32) {
          const bool is_v = c >= HD / 8;
          const int chunk = is_v ? c - HD / 8 : c;
          const int x = is_v ? Swz<HD>::v(r) : Swz<HD>::k(r);
          *reinterpret_cast<uint4*>(page + (is_v ? kPage * RS : 0) + r * RS + 8 * (chunk ^ x)) =
              *reinterpret_cast<const uint4*>(fresh + (size_t)(G + (is_v ? 1 : 0)) * HD + 8 * chunk);
        }
        __syncthreads();
      }
      const bf16* sk = stages + (size_t)(pg % kStages) * Stage<HD>::kElems;
      const int key0 = (page_begin + pg) * kPage + 16 * warp;  // this warp's 16 positions
      if (key0 + 15 <= pos && key0 >= first)  // all 16 keys are visible: nothing to mask
        attend16<HD, false>(qa, qb, sk + 16 * warp * RS, sk + (kPage + 16 * warp) * RS, key0, first, hi0, first, hi1,
                            scale_log2, st, g, t);
      else if (key0 <= pos && key0 + 15 >= first)
        attend16<HD>(qa, qb, sk + 16 * warp * RS, sk + (kPage + 16 * warp) * RS, key0, first, hi0, first, hi1,
                     scale_log2, st, g, t);
      __syncthreads();  // the stage is refilled in the next round
    }
    cp_async_wait<0>();
    __syncthreads();
    // this thread's shares of the row sums -> whole rows
    st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 1); st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 2);
    st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 1); st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 2);

    float* so = smem + (size_t)warp * 16 * HD;
    float* sm = smem + (size_t)NW * 16 * HD + warp * 16;
    float* sl = sm + NW * 16;
    stage_rows<HD>(so, st.o, g, t, g < G, g + 8 < G, 1.f, 1.f);
    if (t == 0) { sm[g] = st.m[0]; sm[g + 8] = st.m[1]; sl[g] = st.l[0]; sl[g + 8] = st.l[1]; }
    __syncthreads();

    const int item = b * a.nkv + kvh;
    const bool alone = n_parts == 1 && a.out != nullptr;
    // merge the warps in fixed order, two columns of a head per thread
    const float* am = smem + (size_t)NW * 16 * HD;
    const float* al = am + NW * 16;
    float* mine = a.part + (size_t)(blockIdx.x + item) * G * (HD + 2);
    for (int idx = threadIdx.x; idx < G * (HD / 2); idx += NW * 32) {
      const int r = idx / (HD / 2), c = 2 * (idx % (HD / 2));
      float M = -INFINITY;
      for (int w = 0; w < NW; ++w) M = fmaxf(M, am[w * 16 + r]);
      const float ref = M == -INFINITY ? 0.f : M;
      float acc0 = 0.f, acc1 = 0.f, L = 0.f;
      for (int w = 0; w < NW; ++w) {
        const float f = exp2f(am[w * 16 + r] - ref);
        const float2 o = *reinterpret_cast<const float2*>(smem + (size_t)w * 16 * HD + staged_index<HD>(r, c));
        acc0 += f * o.x;
        acc1 += f * o.y;
        L += f * al[w * 16 + r];
      }
      if (alone) {  // the whole item: its heads' rows are final
        *reinterpret_cast<__nv_bfloat162*>(a.out + (int64_t)b * a.ldo + (int64_t)(kvh * G + r) * HD + c) =
            __floats2bfloat162_rn(acc0 / L, acc1 / L);
      } else {      // one partial per (slot, head): m, l, acc[HD]
        float* out = mine + (size_t)r * (HD + 2);
        *reinterpret_cast<float2*>(out + 2 + c) = make_float2(acc0, acc1);
        if (c == 0) { out[0] = M; out[1] = L; }
      }
    }
    if (a.out == nullptr) {
      if (page0 == 0 && threadIdx.x == 0) { a.meta[2 * item] = j_first + item; a.meta[2 * item + 1] = n_parts; }
    } else if (!alone) {
      // who finishes last of this item merges its parts, in the order of the parts
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        int* counter = &a.counters[item];
        const int before = atomicAdd(counter, 1);
        merges = before == n_parts - 1;
        if (merges) *counter = 0;  // all are in: ready for the next launch
      }
      __syncthreads();
      if (merges) {
        __threadfence();
        // Every partial is a round trip to the L2, so a thread asks for all of its own at once: two
        // columns of one head, eight parts at a time, folded into the running (maximum, sum, row) in
        // the order of the parts.
        const float* base = a.part + (size_t)(j_first + item) * G * (HD + 2);
        const size_t stride = (size_t)G * (HD + 2);
        for (int idx = threadIdx.x; idx < G * (HD / 2); idx += NW * 32) {
          const int r = idx / (HD / 2), c = 2 * (idx % (HD / 2)), h = kvh * G + r;
          const float* p = base + (size_t)r * (HD + 2);
          float M = -INFINITY, total = 0.f, o0 = 0.f, o1 = 0.f;
          for (int s0 = 0; s0 < n_parts; s0 += 8) {
            float m8[8], l8[8];
            float2 o8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const bool in = s0 + j < n_parts;
              const float* ps = p + (size_t)(s0 + j) * stride;
              const float2 ml = in ? __ldcg(reinterpret_cast<const float2*>(ps)) : make_float2(-INFINITY, 0.f);
              m8[j] = ml.x;
              l8[j] = ml.y;
              o8[j] = in ? __ldcg(reinterpret_cast<const float2*>(ps + 2 + c)) : make_float2(0.f, 0.f);
            }
            float Mn = M;
#pragma unroll
            for (int j = 0; j < 8; ++j) Mn = fmaxf(Mn, m8[j]);
            if (Mn == -INFINITY) continue;
            const float keep = exp2f(M - Mn);  // 0 for the first chunk (M is -inf)
            total *= keep;
            o0 *= keep;
            o1 *= keep;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float f = exp2f(m8[j] - Mn);
              total += f * l8[j];
              o0 += f * o8[j].x;
              o1 += f * o8[j].y;
            }
            M = Mn;
          }
          *reinterpret_cast<__nv_bfloat162*>(a.out + (int64_t)b * a.ldo + (int64_t)h * HD + c) =
              __floats2bfloat162_rn(o0 / total, o1 / total);
        }
      }
    }
    // the next part of this block: the next head of the sequence, or the next sequence's first
    left -= n_pages;
    page0 = 0;
    if (++kvh == a.nkv) { kvh = 0; ++b; }
    if (left > 0) {
      pos = a.tok_pos[b];
      const int2 info = reinterpret_cast<const int2*>(a.items)[b * a.nkv + kvh];
      j_first = info.x;
      n_parts = info.y;
    }
    __syncthreads();  // the staged rows are read; the stages are free for the next part's pages
  }
}

struct MergeArgs { const float* part; const int32_t* meta; bf16* out; int64_t ldo; int nq, nkv, hd; };

__global__ void __launch_bounds__(128) attn_merge_kernel(MergeArgs a) {
  allow_dependents();
  grid_dependency_wait();
  const int h = blockIdx.x, b = blockIdx.y, G = a.nq / a.nkv, item = b * a.nkv + h / G;
  const int n_parts = a.meta[2 * item + 1];
  const size_t stride = (size_t)G * (a.hd + 2);
  const float* p = a.part + ((size_t)a.meta[2 * item] * G + h % G) * (a.hd + 2);
  float M = -INFINITY;
  for (int s = 0; s < n_parts; ++s) M = fmaxf(M, p[s * stride]);
  float total = 0.f;
  for (int s = 0; s < n_parts; ++s) total += exp2f(p[s * stride] - M) * p[s * stride + 1];
  for (int c = threadIdx.x; c < a.hd; c += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_parts; ++s) o += exp2f(p[s * stride] - M) * p[s * stride + 2 + c];
    a.out[(int64_t)b * a.ldo + (int64_t)h * a.hd + c] = __float2bfloat16_rn(o / total);
  }
}

// The plan of a decode step (see kPlanInts) from the positions of its new tokens: all pages laid end to
// end, T in all, and block j gets the run [j * per, (j+1) * per), per = ceil(T / blocks).  One block.
struct PlanArgs { const int32_t* tok_pos; int n_seqs, nkv, window, n_blocks; int32_t* plan; };

__global__ void __launch_bounds__(256) attn_decode_plan_kernel(PlanArgs a) {
  __shared__ long long warp_sum_s[8];
  __shared__ long long carry_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int32_t* table = a.plan + (size_t)a.n_blocks * kPlanInts;
  auto pages_of = [&](int b) -> long long {
    if (b >= a.n_seqs) return 0;
    const int pos = a.tok_pos[b];
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    return pos / kPage + 1 - first / kPage;
  };
  // all pages
  long long mine = 0;
  for (int b = tid; b < a.n_seqs; b += 256) mine += pages_of(b);
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if (lane == 0) warp_sum_s[warp] = mine;
  __syncthreads();
  long long total = 0;
  for (int w = 0; w < 8; ++w) total += warp_sum_s[w];
  total *= a.nkv;
  const long long per = max(1LL, (total + a.n_blocks - 1) / a.n_blocks);
  if (tid == 0) carry_s = 0;
  __syncthreads();
  // every sequence writes its items' lines of the table and the rows of the blocks that start inside it
  for (int base = 0; base < a.n_seqs; base += 256) {
    const int b = base + tid;
    const long long n = pages_of(b);
    long long incl = n;
    for (int o = 1; o < 32; o <<= 1) {
      const long long v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    __syncthreads();  // warp_sum_s and carry_s of the round before are read
    if (lane == 31) warp_sum_s[warp] = incl;
    __syncthreads();
    long long before = carry_s;
    for (int w = 0; w < warp; ++w) before += warp_sum_s[w];
    const long long lo = (before + incl - n) * a.nkv, hi = lo + n * a.nkv;
    if (b < a.n_seqs && n > 0) {
      const int pos = a.tok_pos[b];
      for (int h = 0; h < a.nkv; ++h) {
        const long long item_lo = lo + h * n, jf = item_lo / per;
        table[2 * (b * a.nkv + h)] = (int)jf;
        table[2 * (b * a.nkv + h) + 1] = (int)((item_lo + n - 1) / per - jf + 1);
      }
      for (long long j = (lo + per - 1) / per; j * per < hi && j < a.n_blocks; ++j) {
        const long long r = j * per - lo, h = r / n, item_lo = lo + h * n, jf = item_lo / per;
        int32_t* row = a.plan + j * kPlanInts;
        row[0] = b; row[1] = (int)h; row[2] = (int)(r % n); row[3] = (int)min(per, total - j * per);
        row[4] = pos; row[5] = (int)jf; row[6] = (int)((item_lo + n - 1) / per - jf + 1); row[7] = 0;
      }
    }
    __syncthreads();
    if (tid == 255) carry_s = before + incl;
  }
  __syncthreads();
  for (long long j = (total + per - 1) / per + tid; j < a.n_blocks; j += 256) {  // blocks that get nothing
    int32_t* row = a.plan + j * kPlanInts;
    for (int i = 0; i < kPlanInts; ++i) row[i] = 0;
  }
}

// ----------------------------------------------------------------------- prefill
struct PrefillArgs {
  const bf16* q; int64_t ldq; bf16* out; int64_t ldo;
  int nq, nkv; PagedKV kv; const int32_t* tok_pos; const int32_t* tile_seq; const int32_t* tile_tok0;
  const int32_t* tile_rows; float scale; int window;
};

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(PrefillArgs a) {
  using S = Shape<HD>;
  constexpr int RS = Stage<HD>::RS, kStages = Stage<HD>::kPrefillStages;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* stages = reinterpret_cast<bf16*>(smem_raw);
  allow_dependents();
  grid_dependency_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // a sequence's later tiles see more keys: they go first, so that the short ones fill the end; blocks
  // start in the order of their numbers, so the heads are the fast index: all heads of the longest tile first
  const int tile = (int)(gridDim.x / a.nq) - 1 - (int)(blockIdx.x / a.nq), h = (int)(blockIdx.x % a.nq), kvh = h / (a.nq / a.nkv);
  const int b = a.tile_seq[tile], tok0 = a.tile_tok0[tile], rows = a.tile_rows[tile];
  // the tile's rows are consecutive positions of one sequence
  const int pos_first = a.tok_pos[tok0], pos_last = pos_first + rows - 1;
  const int tile_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int page_begin = tile_lo / kPage, n_pages = pos_last / kPage + 1 - page_begin;
  const int32_t* seq_pages = a.kv.pages + (int64_t)b * a.kv.max_pages;

  auto issue = [&](int i) {
    if (i < n_pages) {
      const size_t row0 = ((size_t)seq_pages[page_begin + i] * a.kv.nkv + kvh) * kPage;
      stage_page<HD, 128>(stages + (size_t)(i % kStages) * Stage<HD>::kElems, a.kv.k + row0 * HD, a.kv.v + row0 * HD,
                          threadIdx.x);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue(i);

  const int r0 = warp * 16 + g, r1 = r0 + 8;
  uint32_t qa[S::NQ], qb[S::NQ];
#pragma unroll
  for (int i = 0; i < S::NQ; ++i) qa[i] = qb[i] = 0u;
  // rows that do not exist see nothing: lo > hi
  int hi0 = 0, hi1 = 0, lo0 = 1, lo1 = 1;
  if (r0 < rows) {
    hi0 = pos_first + r0;
    lo0 = a.window > 0 ? max(0, hi0 - a.window + 1) : 0;
    load_row<HD>(a.q + (int64_t)(tok0 + r0) * a.ldq + (int64_t)h * HD, t, qa);
  }
  if (r1 < rows) {
    hi1 = pos_first + r1;
    lo1 = a.window > 0 ? max(0, hi1 - a.window + 1) : 0;
    load_row<HD>(a.q + (int64_t)(tok0 + r1) * a.ldq + (int64_t)h * HD, t, qb);
  }
  // what any row of this warp sees: the same in all lanes, so the warp stays converged for mma.sync
  const bool warp_live = warp * 16 < rows;
  const int w_first = pos_first + warp * 16, w_last = min(pos_last, w_first + 15);
  const int wlo = a.window > 0 ? max(0, w_first - a.window + 1) : 0, whi = w_last;
  const int whi_lo = a.window > 0 ? max(0, w_first + 15 - a.window + 1) : 0;  // the lowest key the warp's last row sees
  const float scale_log2 = a.scale * kLog2e;

  RowState<HD> st;
  st.init();
  for (int i = 0; i < n_pages; ++i) {
    issue(i + kStages - 1);
    cp_async_wait<kStages - 1>();
    __syncthreads();
    const bf16* sk = stages + (size_t)(i % kStages) * Stage<HD>::kElems;
    if (warp_live) {
#pragma unroll 1
      for (int off = 0; off < kPage; off += 16) {
        const int key0 = (page_begin + i) * kPage + off;
        if (key0 > whi) break;
        if (key0 + 15 < wlo) continue;
        // all 16 keys lie before the warp's first row and inside the window of its last: nothing to mask
        // (rows past the tile's end then compute on zeros; they are never stored)
        if (key0 + 15 <= w_first && key0 >= whi_lo)
          attend16<HD, false>(qa, qb, sk + off * RS, sk + (kPage + off) * RS, key0, lo0, hi0, lo1, hi1, scale_log2, st, g, t);
        else
          attend16<HD>(qa, qb, sk + off * RS, sk + (kPage + off) * RS, key0, lo0, hi0, lo1, hi1, scale_log2, st, g, t);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  if (!warp_live) return;
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 1); st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 2);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 1); st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 2);
  const float inv0 = st.l[0] > 0.f ? 1.f / st.l[0] : 0.f, inv1 = st.l[1] > 0.f ? 1.f / st.l[1] : 0.f;
  // each thread owns HD/4 consecutive columns of its two rows: straight to global memory
  bf16* p0 = r0 < rows ? a.out + (int64_t)(tok0 + r0) * a.ldo + (int64_t)h * HD : nullptr;
  bf16* p1 = r1 < rows ? a.out + (int64_t)(tok0 + r1) * a.ldo + (int64_t)h * HD : nullptr;
  store_rows_bf16<HD>(p0, p1, st.o, t, inv0, inv1);
}

template <int HD>
int launch_decode(const DecodeArgs& a, int n_blocks, cudaStream_t stream) {
  size_t smem = (size_t)(kDecodeWarps * 16 * HD + 2 * kDecodeWarps * 16) * sizeof(float);
  if (smem < (size_t)Stage<HD>::kDecodeStages * Stage<HD>::kPageBytes) smem = (size_t)Stage<HD>::kDecodeStages * Stage<HD>::kPageBytes;
  // after the stages: up to 18 finished heads (bf16) and a float scratch row per warp
  smem += (size_t)18 * HD * sizeof(bf16) + (size_t)kDecodeWarps * HD * sizeof(float);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(kLaunchFailed, "attention_decode: shared memory: %s", cudaGetErrorString(e));
  }
  configured = true;
  launch_overlapped(attn_decode_kernel<HD>, dim3(n_blocks), dim3(kDecodeWarps * 32), smem, stream, a);
  return check_launch("attention_decode");
}
template <int HD>
int launch_prefill(const PrefillArgs& a, int n_tiles, cudaStream_t stream) {
  size_t smem = (size_t)(4 * 16 * HD) * sizeof(float);
  if (smem < (size_t)Stage<HD>::kPrefillStages * Stage<HD>::kPageBytes) smem = (size_t)Stage<HD>::kPrefillStages * Stage<HD>::kPageBytes;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(kLaunchFailed, "attention_prefill: shared memory: %s", cudaGetErrorString(e));
  }
  configured = true;
  launch_overlapped(attn_prefill_kernel<HD>, dim3(n_tiles * a.nq), dim3(128), smem, stream, a);
  return check_launch("attention_prefill");
}

#define SKYLA_HD_SWITCH(hd, CALL)                                                       \
  switch (hd) {                                                                         \
    case 16: { constexpr int HD = 16; CALL; }                                           \
    case 32: { constexpr int HD = 32; CALL; }                                           \
    case 48: { constexpr int HD = 48; CALL; }                                           \
    case 64: { constexpr int HD = 64; CALL; }                                           \
    case 80: { constexpr int HD = 80; CALL; }                                           \
    case 96: { constexpr int HD = 96; CALL; }                                           \
    case 112: { constexpr int HD = 112; CALL; }                                         \
    case 128: { constexpr int HD = 128; CALL; }                                         \
    default: return fail(kBadArgument, "attention_mma: no kernel for head size %d", hd); \
  }

int check_common(const void* q, int64_t ldq, int nq, int nkv, int page_size, const void* k, const void* v) {
  if (nkv <= 0 || nq % nkv) return fail(kBadArgument, "attention_mma: %d query heads over %d key/value heads", nq, nkv);
  if (page_size != kPage) return fail(kBadArgument, "attention_mma: pages of %d positions, the kernels stage pages of %d", page_size, kPage);
  if (((uintptr_t)q) % 16 || (ldq * 2) % 16 || ((uintptr_t)k) % 16 || ((uintptr_t)v) % 16)
    return fail(kBadArgument, "attention_mma: operands must be 16-byte aligned");
  return kOk;
}
}  // namespace

// 1 when the tensor-core kernels take this head size.
extern "C" int skyla_attention_mma_supports(int hd, int group) {
  return (hd % 16 == 0 && hd >= 16 && hd <= 128) ? (group <= 16 ? 2 : 1) : 0;
}

// Floats of scratch that a decode launch of `n_blocks` blocks needs: a partial result per part and head
// (slots 0 .. blocks + items - 1), and two ints per item for the merge kernel.
extern "C" int64_t skyla_attention_decode_scratch_floats(int n_seqs, int nq, int nkv, int hd, int n_blocks) {
  if (n_seqs <= 0 || nkv <= 0) return 0;
  const int64_t items = (int64_t)n_seqs * nkv;
  return (n_blocks + items) * (nq / nkv) * (hd + 2) + 2 * items;
}

// The plan of a decode step, made on the device from the positions of its new tokens (a host that knows
// the positions can write a plan itself): [n_blocks][8] ints of rows, then [n_seqs * nkv][2] ints of items.
extern "C" int skyla_attention_decode_plan(const int32_t* tok_pos, int n_seqs, int nkv, int window, int n_blocks,
                                           int32_t* plan, cudaStream_t stream) {
  if (n_seqs <= 0 || n_blocks <= 0 || nkv <= 0) return fail(kBadArgument, "attention_decode_plan: bad sizes");
  PlanArgs a{tok_pos, n_seqs, nkv, window, n_blocks, plan};
  attn_decode_plan_kernel<<<1, 256, 0, stream>>>(a);
  return check_launch("attention_decode_plan");
}

namespace {
int run_decode(DecodeArgs& a, void* out, int64_t ldo, float* part, int64_t part_floats, int n_seqs, int hd, int max_pages,
               int n_blocks, int* counters, int n_counters, cudaStream_t stream) {
  if (a.nq / a.nkv > 16) return fail(kBadArgument, "attention_decode: groups of %d query heads exceed 16", a.nq / a.nkv);
  if (n_blocks < 1 || a.plan == nullptr) return fail(kBadArgument, "attention_decode: no plan");
  const int64_t items = (int64_t)n_seqs * a.nkv;
  if (items * max_pages >= (1LL << 31)) return fail(kBadArgument, "attention_decode: too many pages to number");
  const int64_t need = skyla_attention_decode_scratch_floats(n_seqs, a.nq, a.nkv, hd, n_blocks);
  if (part == nullptr || part_floats < need)
    return fail(kBadArgument, "attention_decode: %lld floats of scratch needed, %lld given", (long long)need, (long long)part_floats);
  a.part = part;
  a.items = a.plan + (size_t)n_blocks * kPlanInts;
  a.meta = reinterpret_cast<int32_t*>(part + (need - 2 * items));
  const bool merge_inside = counters != nullptr && items <= n_counters;
  a.counters = counters;
  if (merge_inside) { a.out = (bf16*)out; a.ldo = ldo; }
  int rc = kOk;
  SKYLA_HD_SWITCH(hd, { rc = launch_decode<HD>(a, n_blocks, stream); break; });
  if (rc || merge_inside) return rc;
  MergeArgs m{part, a.meta, (bf16*)out, ldo, a.nq, a.nkv, hd};
  launch_overlapped(attn_merge_kernel, dim3(a.nq, n_seqs), dim3(128), 0, stream, m);
  return check_launch("attention_merge");
}
}  // namespace

// Decode: token b of the step is the one new token of sequence b.  `plan` deals the step's pages to
// `n_blocks` blocks (skyla_attention_decode_plan); `part` holds `part_floats` floats of scratch
// (skyla_attention_decode_scratch_floats); out is [n_seqs, nq*hd] bf16.
// `counters`: n_counters zeroed ints that stay the caller's between launches (they are zero again
// when a launch ends); with n_seqs * nkv of them the part that finishes last merges an item's parts
// inside the kernel, with fewer (or none) a merge kernel follows.
extern "C" int skyla_attention_decode(const void* q, int64_t ldq, void* out, int64_t ldo, float* part, int64_t part_floats,
                                      int n_seqs, int nq, int nkv, int hd, const void* k_pool, const void* v_pool,
                                      const int32_t* pages, int max_pages, int page_size, const int32_t* tok_pos,
                                      float scale, int window, const int32_t* plan, int n_blocks, int* counters,
                                      int n_counters, cudaStream_t stream) {
  if (n_seqs <= 0) return kOk;
  int rc = check_common(q, ldq, nq, nkv, page_size, k_pool, v_pool);
  if (rc) return rc;
  DecodeArgs a{(const bf16*)q, ldq, nullptr, nq, nkv,
               PagedKV{(const bf16*)k_pool, (const bf16*)v_pool, pages, max_pages, page_size, nkv}, tok_pos, scale, window,
               FusedPrep{}, plan, nullptr, nullptr, 0, nullptr, nullptr};
  return run_decode(a, out, ldo, part, part_floats, n_seqs, hd, max_pages, n_blocks, counters, n_counters, stream);
}

// Decode with the new token's q, k and v finished inside the kernel: `qkv` are the rows [n_seqs][ld]
// (float) of the QKV product.  k and v of the new token are written to the pools (which this call
// therefore changes).  The plan must be older than the kernel that runs before this one (the kernel
// reads it while that one may still be running): written by the host, or by a kernel the stream has
// been waited for.
extern "C" int skyla_attention_decode_fused(
    const float* qkv, int64_t ld, int q_off, int k_off, int v_off, const float* q_norm, const float* k_norm,
    float eps, const float* cos_t, const float* sin_t, int n_rot, void* out, int64_t ldo, float* part, int64_t part_floats,
    int n_seqs, int nq, int nkv, int hd, void* k_pool, void* v_pool, const int32_t* pages, int max_pages, int page_size,
    const int32_t* tok_pos, float scale, int window, const int32_t* plan, int n_blocks, int* counters, int n_counters,
    cudaStream_t stream) {
  if (n_seqs <= 0) return kOk;
  int rc = check_common(k_pool, 8, nq, nkv, page_size, k_pool, v_pool);
  if (rc) return rc;
  if (qkv == nullptr || n_rot < 0 || n_rot > hd || n_rot % 2)
    return fail(kBadArgument, "attention_decode_fused: bad description of the unfinished q, k and v");
  DecodeArgs a{nullptr, 0, nullptr, nq, nkv,
               PagedKV{(const bf16*)k_pool, (const bf16*)v_pool, pages, max_pages, page_size, nkv}, tok_pos, scale, window,
               FusedPrep{qkv, ld, q_off, k_off, v_off,
                         q_norm, k_norm, eps, cos_t, sin_t, cos_t ? n_rot : 0, (bf16*)k_pool, (bf16*)v_pool, n_seqs},
               plan, nullptr, nullptr, 0, nullptr, nullptr};
  return run_decode(a, out, ldo, part, part_floats, n_seqs, hd, max_pages, n_blocks, counters, n_counters, stream);
}

// Prefill: tiles of up to 64 consecutive new tokens of one sequence.
extern "C" int skyla_attention_prefill(const void* q, int64_t ldq, void* out, int64_t ldo, int n_tiles, int nq, int nkv,
                                       int hd, const void* k_pool, const void* v_pool, const int32_t* pages,
                                       int max_pages, int page_size, const int32_t* tok_pos, const int32_t* tile_seq,
                                       const int32_t* tile_tok0, const int32_t* tile_rows, float scale, int window,
                                       cudaStream_t stream) {
  if (n_tiles <= 0) return kOk;
  int rc = check_common(q, ldq, nq, nkv, page_size, k_pool, v_pool);
  if (rc) return rc;
  if ((int64_t)n_tiles * nq >= (1LL << 31)) return fail(kBadArgument, "attention_prefill: too many tiles");
  PrefillArgs a{(const bf16*)q, ldq, (bf16*)out, ldo, nq, nkv,
                PagedKV{(const bf16*)k_pool, (const bf16*)v_pool, pages, max_pages, page_size, nkv},
                tok_pos, tile_seq, tile_tok0, tile_rows, scale, window};
  SKYLA_HD_SWITCH(hd, { rc = launch_prefill<HD>(a, n_tiles, stream); break; });
  return rc;
}

// ---------------------------------------------------------------- no allocation
#include "attention_no_alloc.h"

// The scratch of the entry point below: part of the library's device image on every
// GPU that loads it.  Host code may not use this name as an address; it asks the
// runtime for the device address once per device (see scratch_address()).
static __device__ __align__(256) float g_no_alloc_scratch[SKYLA_NO_ALLOC_SCRATCH_FLOATS];
// Its "who finishes last" counters, one per (sequence, kv head): the entry point's own, so that it
// shares nothing with an engine that runs on the same device.  They start at zero (the image is
// zero-filled) and every launch leaves them at zero.
static __device__ __align__(256) int g_no_alloc_counters[SKYLA_NO_ALLOC_COUNTERS];
// And the plan of its launch: which pages each block reads.
static __device__ __align__(256) int32_t g_no_alloc_plan[8 * SKYLA_NO_ALLOC_BLOCKS + 2 * SKYLA_NO_ALLOC_ITEMS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {nullptr};
int* g_counters_address[kMaxDevices] = {nullptr};
int32_t* g_plan_address[kMaxDevices] = {nullptr};

// Device addresses of g_no_alloc_scratch, g_no_alloc_counters and g_no_alloc_plan on the current device,
// looked up on first use.
int scratch_address(float** out, int** counters, int32_t** plan) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(kLaunchFailed, "attention_decode_no_alloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(kBadArgument, "attention_decode_no_alloc: device %d is out of range", dev);
  if (g_scratch_address[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(kLaunchFailed, "attention_decode_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    void* c = nullptr;
    e = cudaGetSymbolAddress(&c, g_no_alloc_counters);
    if (e != cudaSuccess || c == nullptr)
      return fail(kLaunchFailed, "attention_decode_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    void* pl = nullptr;
    e = cudaGetSymbolAddress(&pl, g_no_alloc_plan);
    if (e != cudaSuccess || pl == nullptr)
      return fail(kLaunchFailed, "attention_decode_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_plan_address[dev] = static_cast<int32_t*>(pl);
    g_counters_address[dev] = static_cast<int*>(c);
    g_scratch_address[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_address[dev];
  *counters = g_counters_address[dev];
  *plan = g_plan_address[dev];
  return kOk;
}
}  // namespace

extern "C" int skyla_attention_decode_no_alloc(const void* q, int64_t ldq, void* out, int64_t ldo, int n_seqs, int nq,
                                               int nkv, int hd, const void* k_pool, const void* v_pool,
                                               const int32_t* pages, int max_pages, int page_size,
                                               const int32_t* tok_pos, float scale, int window, int n_blocks,
                                               cudaStream_t stream) {
  if (n_seqs <= 0) return kOk;
  if (nq <= 0 || hd <= 0 || nkv <= 0 || nq % nkv || n_blocks <= 0) return fail(kBadArgument, "attention_decode_no_alloc: bad sizes");
  if (n_blocks > SKYLA_NO_ALLOC_BLOCKS)
    return fail(kBadArgument, "attention_decode_no_alloc: %d blocks, the built-in plan holds %d", n_blocks, SKYLA_NO_ALLOC_BLOCKS);
  if ((long long)n_seqs * nkv > SKYLA_NO_ALLOC_ITEMS)
    return fail(kBadArgument, "attention_decode_no_alloc: %d sequences x %d key/value heads, the built-in plan holds %d such pairs",
                n_seqs, nkv, SKYLA_NO_ALLOC_ITEMS);
  const long long need = skyla_attention_decode_scratch_floats(n_seqs, nq, nkv, hd, n_blocks);
  if (need > (long long)SKYLA_NO_ALLOC_SCRATCH_FLOATS)
    return fail(kBadArgument,
                "attention_decode_no_alloc: %lld floats of scratch needed ((%d blocks + %d sequences x %d key/value heads) x "
                "%d heads x %d), the built-in array holds %u; use fewer blocks or skyla_attention_decode with a buffer of "
                "your own", need, n_blocks, n_seqs, nkv, nq / nkv, hd + 2, (unsigned)SKYLA_NO_ALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  int* counters = nullptr;
  int32_t* plan = nullptr;
  int rc = scratch_address(&scratch, &counters, &plan);
  if (rc) return rc;
  rc = skyla_attention_decode_plan(tok_pos, n_seqs, nkv, window, n_blocks, plan, stream);
  if (rc) return rc;
  // more (sequence, kv head) pairs than counters: the parts are merged by a second kernel instead
  return skyla_attention_decode(q, ldq, out, ldo, scratch, SKYLA_NO_ALLOC_SCRATCH_FLOATS, n_seqs, nq, nkv, hd, k_pool,
                                v_pool, pages, max_pages, page_size, tok_pos, scale, window, plan, n_blocks, counters,
                                SKYLA_NO_ALLOC_COUNTERS, stream);
}
