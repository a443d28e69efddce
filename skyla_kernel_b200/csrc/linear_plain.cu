// Plain matrix product y = x W^T for row-major x[M,K] and W[N,K] (rows are
// outputs, as in skyla-ref/src/matrix.rs:38-58).  32-bit FMA accumulation over
// k in ascending order for every output element, whatever M is: the result of a
// row never depends on which other rows share the launch.  This is the matrix
// product of the true 32-bit path and the reference twin of the tensor-core
// kernels.  Epilogues:
//   0  store            y = acc
//   1  accumulate       y += acc            (y is 32-bit: the residual sum,
//                                            skyla-engine/src/graph.rs:110-112)
//   2  gated            y[m,j] = silu(gate_j) * up_j   (skyla-ref/src/ffn.rs:21-28)
//      W holds 2N rows in groups: g gate rows, then the g up rows of the same
//      outputs, and so on; g = N is the plain "gate block, up block" layout.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TY, int MODE>
__global__ void __launch_bounds__(256)
linear_plain_kernel(const TX* __restrict__ x, int64_t ldx, const TW* __restrict__ w, int M, int N,
                    int K, TY* __restrict__ y, int64_t ldy, int glu_group) {
  constexpr bool GLU = MODE == 2;
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  __shared__ float us[GLU ? BK : 1][BN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN] = {}, acc2[GLU ? TM : 1][TN] = {};

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k per tile: thread i loads row i/4... four elements each
    for (int i = threadIdx.x; i < BM * BK; i += 256) {
      const int r = i / BK, kk = i % BK;
      const int m = m0 + r, k = k0 + kk;
      xs[kk][r] = (m < M && k < K) ? to_float(x[(int64_t)m * ldx + k]) : 0.f;
      const int n = n0 + r;
      float wv = 0.f, uv = 0.f;
      if (n < N && k < K) {
        if (GLU) {
          const int64_t gr = (int64_t)(n / glu_group) * 2 * glu_group + n % glu_group;
          wv = to_float(w[gr * K + k]);
          uv = to_float(w[(gr + glu_group) * K + k]);
        } else {
          wv = to_float(w[(int64_t)n * K + k]);
        }
      }
      ws[kk][r] = wv;
      if (GLU) us[kk][r] = uv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN], c[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b[j] = ws[kk][tx * TN + j];
        if (GLU) c[j] = us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GLU) acc2[i][j] = fmaf(a[i], c[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      TY* p = y + (int64_t)m * ldy + n;
      if (MODE == 0) {
        *p = from_float<TY>(acc[i][j]);
      } else if (MODE == 1) {
        *p = from_float<TY>(to_float(*p) + acc[i][j]);
      } else {
        const float g = acc[i][j];
        *p = from_float<TY>(g / (1.0f + expf(-g)) * acc2[GLU ? i : 0][j]);
      }
    }
  }
}

template <typename TX, typename TW, typename TY>
int launch(const void* x, int64_t ldx, const void* w, int M, int N, int K, void* y, int64_t ldy,
           int mode, int glu_group, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return fail(kBadArgument, "linear_plain: %d rows exceed the grid", M);
#define SKYLA_LAUNCH(MODE)                                                           \
  linear_plain_kernel<TX, TW, TY, MODE><<<grid, 256, 0, stream>>>(                    \
      (const TX*)x, ldx, (const TW*)w, M, N, K, (TY*)y, ldy, glu_group)
  if (mode == 0) SKYLA_LAUNCH(0);
  else if (mode == 1) SKYLA_LAUNCH(1);
  else SKYLA_LAUNCH(2);
#undef SKYLA_LAUNCH
  return check_launch("linear_plain");
}
}  // namespace

// N counts output columns; in gated mode W has 2N rows.
extern "C" int skyla_linear_plain(const void* x, int x_dtype, int64_t ldx, const void* w,
                                  int w_dtype, int M, int N, int K, void* y, int y_dtype,
                                  int64_t ldy, int mode, int glu_group, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || ldx < K || ldy < N) return fail(kBadArgument, "linear_plain: bad sizes M=%d N=%d K=%d", M, N, K);
  if (mode < 0 || mode > 2) return fail(kBadArgument, "linear_plain: unknown epilogue %d", mode);
  if (mode == 1 && y_dtype != kF32) return fail(kBadArgument, "linear_plain: the accumulate epilogue needs a 32-bit output");
  if (mode == 2 && (glu_group <= 0 || N % glu_group))
    return fail(kBadArgument, "linear_plain: gate/up group %d does not divide N=%d", glu_group, N);
  SKYLA_DISPATCH(x_dtype, TX, SKYLA_DISPATCH(w_dtype, TW, SKYLA_DISPATCH(y_dtype, TY, {
    return launch<TX, TW, TY>(x, ldx, w, M, N, K, y, ldy, mode, glu_group, stream);
  });););
  return kOk;
}
