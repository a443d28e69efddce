// Embedding gather: x[t, :] = table[token[t], :], no scaling
// (skyla-ref/src/model.rs:99-100; the reference dequantizes the row on the CPU,
// skyla-engine/src/engine.rs:109-115).  One block per token.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

template <typename TW, typename TO>
__global__ void embed_gather_kernel(const int32_t* __restrict__ tokens, const TW* __restrict__ table,
                                    int hidden, TO* __restrict__ out, int64_t ldo) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const TW* row = table + (int64_t)tokens[t] * hidden;
  TO* o = out + (int64_t)t * ldo;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TO>(to_float(row[i]));
}

// tokens must already be checked against the vocabulary on the host.
extern "C" int skyla_embed_gather(const int32_t* tokens, int n_tokens, const void* table,
                                  int table_dtype, int hidden, void* out, int out_dtype,
                                  int64_t ldo, cudaStream_t stream) {
  if (n_tokens <= 0) return kOk;
  if (hidden <= 0 || ldo < hidden) return fail(kBadArgument, "embed_gather: bad width %d", hidden);
  const int threads = hidden >= 1024 ? 256 : 128;
  SKYLA_DISPATCH(table_dtype, TW, SKYLA_DISPATCH(out_dtype, TO, {
    launch_overlapped(embed_gather_kernel<TW, TO>, dim3(n_tokens), dim3(threads), 0, stream,
                      tokens, (const TW*)table, hidden, (TO*)out, ldo);
  }););
  return check_launch("embed_gather");
}
