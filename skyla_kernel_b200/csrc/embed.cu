// Embedding gather: x[t, :] = table[token[t], :], no scaling
// (skyla-ref/src/model.rs:99-100; the reference dequantizes the row on the CPU,
// skyla-engine/src/engine.rs:109-115).  One block per token.
#include "common.cuh"
using namespace skyla;
SKYLA_EXPORT_ERROR_MESSAGE()

// A token outside the table (it can only come from the device: the host checks what it feeds) reads
// nothing: its row is filled with zeros and the device's error word is raised (code 32).
constexpr int kTokenOutsideCode = 32;

template <typename TW, typename TO>
__global__ void embed_gather_kernel(const int32_t* __restrict__ tokens, const TW* __restrict__ table,
                                    int vocab, int hidden, TO* __restrict__ out, int64_t ldo, int* error_flag) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int token = tokens[t];
  TO* o = out + (int64_t)t * ldo;
  if (token < 0 || token >= vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TO>(0.f);
    if (threadIdx.x == 0 && error_flag != nullptr) atomicCAS(error_flag, 0, kTokenOutsideCode);
    return;
  }
  const TW* row = table + (int64_t)token * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TO>(to_float(row[i]));
}

// The host checks the tokens it feeds against the vocabulary; tokens fed on the device (a sampler's
// output) are checked here.  error_flag may be null.
extern "C" int skyla_embed_gather(const int32_t* tokens, int n_tokens, const void* table,
                                  int table_dtype, int vocab, int hidden, void* out, int out_dtype,
                                  int64_t ldo, int* error_flag, cudaStream_t stream) {
  if (n_tokens <= 0) return kOk;
  if (hidden <= 0 || ldo < hidden || vocab <= 0) return fail(kBadArgument, "embed_gather: bad table %d x %d", vocab, hidden);
  const int threads = hidden >= 1024 ? 256 : 128;
  SKYLA_DISPATCH(table_dtype, TW, SKYLA_DISPATCH(out_dtype, TO, {
    launch_overlapped(embed_gather_kernel<TW, TO>, dim3(n_tokens), dim3(threads), 0, stream,
                      tokens, (const TW*)table, vocab, hidden, (TO*)out, ldo, error_flag);
  }););
  return check_launch("embed_gather");
}
