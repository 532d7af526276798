// Token embedding: residual stream (float32) <- table[ids].
// Reference formula: pygguf_engine/quant_kernels.py:1846-1847 (row gather, cast to float32).
#include "api.h"
#include "common.cuh"

namespace pe {

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* ids,
                                    float* __restrict__ out, int n_tokens, int hidden, int vocab, int* status) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  if (row >= n_tokens) return;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) report(status, kStatusTokenOutOfRange, row, id, vocab);
    // the row is still defined: zeros
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[(size_t)row * hidden + c] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  float* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32<T>(src[c]);
}

}  // namespace pe

extern "C" int pe_embed_gather(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden,
                               int vocab, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (hidden <= 0 || vocab <= 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == PE_F32)
    pe::launch(pe::embed_gather_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, out, n_tokens, hidden, vocab, status);
  else if (dtype == PE_BF16)
    pe::launch(pe::embed_gather_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, n_tokens, hidden, vocab, status);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
