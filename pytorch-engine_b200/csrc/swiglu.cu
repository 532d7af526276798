// SwiGLU activation: out[r, c] = silu(gate[r, c]) * up[r, c], gate and up being the two halves of
// one row of the fused gate|up projection (gate first).
// Reference formula: pygguf_engine/quant_kernels.py:1467-1472 (silu and product in float32).  The
// reference's float16 row scale (1473-1474) cancels exactly and is not needed in bfloat16/float32.
#include "api.h"
#include "common.cuh"

namespace pe {

template <typename T>
__global__ void silu_mul_kernel(const T* gate_up, T* __restrict__ out, int n_rows, int inter,
                                size_t in_stride) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t total = (size_t)n_rows * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter, c = i - r * inter;
    const float g = to_f32<T>(gate_up[r * in_stride + c]);
    const float u = to_f32<T>(gate_up[r * in_stride + inter + c]);
    const float s = g / (1.0f + expf(-g));
    out[i] = from_f32<T>(s * u);
  }
}

}  // namespace pe

extern "C" int pe_silu_mul(int dtype, const void* gate_up, void* out, int n_rows, int inter, cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (inter <= 0) return PE_ERR_BAD_ARGUMENT;
  const size_t total = (size_t)n_rows * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > pe::kSMs * 16) blocks = pe::kSMs * 16;
  if (dtype == PE_F32)
    pe::launch(pe::silu_mul_kernel<float>, (int)blocks, threads, 0, stream, (const float*)gate_up, (float*)out, n_rows, inter, (size_t)2 * inter);
  else if (dtype == PE_BF16)
    pe::launch(pe::silu_mul_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n_rows, inter, (size_t)2 * inter);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
