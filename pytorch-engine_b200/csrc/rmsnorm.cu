// RMSNorm over the last dimension with the residual add fused in.
//
//   h   = residual[row] (+ delta[row])            float32
//   out = h * rsqrt(mean(h^2) + eps) * w          float32 math, stored in the run dtype
//
// Reference formulas: pygguf_engine/quant_kernels.py:1595-1596 (add, then norm), 831-833 (mean,
// rsqrt, multiply in float32), weight held in float32 (pygguf_engine/model.py:63).
// Modes:  rows == nullptr: row r of the output is row r of the stream; with `delta` the sum is
//         written back to the stream (the residual add of the block).
//         rows != nullptr: output row r is stream row rows[r] (+ delta row rows[r]); nothing is
//         written back (the final norm on the rows whose logits are wanted).
#include "common.cuh"

namespace pe {

template <typename TDelta, typename TOut>
__global__ void rmsnorm_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta,
                               const float* __restrict__ weight, TOut* __restrict__ out,
                               const int* __restrict__ rows, int n_rows, int dim, float eps) {
  extern __shared__ float row_buf[];  // dim floats
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* res_row = residual + src * dim;
  const TDelta* d_row = delta ? delta + src * dim : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float h = res_row[c];
    if (d_row) h += to_f32<TDelta>(d_row[c]);
    row_buf[c] = h;
    ss += h * h;
  }
  const float total = block_sum(ss, red);
  const float inv = rsqrtf(total / (float)dim + eps);
  const bool write_back = (d_row != nullptr) && (rows == nullptr);
  TOut* o_row = out + (size_t)r * dim;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float h = row_buf[c];
    if (write_back) res_row[c] = h;
    o_row[c] = from_f32<TOut>(h * inv * weight[c]);
  }
}

// Plain RMSNorm of a tensor in the run dtype (rows of any width), used by parts that normalise
// something other than the residual stream.
template <typename T>
__global__ void rmsnorm_plain_kernel(const T* __restrict__ x, const float* __restrict__ weight, T* __restrict__ out,
                                     int n_rows, int dim, float eps) {
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float h = to_f32<T>(x[(size_t)r * dim + c]);
    row_buf[c] = h;
    ss += h * h;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)dim + eps);
  for (int c = threadIdx.x; c < dim; c += blockDim.x)
    out[(size_t)r * dim + c] = from_f32<T>(row_buf[c] * inv * weight[c]);
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace pe

extern "C" int pe_rmsnorm_residual(int dtype, float* residual, const void* delta, const float* weight, void* out,
                                   const int* rows, int n_rows, int dim, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0) return PE_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)dim * sizeof(float);
  if (smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;  // rows wider than 51,200 features
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  int e;
  if (dtype == PE_F32) {
    auto k = pe::rmsnorm_kernel<float, float>;
    if ((e = pe::set_smem(k, smem))) return e;
    pe::launch(k, n_rows, threads, smem, stream, residual, (const float*)delta, weight, (float*)out, rows, n_rows, dim, eps);
  } else if (dtype == PE_BF16) {
    auto k = pe::rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>;
    if ((e = pe::set_smem(k, smem))) return e;
    pe::launch(k, n_rows, threads, smem, stream, residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, n_rows, dim, eps);
  } else {
    return PE_ERR_UNSUPPORTED_DTYPE;
  }
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_rmsnorm(int dtype, const void* x, const float* weight, void* out, int n_rows, int dim, float eps,
                          cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0) return PE_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)dim * sizeof(float);
  if (smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  int e;
  if (dtype == PE_F32) {
    auto k = pe::rmsnorm_plain_kernel<float>;
    if ((e = pe::set_smem(k, smem))) return e;
    pe::launch(k, n_rows, threads, smem, stream, (const float*)x, weight, (float*)out, n_rows, dim, eps);
  } else if (dtype == PE_BF16) {
    auto k = pe::rmsnorm_plain_kernel<__nv_bfloat16>;
    if ((e = pe::set_smem(k, smem))) return e;
    pe::launch(k, n_rows, threads, smem, stream, (const __nv_bfloat16*)x, weight, (__nv_bfloat16*)out, n_rows, dim, eps);
  } else {
    return PE_ERR_UNSUPPORTED_DTYPE;
  }
  PE_LAUNCH_CHECK();
  return PE_OK;
}
