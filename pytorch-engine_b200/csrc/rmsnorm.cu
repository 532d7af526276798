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
#include "api.h"
#include "common.cuh"

namespace pe {

template <typename TDelta, typename TOut>
__global__ void rmsnorm_kernel(float* __restrict__ residual, const TDelta* delta,
                               const float* __restrict__ weight, TOut* __restrict__ out,
                               const int* rows, int n_rows, int dim, float eps) {
  extern __shared__ float row_buf[];  // dim floats
  __shared__ float red[32];
  pdl_wait_block();
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

// The same with 4-element accesses (16-byte loads and stores of the float32 stream), for widths that
// are a multiple of 4; rows then start on 16-byte boundaries.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <typename TDelta, typename TOut>
__global__ void __launch_bounds__(1024) rmsnorm_vec4_kernel(float* __restrict__ residual, const TDelta* delta,
                                                             const float* __restrict__ weight, TOut* __restrict__ out,
                                                             const int* rows, int n_rows, int dim, float eps) {
  extern __shared__ float row_buf[];  // dim floats
  __shared__ float red[32];
  // The norm's weight does not depend on the kernels before this one: the part of it that this thread
  // needs first is on its way before the wait (a decode step waits for this kernel's latency 73 times).
  const int c0 = threadIdx.x * 4;
  float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c0 < dim) w0 = Vec4<float>::load(weight + c0);
  pdl_wait_block();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* res_row = residual + src * dim;
  const TDelta* d_row = delta ? delta + src * dim : nullptr;
  const bool write_back = (d_row != nullptr) && (rows == nullptr);
  float ss = 0.f;
  for (int c = c0; c < dim; c += blockDim.x * 4) {
    float4 h = Vec4<float>::load(res_row + c);
    if (d_row) {
      const float4 d = Vec4<TDelta>::load(d_row + c);
      h.x += d.x; h.y += d.y; h.z += d.z; h.w += d.w;
      if (write_back) Vec4<float>::store(res_row + c, h);
    }
    *reinterpret_cast<float4*>(row_buf + c) = h;
    ss += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)dim + eps);
  TOut* o_row = out + (size_t)r * dim;
  for (int c = c0; c < dim; c += blockDim.x * 4) {
    const float4 h = *reinterpret_cast<const float4*>(row_buf + c);
    const float4 w = c == c0 ? w0 : Vec4<float>::load(weight + c);
    Vec4<TOut>::store(o_row + c, make_float4(h.x * inv * w.x, h.y * inv * w.y, h.z * inv * w.z, h.w * inv * w.w));
  }
}

// Plain RMSNorm of a tensor in the run dtype (rows of any width), used by parts that normalise
// something other than the residual stream.
template <typename T>
__global__ void rmsnorm_plain_kernel(const T* x, const float* __restrict__ weight, T* __restrict__ out,
                                     int n_rows, int dim, float eps) {
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  pdl_wait_block();
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
  int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  int e;
  const bool vec = (dim % 4 == 0) && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0) && ((uintptr_t)delta % 16 == 0);
  // A handful of rows (a decode step): what counts is the kernel's latency, and a thread that has a
  // second 16-byte piece to fetch waits for memory a second time (8B shape, batch 8: 3.97 ms a step with
  // 512 threads a row, 3.95 with 1,024, 4.08 with 256, 5.18 with 128).
  if (vec && n_rows <= 64 && dim > 2048) threads = 1024;
  if (dtype == PE_F32) {
    auto k = vec ? pe::rmsnorm_vec4_kernel<float, float> : pe::rmsnorm_kernel<float, float>;
    if ((e = pe::set_smem(k, smem))) return e;
    pe::launch(k, n_rows, threads, smem, stream, residual, (const float*)delta, weight, (float*)out, rows, n_rows, dim, eps);
  } else if (dtype == PE_BF16) {
    auto k = vec ? pe::rmsnorm_vec4_kernel<__nv_bfloat16, __nv_bfloat16> : pe::rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>;
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
