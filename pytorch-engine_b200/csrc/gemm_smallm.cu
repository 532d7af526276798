// y[M, N] = x[M, K] . W[N, K]^T for a handful of rows (M <= 16): the decode-step matrix products.
// bfloat16 operands, float32 accumulation on the tensor cores (mma.sync m16n8k16), output bfloat16 or
// float32, optionally with the SwiGLU gate fused into the epilogue.
//
// With so few rows the product is a stream of the weight matrix through the SMs; everything here
// serves that stream.  The roles of the MMA operands are swapped: 16 weight rows are the MMA's M
// dimension, the (up to 8) activation rows are its N dimension.  A warp owns 16 weight rows and a
// slice of K and loads its fragments straight from global memory with 16-byte loads: lane (g, t)
// reads elements [8t, 8t+8) of rows g and g+8 of every 32-wide k block.  The contraction index
// inside a block is permuted accordingly (the same permutation for both operands, so the sum is
// unchanged), which is what lets a fragment be one contiguous 16-byte load instead of four 4-byte
// ones.  Weights are read once and bypass L1; the activations (a few KB per row) are re-read by every
// warp and stay in L1.  The warps of a block split K among themselves and are summed through shared
// memory in warp order (no atomics: the result does not depend on scheduling).
//
// The library matrix product (cuBLAS) stands for larger M and for shapes refused here
// (K not a multiple of 8, M > 16), as the reference uses a library product for its unquantised
// linears (pygguf_engine/quant_kernels.py:1836).  The fused epilogue restates
// pygguf_engine/quant_kernels.py:1467-1472 (silu(gate) * up in float32).
#include "api.h"
#include "common.cuh"

namespace pe {
namespace smallm {

struct Args {
  const __nv_bfloat16* x; long long ldx;
  const __nv_bfloat16* w;      // [n_rows_total, K]
  void* y; long long ldy;
  int M, N, K;
  int pair_offset;             // PAIR: row n is combined with row n + pair_offset; N counts output columns
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Activations come from the kernel before this one, which may still be running when this kernel starts:
// an ordinary (coherent) load that neither the compiler nor the assembler may move above the
// dependency wait.  A non-coherent load (ld.global.nc) promises data that nobody writes while the
// kernel lives, and may be hoisted.
__device__ __forceinline__ uint4 ldg_cached(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// NT: 8-row groups of activations (1: M <= 8, 2: M <= 16).  PAIR: two weight-row blocks per warp
// (gate and up), combined as silu(gate) * up.  WARPS: warps per block = K slices.  U: k blocks per batch
// of loads.
// Registers are capped at 128 per thread for M <= 8 so that 16 warps fit on an SM: what limits this
// kernel is how many bytes its SM has in flight.  For M <= 16 that cap would spill.
template <int NT, bool PAIR, int WARPS, int U, typename OutT>
__global__ void __launch_bounds__(WARPS * 32, NT == 1 ? 16 / WARPS : 1) gemm_smallm_kernel(Args a) {
  __shared__ float red[WARPS][(PAIR ? 2 : 1) * NT][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int K = a.K;
  const int kblocks = (K + 31) / 32;
  const int per = (kblocks + WARPS - 1) / WARPS;
  const int kb_lo = warp * per, kb_hi = min(kblocks, kb_lo + per);
  // weight rows of this lane; rows beyond the matrix are clamped (their results are never stored)
  const int r_lo = min(n0 + g, a.N - 1), r_hi = min(n0 + g + 8, a.N - 1);
  const uint4* w_lo = reinterpret_cast<const uint4*>(a.w + (size_t)r_lo * K) + t;
  const uint4* w_hi = reinterpret_cast<const uint4*>(a.w + (size_t)r_hi * K) + t;
  const uint4* w2_lo = nullptr;
  const uint4* w2_hi = nullptr;
  if (PAIR) {
    w2_lo = reinterpret_cast<const uint4*>(a.w + (size_t)(r_lo + a.pair_offset) * K) + t;
    w2_hi = reinterpret_cast<const uint4*>(a.w + (size_t)(r_hi + a.pair_offset) * K) + t;
  }
  const uint4* xr[NT];
  bool x_ok[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int m = n * 8 + g;
    x_ok[n] = m < a.M;
    xr[n] = reinterpret_cast<const uint4*>(a.x + (size_t)(x_ok[n] ? m : 0) * a.ldx) + t;
  }
  float c[(PAIR ? 2 : 1) * NT][4];
#pragma unroll
  for (int i = 0; i < (PAIR ? 2 : 1) * NT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
  const int k_chunks = K / 8;  // 16-byte chunks per row (K is a multiple of 8)

  // Two batches of U k blocks are in flight at any time: the loads of the next batch are issued
  // before the MMAs of the current one.
  struct Batch {
    uint4 wl[U], wh[U], vl[PAIR ? U : 1], vh[PAIR ? U : 1], xb[U][NT];
  };
  auto load_w = [&](Batch& bt, int kb) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int blk = kb + u;
      const bool live = blk < kb_hi && (blk * 4 + t) < k_chunks;
      bt.wl[u] = live ? ldg_stream(w_lo + blk * 4) : zero;
      bt.wh[u] = live ? ldg_stream(w_hi + blk * 4) : zero;
      if (PAIR) {
        bt.vl[u] = live ? ldg_stream(w2_lo + blk * 4) : zero;
        bt.vh[u] = live ? ldg_stream(w2_hi + blk * 4) : zero;
      }
    }
  };
  auto load_x = [&](Batch& bt, int kb) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int blk = kb + u;
      const bool live = blk < kb_hi && (blk * 4 + t) < k_chunks;
#pragma unroll
      for (int n = 0; n < NT; ++n) bt.xb[u][n] = (live && x_ok[n]) ? ldg_cached(xr[n] + blk * 4) : zero;
    }
  };
  auto load = [&](Batch& bt, int kb) {
    load_w(bt, kb);
    load_x(bt, kb);
  };
  auto fold = [&](const Batch& bt) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mma_bf16(c[n], bt.wl[u].x, bt.wh[u].x, bt.wl[u].y, bt.wh[u].y, bt.xb[u][n].x, bt.xb[u][n].y);
        mma_bf16(c[n], bt.wl[u].z, bt.wh[u].z, bt.wl[u].w, bt.wh[u].w, bt.xb[u][n].z, bt.xb[u][n].w);
        if (PAIR) {
          mma_bf16(c[NT + n], bt.vl[u].x, bt.vh[u].x, bt.vl[u].y, bt.vh[u].y, bt.xb[u][n].x, bt.xb[u][n].y);
          mma_bf16(c[NT + n], bt.vl[u].z, bt.vh[u].z, bt.vl[u].w, bt.vh[u].w, bt.xb[u][n].z, bt.xb[u][n].w);
        }
      }
    }
  };
  // The weights do not depend on the kernels before this one: start the first batch of weight loads,
  // and only then wait for the predecessor, whose output is the activations.  (Starting both batches
  // before the wait, or asking for the rest of the warp's slab with prefetch.global.L2, was measured
  // slower: 4.37 and 4.67 ms against 4.34 ms for a decode step of 8 sequences.)
  Batch b0, b1;
  load_w(b0, kb_lo);
  pdl_wait_block();
  load_x(b0, kb_lo);
  for (int kb = kb_lo; kb < kb_hi; kb += 2 * U) {
    load(b1, kb + U);
    fold(b0);
    load(b0, kb + 2 * U);
    fold(b1);
  }
  pdl_launch_dependents();  // the stream of weights is done: the next kernel may start its own
  // sum the K slices in warp order
  if (WARPS > 1) {
#pragma unroll
    for (int i = 0; i < (PAIR ? 2 : 1) * NT; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) red[warp][i][e][lane] = c[i][e];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < (PAIR ? 2 : 1) * NT; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float s = red[0][i][e][lane];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) s += red[w][i][e][lane];
        c[i][e] = s;
      }
  }
  // c[n][e]: weight row n0 + g (+8 for e >= 2), activation row n*8 + 2t + (e & 1)
  OutT* y = reinterpret_cast<OutT*>(a.y);
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = n0 + g + ((e >= 2) ? 8 : 0);
      const int m = n * 8 + 2 * t + (e & 1);
      if (col >= a.N || m >= a.M) continue;
      float v = c[n][e];
      if (PAIR) {
        const float up = c[NT + n][e];
        v = sizeof(OutT) == 2 ? silu_mul_fast(v, up) : v / (1.0f + expf(-v)) * up;   // exact for a float32 result
      }
      store_out<OutT>(y + (size_t)m * a.ldy + col, v);
    }
}

template <int NT, bool PAIR, typename OutT>
static int launch(const Args& a, int n_sms, cudaStream_t stream) {
  const int blocks = (a.N + 15) / 16;
  const int kblocks = (a.K + 31) / 32;
  constexpr int U = PAIR ? 2 : 4;
  // K slices per block of 16 weight rows: enough warps in flight over the whole GPU to cover the
  // memory latency, but at least two batches of k blocks per warp.  An SM holds 16 warps of the
  // M <= 8 kernels (128 registers) and 12 of the M <= 16 kernels (up to 168 registers) as long as their
  // blocks have at most 4 warps; a block of 8 would be alone on its SM.
  constexpr int kMaxWarps = NT == 1 ? 8 : 4;
  const long long slots = (long long)n_sms * (NT == 1 ? 16 : 12);
  const long long want_warps = (long long)n_sms * 24;
  int warps = 1;
  while (warps < kMaxWarps && (long long)blocks * warps < want_warps && kblocks / (warps * 2) >= 2 * U) warps *= 2;
  // A second wave that fills less than half of the GPU costs more than longer K slices in one wave
  // (6144 x 4096 at 8 rows: 11.5 us with 8 warps a block, 1.3 waves; 10.2 us with 4).
  if (warps > 1 && (long long)blocks * warps > slots && (long long)blocks * warps * 2 <= slots * 3) warps /= 2;
  switch (warps) {
    case 1: pe::launch(gemm_smallm_kernel<NT, PAIR, 1, U, OutT>, blocks, 32, 0, stream, a); break;
    case 2: pe::launch(gemm_smallm_kernel<NT, PAIR, 2, U, OutT>, blocks, 64, 0, stream, a); break;
    case 4: pe::launch(gemm_smallm_kernel<NT, PAIR, 4, U, OutT>, blocks, 128, 0, stream, a); break;
    default: pe::launch(gemm_smallm_kernel<NT, PAIR, 8, U, OutT>, blocks, 256, 0, stream, a); break;
  }
  PE_LAUNCH_CHECK();
  return PE_OK;
}

}  // namespace smallm
}  // namespace pe

extern "C" int pe_gemm_smallm_supported(int M, int N, int K) {
  return (M >= 1 && M <= 16 && N >= 1 && K >= 8 && K % 8 == 0) ? 1 : 0;
}

// out_f32 != 0: y is float32, else bfloat16.  pair_offset > 0: W has 2 * N rows, row n (gate) is paired with
// row n + pair_offset (up) and y[m, n] = silu(x.gate_n) * (x.up_n).  n_sms: the device's SM count (it sizes the
// split of K over a block's warps; 0: a B200's).
extern "C" int pe_gemm_smallm(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
                              int out_f32, int pair_offset, int n_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return PE_OK;
  if (!pe_gemm_smallm_supported(M, N, K)) return PE_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || (ldx * 2) % 16) return PE_ERR_BAD_ARGUMENT;
  pe::smallm::Args a;
  a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.w = (const __nv_bfloat16*)w; a.y = y; a.ldy = ldy;
  a.M = M; a.N = N; a.K = K; a.pair_offset = pair_offset;
  using namespace pe::smallm;
  if (n_sms <= 0) n_sms = pe::kSMs;
  const bool pair = pair_offset > 0;
  if (M <= 8) {
    if (pair) return out_f32 ? launch<1, true, float>(a, n_sms, stream) : launch<1, true, __nv_bfloat16>(a, n_sms, stream);
    return out_f32 ? launch<1, false, float>(a, n_sms, stream) : launch<1, false, __nv_bfloat16>(a, n_sms, stream);
  }
  if (pair) return out_f32 ? launch<2, true, float>(a, n_sms, stream) : launch<2, true, __nv_bfloat16>(a, n_sms, stream);
  return out_f32 ? launch<2, false, float>(a, n_sms, stream) : launch<2, false, __nv_bfloat16>(a, n_sms, stream);
}
