// Shared device helpers: element types, reductions, the status word.
//
// Every kernel of this library is reached through an extern "C" launcher (see api.h) that takes raw
// device pointers and a stream, checks its sizes on the host and returns a negative PE_ERR_* code for
// a size it refuses.  Kernels never trap: a bad index or a wait that ran out is recorded in a status
// word in global memory, the access is skipped, and the host reads the word after the step.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace pe {

constexpr int kPageTokens = 64;  // tokens per cache page (the unit in which the cache is handed out)

// ---- status word -------------------------------------------------------------------------------
// status[0]: first error code seen (0 = none); status[1..3]: details of that first error.
enum StatusCode : int {
  kStatusOk = 0,
  kStatusTokenOutOfRange = 1,   // embedding: token id outside the table
  kStatusPageOutOfRange = 2,    // cache: page table entry outside the pool
  kStatusPositionOutOfRange = 3,// position beyond the tables or the page table
  kStatusWaitTimedOut = 4,      // a bounded wait (mbarrier / TMA / MMA commit) ran out
  kStatusSlotOutOfRange = 5,
};

__device__ __forceinline__ void report(int* status, int code, int a = 0, int b = 0, int c = 0) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = a;
    status[2] = b;
    status[3] = c;
  }
}

// SMs of a B200.  Used only to size grids and in launch heuristics, never for correctness.
constexpr int kSMs = 148;

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of this library is launched so that it may start while its predecessor in the stream
// is still draining: it does whatever does not depend on earlier kernels (a matrix product starts
// loading its weights), waits for the predecessor to have completed and flushed (`pdl_wait_block`), and only
// then lets its own successor start (`pdl_launch_dependents`; a long kernel does so when its main
// loop is done).  So at most one successor is resident and waiting at any time: letting successors
// start earlier was measured to cost more (their waiting blocks take registers and warp slots from
// the kernel that is running) than it gains.  Nothing is read from, or written to, memory that
// another kernel of the step touches before the wait, and what an earlier kernel wrote is read with
// ordinary loads only (no ld.global.nc, no `const __restrict__` pointer: such a load may be moved
// above the wait, where the data is not there yet).  Launch latency and the ramp-up of the weight
// stream thus overlap the previous kernel's tail.  PE_B200_PDL=0 switches the launch attribute off
// (the two instructions are then no-ops).  One kernel is launched without it, because that was measured
// faster: the merge of the decode attention's ranges (attention_mma.cu).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// The wait of a whole block: its first warp waits for the predecessor, the others wait for that warp at
// the block's barrier (the predecessor's writes are visible to the whole grid once one thread's wait has
// returned).  Fewer warps in griddepcontrol.wait was measured faster: decode at batch 8 4.02 -> 3.97 ms a
// step, at batch 1 290 -> 301 tokens/s, all of it from the weight-streaming products (8 warps a block).
// Every thread of the block must reach it (blocks are one-dimensional).
__device__ __forceinline__ void pdl_wait_block() {
  if (threadIdx.x < 32) pdl_wait();
  __syncthreads();
}

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("PE_B200_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_as(bool early_start, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (early_start && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The usual launch: the kernel may start while its predecessor drains.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  return launch_as(true, kernel, grid, block, smem, stream, args...);
}

// A launch that starts only when its predecessor has completed (the two instructions in the kernel are
// then no-ops for it; its own successor may still start early).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args... args) {
  return launch_as(false, kernel, grid, block, smem, stream, args...);
}

// ---- element conversion ----------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// silu(g) * u for an epilogue that rounds its result to bfloat16: the exponential and the reciprocal are
// the hardware approximations (about 2 ulp each, far inside bfloat16's 8 bits).  With expf and an IEEE
// division the epilogue of the fused gate|up product took longer than the tile's matrix products
// (358 us against 260 us for 2,048 rows of the 8B shape).  Large |g|: exp(-g) = inf gives -0, = 0 gives g.
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// ---- reductions --------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum in a fixed tree order (deterministic); `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

}  // namespace pe

// ---- error codes of the extern "C" launchers (negative; CUDA runtime errors are returned positive)
#define PE_OK 0
#define PE_ERR_UNSUPPORTED_SIZE (-1)
#define PE_ERR_BAD_ARGUMENT (-2)
#define PE_ERR_UNSUPPORTED_DTYPE (-3)

// dtype tags of the C interface
#define PE_F32 0
#define PE_BF16 1

#define PE_LAUNCH_CHECK()                         \
  do {                                            \
    cudaError_t e__ = cudaGetLastError();         \
    if (e__ != cudaSuccess) return (int)e__;      \
  } while (0)
