// y[M, N] = x[M, K] . W[N, K]^T for many rows (prefill), bfloat16 operands, float32 accumulation, on
// the fifth-generation tensor cores: tcgen05.mma issued by one thread, operands staged in shared
// memory by TMA, accumulators in tensor memory (TMEM), read back with tcgen05.ld for the epilogue.
//
// One persistent block per SM walks output tiles of 128 x 256.  Its warps have fixed roles:
//   warp 0  producer: waits for a free stage, starts the TMA copies of a 128x64 tile of x and a
//           256x64 tile of W (128-byte swizzle, K-major) and lets the stage's mbarrier count the bytes;
//   warp 1  MMA: waits for a full stage, issues four tcgen05.mma (K = 16 each) into the tile's
//           accumulator, and commits the stage back to the producer; after the last k block it
//           commits the accumulator to the epilogue;
//   warps 2-5  epilogue: wait for the accumulator, read their 32 TMEM lanes (= 32 output rows) in
//           chunks of 32 columns, convert and store, then hand the accumulator back.
// There are two accumulators (2 x 256 TMEM columns), so the epilogue of one tile overlaps the
// matrix products of the next.  Epilogues: bfloat16 or float32 store, or the SwiGLU gate: the W tile
// is then 128 gate rows and the 128 matching up rows, and out[m, n] = silu(gate) * up
// (pygguf_engine/quant_kernels.py:1467-1472) without the gate|up matrix ever reaching memory.
//
// Every wait is bounded (tma.cuh); a wait that runs out records kStatusWaitTimedOut, every role
// leaves its loop, and the block frees its TMEM before it returns.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace pe {
namespace umma {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int kBytesA = BM * BK * 2, kBytesB = BN * BK * 2, kStage = kBytesA + kBytesB;
constexpr int kTmemCols = 512;  // two accumulators of 256 float32 columns
constexpr int kThreads = 192;

struct Params {
  int M, N, K;            // N counts output columns (PAIR: I)
  void* y; long long ldy;
  int mode;               // 0: bfloat16, 1: float32, 2: silu(gate) * up -> bfloat16
  int pair_offset;        // mode 2: row of W that pairs with row 0
  int m_tiles, n_tiles, n_per_tile;
  int* status;
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(holder_smem)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// arrive on `bar` once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tma::smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive float32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 64 bfloat16
// (128 bytes), groups of 8 rows 1024 bytes apart.  Bits: start address >> 4 [0,14), leading byte
// offset >> 4 [16,30) (unused by swizzled K-major layouts), stride byte offset >> 4 [32,46) = 1024 >> 4,
// descriptor version 1 [46,48), layout type SWIZZLE_128B = 2 [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of kind::f16: D float32 (1 << 4), A and B bfloat16 (1 << 7, 1 << 10), both
// K-major (bits 15, 16 clear), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_umma_kernel(Params p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap) {
  extern __shared__ char smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ volatile int failed;
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int n_tiles_total = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tma::mbar_init(&full_bar[s], 1);
      tma::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tma::mbar_init(&acc_full[b], 1);
      tma::mbar_init(&acc_empty[b], 4);
    }
    failed = 0;
    tma::fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(&tmem_holder, kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_holder;
  pdl_wait_block();  // set-up (barriers, tensor memory) is done; now the inputs must be complete
  pdl_launch_dependents();

  if (warp == 0) {
    // ---- producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < n_tiles_total && !failed; tile += gridDim.x) {
        const int m0 = (tile % p.m_tiles) * BM;
        const int n0 = (tile / p.m_tiles) * p.n_per_tile;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!tma::mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report(p.status, kStatusWaitTimedOut, 10, tile, kb);
            failed = 1;
            break;
          }
          char* sa = smem + stage * kStage;
          char* sb = sa + kBytesA;
          tma::mbar_expect_tx(&full_bar[stage], kStage);
          tma::load_2d(sa, &amap, kb * BK, m0, &full_bar[stage]);
          if (p.mode == 2) {
            tma::load_2d(sb, &bmap, kb * BK, n0, &full_bar[stage]);
            tma::load_2d(sb + kBytesB / 2, &bmap, kb * BK, p.pair_offset + n0, &full_bar[stage]);
          } else {
            tma::load_2d(sb, &bmap, kb * BK, n0, &full_bar[stage]);
            tma::load_2d(sb + kBytesB / 2, &bmap, kb * BK, n0 + BN / 2, &full_bar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = instr_desc(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles_total && !failed; tile += gridDim.x, ++it) {
        const int ab = it & 1;
        if (!tma::mbar_wait(&acc_empty[ab], ((it >> 1) & 1) ^ 1)) {
          report(p.status, kStatusWaitTimedOut, 11, tile, ab);
          failed = 1;
          break;
        }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!tma::mbar_wait(&full_bar[stage], phase)) {
            report(p.status, kStatusWaitTimedOut, 12, tile, kb);
            failed = 1;
            break;
          }
          fence_after_sync();
          const uint32_t sa = tma::smem_addr(smem + stage * kStage);
          const uint32_t sb = sa + kBytesA;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(d_tmem, smem_desc(sa + k * 32), smem_desc(sb + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);   // the stage is free once these products have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&acc_full[ab]);          // the accumulator is complete once all products are done
      }
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles_total && !failed; tile += gridDim.x, ++it) {
      const int ab = it & 1;
      const int m0 = (tile % p.m_tiles) * BM;
      const int n0 = (tile / p.m_tiles) * p.n_per_tile;
      if (!tma::mbar_wait(&acc_full[ab], (it >> 1) & 1)) {
        if (lane == 0) report(p.status, kStatusWaitTimedOut, 13, tile, ab);
        failed = 1;
        break;
      }
      fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ab * BN + ((uint32_t)(quarter * 32) << 16);
      if (p.mode == 2) {
        __nv_bfloat16* yrow = reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)row * p.ldy + n0;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(t_row + c, g);
          tmem_ld32(t_row + 128 + c, u);
          tmem_ld_wait();
          if (row < p.M) {
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
              const float v0 = silu_mul_fast(g0, __uint_as_float(u[2 * j]));
              const float v1 = silu_mul_fast(g1, __uint_as_float(u[2 * j + 1]));
              o[j] = pack2(v0, v1);
            }
            if (n0 + c + 32 <= p.N && (p.ldy % 8) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(yrow + c)[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (n0 + c + j < p.N) yrow[c + j] = reinterpret_cast<__nv_bfloat16*>(o)[j];
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(t_row + c, v);
          tmem_ld_wait();
          if (row < p.M && n0 + c < p.N) {
            if (p.mode == 1) {
              float* yrow = reinterpret_cast<float*>(p.y) + (size_t)row * p.ldy + n0 + c;
              if (n0 + c + 32 <= p.N && (p.ldy % 4) == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  reinterpret_cast<uint4*>(yrow)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              } else {
                for (int j = 0; j < 32; ++j)
                  if (n0 + c + j < p.N) yrow[j] = __uint_as_float(v[j]);
              }
            } else {
              __nv_bfloat16* yrow = reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)row * p.ldy + n0 + c;
              uint32_t o[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = pack2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
              if (n0 + c + 32 <= p.N && (p.ldy % 8) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  reinterpret_cast<uint4*>(yrow)[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
              } else {
                for (int j = 0; j < 32; ++j)
                  if (n0 + c + j < p.N) yrow[j] = reinterpret_cast<__nv_bfloat16*>(o)[j];
              }
            }
          }
        }
      }
      // hand the accumulator back: one arrival per epilogue warp
      fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&acc_empty[ab]);
    }
  }
  // teardown: everyone meets, then the allocating warp frees the tensor memory
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace umma
}  // namespace pe

extern "C" int pe_gemm_umma_supported(int M, int N, int K, int pair_offset) {
  if (M < 1 || N < 1 || K < 8 || (K % 8)) return 0;
  if (pair_offset > 0 && (N % 128 || pair_offset != N)) return 0;  // gate and up blocks of 128 rows
  return 1;
}

// mode: 0 bfloat16 out, 1 float32 out; pair_offset > 0: W holds N gate rows then N up rows and
// y[m, n] = silu(x . gate_n) * (x . up_n), bfloat16.  x rows may be strided (ldx), W rows are dense.
extern "C" int pe_gemm_umma(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
                            int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream) {
  using namespace pe::umma;
  if (M <= 0 || N <= 0) return PE_OK;
  if (!pe_gemm_umma_supported(M, N, K, pair_offset)) return PE_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || (ldx * 2) % 16) return PE_ERR_BAD_ARGUMENT;
  Params p;
  p.M = M; p.N = N; p.K = K; p.y = y; p.ldy = ldy; p.status = status;
  p.mode = pair_offset > 0 ? 2 : (out_f32 ? 1 : 0);
  p.pair_offset = pair_offset;
  p.n_per_tile = pair_offset > 0 ? 128 : BN;
  p.m_tiles = (M + BM - 1) / BM;
  p.n_tiles = (N + p.n_per_tile - 1) / p.n_per_tile;
  CUtensorMap amap, bmap;
  const uint64_t w_rows = pair_offset > 0 ? 2ull * N : (uint64_t)N;
  int e = pe::tma::make_map_2d_bf16(&amap, x, K, M, ldx, BK, BM);
  if (e == 0) e = pe::tma::make_map_2d_bf16(&bmap, w, K, w_rows, K, BK, BN / 2);
  if (e != 0) return e < 0 ? e : PE_ERR_BAD_ARGUMENT;
  const size_t smem = 1024 + (size_t)STAGES * kStage;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < n_sms ? tiles : n_sms;
  pe::launch(gemm_umma_kernel, grid, kThreads, smem, stream, p, amap, bmap);
  PE_LAUNCH_CHECK();
  return PE_OK;
}
