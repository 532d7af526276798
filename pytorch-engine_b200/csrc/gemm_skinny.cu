// y[M, N] = x[M, K] . W[N, K]^T for 9..128 rows (decode at larger batches).  The weights are read
// once from HBM and that read is the cost, so everything serves the weight stream:
//   * the rows of x are the MMA's M side (64 or 128, padded with zeros by TMA), a narrow slice of W
//     rows its N side; the slice is as narrow as it takes to give every SM a tile (6144 features on
//     148 SMs: 48 per tile), so no SM idles and nothing has to be summed across blocks;
//   * a stage holds up to four k blocks of 64 (one 3-D TMA copy per operand brings them all: a thread
//     can issue a copy only every ~150 ns, and 512 contiguous bytes per weight row suit HBM better
//     than 128), and as many stages as fit keep the weights in flight;
//   * the producer starts the first W copies before the programmatic-dependent-launch wait: weights
//     do not depend on the preceding kernel, only x does.
// Persistent blocks walk the tiles; two accumulators in tensor memory let a tile's epilogue overlap
// the next tile's products (this matters for the output head, which has more tiles than SMs).
//   warp 0  producer (TMA, mbarrier per stage), warp 1  MMA issuer (tcgen05.mma kind::f16, M = 64 or
//   128), warps 2-5  epilogue (tcgen05.ld, convert, store).
// With M = 64 the accumulator's row r lies in TMEM lane 32 * (r / 16) + r % 16: every warp's lane
// quarter holds 16 rows in its lanes 0..15.
// Epilogues: bfloat16, float32, or silu(gate) * up, where a W slice is T gate rows and the T matching
// up rows (pygguf_engine/quant_kernels.py:1467-1472).
// Every wait is bounded; a wait that runs out records kStatusWaitTimedOut, every role leaves its
// loop and the block frees its tensor memory.
#include "common.cuh"
#include "tma.cuh"

namespace pe {
namespace skinny {

constexpr int BK = 64;
constexpr int kMaxStages = 16;
constexpr int kSmemBudget = 200 * 1024;
constexpr int kThreads = 192;

struct Params {
  int M, N, K;            // N counts output features (PAIR: I)
  void* y; long long ldy;
  int mode;               // 0: bfloat16, 1: float32, 2: silu(gate) * up -> bfloat16
  int pair_offset;
  int bm;                 // 64 or 128: rows of the MMA
  int bn;                 // columns of the MMA (PAIR: 2 * features per tile)
  int per_tile;           // output features per tile
  int n_tiles;
  int kbs;                // k blocks of 64 per stage (one TMA copy per operand brings them all)
  int stages, stage_bytes, x_bytes, w_bytes;   // bytes per stage
  int tmem_cols;          // two accumulators
  int* status;
};

// W[rows, K] (or x) seen as [k block][row][64]: one copy brings `kbs` k blocks of a slice of rows and
// leaves them in shared memory as `kbs` consecutive K-major swizzled tiles.  K must be a multiple of 64.
static int make_map_kblocks(CUtensorMap* map, const void* base, uint64_t K, uint64_t rows, uint64_t row_stride_elems,
                            uint32_t box_rows, uint32_t kbs) {
  tma::EncodeTiledFn fn = tma::encode_fn();
  if (fn == nullptr) return -5;
  if (((uintptr_t)base % 16) || ((row_stride_elems * 2) % 16) || box_rows > 256 || (K % BK)) return -2;
  cuuint64_t dims[3] = {BK, rows, K / BK};
  cuuint64_t strides[2] = {row_stride_elems * 2, BK * 2};
  cuuint32_t box[3] = {BK, box_rows, kbs};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}
__device__ __forceinline__ void load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(tma::smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(tma::smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(holder_smem)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
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
// 8 consecutive float32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// K-major tile, 128-byte swizzle (see gemm_umma.cu)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(Params p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ char smem_raw[];
  __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ volatile int failed;
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = p.K / BK;
  const int k_steps = (k_blocks + p.kbs - 1) / p.kbs;   // stages per tile
  // this block's tiles: blockIdx.x, + gridDim.x, ...
  const int my_tiles = p.n_tiles > (int)blockIdx.x ? (p.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const long long my_units = (long long)my_tiles * k_steps;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
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
  if (warp == 1) tmem_alloc(&tmem_holder, (uint32_t)p.tmem_cols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_holder;

  if (warp == 0) {
    // ---- producer ----
    if (lane == 0) {
      auto load_w = [&](long long u, int stage) {
        const int tile = (int)blockIdx.x + (int)(u / k_steps) * (int)gridDim.x;
        const int kb = (int)(u % k_steps) * p.kbs;
        char* sw = smem + stage * p.stage_bytes + p.x_bytes;
        // a copy that reaches beyond K is filled with zeros and still counts its whole box
        tma::mbar_expect_tx(&full_bar[stage], (uint32_t)(p.x_bytes + p.w_bytes));
        if (p.mode == 2) {
          // gate rows and up rows of each k block lie side by side: [k block][gate rows | up rows][64]
          for (int j = 0; j < p.kbs; ++j) {
            char* t = sw + j * (p.w_bytes / p.kbs);
            load_3d(t, &wmap, 0, tile * p.per_tile, kb + j, &full_bar[stage]);
            load_3d(t + p.w_bytes / p.kbs / 2, &wmap, 0, p.pair_offset + tile * p.per_tile, kb + j, &full_bar[stage]);
          }
        } else {
          load_3d(sw, &wmap, 0, tile * p.per_tile, kb, &full_bar[stage]);
        }
      };
      auto load_x = [&](long long u, int stage) {
        load_3d(smem + stage * p.stage_bytes, &xmap, 0, 0, (int)(u % k_steps) * p.kbs, &full_bar[stage]);
      };
      // the first round of weight slices does not wait for the preceding kernel
      const int early = my_units < p.stages ? (int)my_units : p.stages;
      for (int i = 0; i < early; ++i) load_w(i, i);
      pdl_wait();
      for (int i = 0; i < early; ++i) load_x(i, i);
      int stage = early == p.stages ? 0 : early;
      uint32_t phase = early == p.stages ? 1 : 0;
      for (long long u = early; u < my_units && !failed; ++u) {
        if (!tma::mbar_wait(&empty_bar[stage], phase ^ 1)) {
          report(p.status, kStatusWaitTimedOut, 40, (int)blockIdx.x, (int)u);
          failed = 1;
          break;
        }
        load_w(u, stage);
        load_x(u, stage);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = instr_desc(p.bm, p.bn);
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0; it < my_tiles && !failed; ++it) {
        const int ab = it & 1;
        if (!tma::mbar_wait(&acc_empty[ab], ((it >> 1) & 1) ^ 1)) {
          report(p.status, kStatusWaitTimedOut, 41, (int)blockIdx.x, it);
          failed = 1;
          break;
        }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + ab * (p.tmem_cols / 2);
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!tma::mbar_wait(&full_bar[stage], phase)) {
            report(p.status, kStatusWaitTimedOut, 42, (int)blockIdx.x, ks);
            failed = 1;
            break;
          }
          fence_after_sync();
          const uint32_t sx = tma::smem_addr(smem + stage * p.stage_bytes);
          const uint32_t sw = sx + p.x_bytes;
          const int n_kb = min(p.kbs, k_blocks - ks * p.kbs);
          for (int j = 0; j < n_kb; ++j) {
            const uint32_t ax = sx + j * (p.x_bytes / p.kbs), aw = sw + j * (p.w_bytes / p.kbs);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16(d_tmem, smem_desc(ax + k * 32), smem_desc(aw + k * 32), idesc, (ks > 0 || j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&acc_full[ab]);
      }
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----
    pdl_wait();   // y may still be read by the preceding kernel's consumers
    const int quarter = warp & 3;
    // the row of x that this thread's TMEM lane holds (see the header for M = 64)
    const int row = p.bm == 128 ? quarter * 32 + lane : quarter * 16 + lane;
    const bool has_row = (p.bm == 128 || lane < 16) && row < p.M;
    for (int it = 0; it < my_tiles && !failed; ++it) {
      const int ab = it & 1;
      const int tile = (int)blockIdx.x + it * (int)gridDim.x;
      const int n0 = tile * p.per_tile;
      if (!tma::mbar_wait(&acc_full[ab], (it >> 1) & 1)) {
        if (lane == 0) report(p.status, kStatusWaitTimedOut, 43, tile, ab);
        failed = 1;
        break;
      }
      fence_after_sync();
      const uint32_t t_row = tmem_base + ab * (p.tmem_cols / 2) + ((uint32_t)(quarter * 32) << 16);
      for (int c = 0; c < p.per_tile; c += 8) {
        uint32_t v[8], u[8];
        tmem_ld8(t_row + c, v);
        if (p.mode == 2) tmem_ld8(t_row + p.per_tile + c, u);
        tmem_ld_wait();
        if (!has_row || n0 + c >= p.N) continue;
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float g = __uint_as_float(v[j]);
          o[j] = p.mode == 2 ? silu_mul_fast(g, __uint_as_float(u[j])) : g;
        }
        const bool whole = n0 + c + 8 <= p.N;
        if (p.mode == 1) {
          float* dst = reinterpret_cast<float*>(p.y) + (size_t)row * p.ldy + n0 + c;
          if (whole && (p.ldy % 4) == 0 && (reinterpret_cast<uintptr_t>(p.y) % 16) == 0) {
            reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
          } else {
            for (int j = 0; j < 8; ++j)
              if (n0 + c + j < p.N) dst[j] = o[j];
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)row * p.ldy + n0 + c;
          if (whole && (p.ldy % 8) == 0 && (reinterpret_cast<uintptr_t>(p.y) % 16) == 0) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
          } else {
            for (int j = 0; j < 8; ++j)
              if (n0 + c + j < p.N) dst[j] = __float2bfloat16_rn(o[j]);
          }
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&acc_empty[ab]);
    }
  }
  pdl_launch_dependents();
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace skinny
}  // namespace pe

extern "C" int pe_gemm_skinny_supported(int M, int N, int K, int pair_offset) {
  if (M < 1 || M > 128 || N < 1 || K < 64 || (K % 64)) return 0;   // whole k blocks (the copies' 3-D view needs it)
  if (pair_offset > 0 && (N % 8 || pair_offset != N)) return 0;
  return 1;
}

// The arguments of pe_gemm_umma (gemm_umma.cu); 1 <= M <= 128, K a multiple of 64.
extern "C" int pe_gemm_skinny(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
                              int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream) {
  using namespace pe::skinny;
  if (M <= 0 || N <= 0) return PE_OK;
  if (!pe_gemm_skinny_supported(M, N, K, pair_offset) || n_sms < 1) return PE_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || (ldx * 2) % 16) return PE_ERR_BAD_ARGUMENT;
  Params p;
  p.M = M; p.N = N; p.K = K; p.y = y; p.ldy = ldy; p.status = status;
  p.mode = pair_offset > 0 ? 2 : (out_f32 ? 1 : 0);
  p.pair_offset = pair_offset;
  p.bm = M <= 64 ? 64 : 128;
  // output features per tile: enough tiles for every SM, in steps of 16 (PAIR: 8, doubled in the MMA)
  const int step = pair_offset > 0 ? 8 : 16;
  const int most = pair_offset > 0 ? 128 : 256;
  int per_tile = ((N + n_sms - 1) / n_sms + step - 1) / step * step;
  if (per_tile > most) per_tile = most;
  p.per_tile = per_tile;
  p.bn = pair_offset > 0 ? 2 * per_tile : per_tile;
  p.n_tiles = (N + per_tile - 1) / per_tile;
  // k blocks per stage: few, large copies (a thread issues a copy every ~150 ns), but at least 4 stages
  int kbs = 4;
  while (kbs > 1 && (kSmemBudget - 1024) / (kbs * (p.bm + p.bn) * BK * 2) < 4) kbs /= 2;
  if (kbs > K / BK) kbs = K / BK;
  p.kbs = kbs;
  p.x_bytes = kbs * p.bm * BK * 2;
  p.w_bytes = kbs * p.bn * BK * 2;
  p.stage_bytes = p.x_bytes + p.w_bytes;   // multiples of 1,024: bm and bn are multiples of 8
  p.stages = (kSmemBudget - 1024) / p.stage_bytes;
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages < 2) return PE_ERR_UNSUPPORTED_SIZE;
  int cols = 32;
  while (cols < p.bn) cols *= 2;
  p.tmem_cols = 2 * cols;
  CUtensorMap xmap, wmap;
  const uint64_t w_rows = pair_offset > 0 ? 2ull * N : (uint64_t)N;
  int e = make_map_kblocks(&xmap, x, K, M, ldx, p.bm, kbs);
  if (e == 0) e = make_map_kblocks(&wmap, w, K, w_rows, K, per_tile, pair_offset > 0 ? 1 : kbs);
  if (e != 0) return e < 0 ? e : PE_ERR_BAD_ARGUMENT;
  const size_t smem = 1024 + (size_t)p.stages * p.stage_bytes;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  const int grid = p.n_tiles < n_sms ? p.n_tiles : n_sms;
  pe::launch(gemm_skinny_kernel, grid, kThreads, smem, stream, p, xmap, wmap);
  PE_LAUNCH_CHECK();
  return PE_OK;
}
