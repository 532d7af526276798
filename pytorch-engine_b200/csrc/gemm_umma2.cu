// y[M, N] = x[M, K] . W[N, K]^T for many rows, as gemm_umma.cu, but with two SMs on one output tile:
// tcgen05.mma.cta_group::2.  A cluster of two blocks owns a tile of 256 x 256.  Each block stages its
// own 128 rows of x and its own 128 rows of W per k block (32 KB instead of the 48 KB that a
// 128 x 256 tile of one SM needs: operand traffic from L2 into the SM is what bounds the one-SM
// kernel), the tensor cores of both SMs read both halves of W through the pair's shared memory, and
// each SM accumulates its 128 rows x 256 columns in its own tensor memory.
//
// Roles, in both blocks unless said otherwise:
//   warp 0  producer: waits for its own free stage, starts the TMA copies of its halves; the bytes of
//           both blocks are counted on the leader's (rank 0) mbarrier (cp.async.bulk.tensor with
//           .cta_group::2 may signal the peer's barrier);
//   warp 1  allocates tensor memory (both blocks together, cta_group::2); in the leader it issues the
//           MMAs and commits each stage back to both producers and each finished accumulator to both
//           epilogues (tcgen05.commit with a two-block multicast mask);
//   warps 2-5  epilogue: read their block's 128 accumulator rows, convert, store, and hand the
//           accumulator back to the leader (a remote mbarrier arrive from the second block).
// Two accumulators (2 x 256 columns) let the epilogue of one tile overlap the products of the next.
// Epilogues as in gemm_umma.cu: bfloat16, float32, or silu(gate) * up, where the leader stages 128
// gate rows of W and the second block the 128 matching up rows
// (pygguf_engine/quant_kernels.py:1467-1472).
//
// Every wait is bounded; a wait that runs out records kStatusWaitTimedOut, every role leaves its
// loop, the pair meets at a cluster barrier and frees its tensor memory.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace pe {
namespace umma2 {

constexpr int BM = 128;        // rows of x per block (the pair: 256)
constexpr int BN = 256;        // accumulator columns
constexpr int BNH = 128;       // rows of W per block
constexpr int BK = 64;
constexpr int KBS = 2;         // k blocks per stage: one 3-D TMA copy per operand brings both
constexpr int STAGES = 3;
constexpr int kTileA = BM * BK * 2, kTileB = BNH * BK * 2;   // one k block of each operand
constexpr int kBytesA = KBS * kTileA, kBytesB = KBS * kTileB, kStage = kBytesA + kBytesB;
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;

// Mode 3: the product is the fused q|k|v projection of an attention layer with head size 128, and the epilogue
// does what csrc/rope_append.cu does in a kernel of its own: per-head q/k RMSNorm, rotary encoding, q written to
// the output rows, k and v appended to the paged cache.  A 256-column tile is two whole heads and an epilogue
// thread owns a token's row of it, so everything a head needs is in that thread's lane of tensor memory.
struct RopeFuse {
  int n_heads, n_kv_heads;
  const float* q_norm_w;   // [128] or null
  const float* k_norm_w;
  float eps;
  const float* cos_table;  // [table_rows, 64] or null (no rotation)
  const float* sin_table;
  int table_rows;
  const int* token_seq; const int* token_pos; const int* seq_slot; const int* seq_qstart;
  const int* page_table; int table_stride, num_pages;
  __nv_bfloat16* k_pages; __nv_bfloat16* v_pages;   // [num_pages, n_kv_heads, 64, 128]
  int write_cache;
};

struct Params {
  int M, N, K;
  void* y; long long ldy;
  int mode;               // 0: bfloat16, 1: float32, 2: silu(gate) * up -> bfloat16, 3: q|k|v with RopeFuse
  int pair_offset;
  int m_tiles, n_tiles, n_per_tile;
  int* status;
  RopeFuse rope;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t n_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;\n" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of `addr` in the block of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// a box into this block's shared memory, its bytes counted on a barrier that may be the peer's
// The operands are seen as [k block][row][64] (K is a multiple of 64), so that one copy brings KBS k
// blocks of a slice of rows as KBS consecutive K-major swizzled tiles: a thread can issue a copy only
// every ~150 ns, which two copies per k block of 0.3 us would leave no room for.
__device__ __forceinline__ void load_3d_pair(void* dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(tma::smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr) : "memory");
}
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

__device__ __forceinline__ void tmem_alloc(uint32_t* holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(holder_smem)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// arrive on the barrier at this offset in both blocks once every MMA issued so far has completed
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(tma::smem_addr(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
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

// K-major tile, 128-byte swizzle: rows of 64 bfloat16, groups of 8 rows 1024 bytes apart (see gemm_umma.cu)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16: D float32, A and B bfloat16, both K-major, N >> 3 at [17,23), M >> 4 at [24,29); with
// cta_group::2 M counts the rows of both blocks
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_round(uint32_t bits) {
  return __bfloat162float(__float2bfloat16_rn(__uint_as_float(bits)));
}

// The epilogue of mode 3 for one token row of a 256-column tile (two heads of 128 features).  Formulas and order
// as csrc/rope_append.cu (pygguf_engine/model.py:471-474 q/k-norm before RoPE, not on v; 232-241 split-half
// rotation; 482-483 append): the accumulator is rounded to bfloat16 first (the value the projection would have
// stored), the norm's sum runs over those values, norm and rotation are one float32 computation, the result is
// rounded once.  Every thread of the warp runs every tensor-memory load; only live rows store.
__device__ __forceinline__ void rope_epilogue(const Params& p, int row, int n0, uint32_t t_row) {
  const RopeFuse& r = p.rope;
  constexpr int D = 128, HALF = 64;
  const bool live = row < p.M;
  int pos = 0;
  if (live) pos = r.token_pos[row];
  const bool rotates = r.cos_table != nullptr;
  const bool pos_ok = !rotates || (pos >= 0 && pos < r.table_rows);
  if (live && !pos_ok) report(p.status, kStatusPositionOutOfRange, row, pos, r.table_rows);
#pragma unroll 1
  for (int h = 0; h < BN / D; ++h) {
    const int col0 = n0 + h * D;
    if (col0 >= p.N) break;
    const int head = col0 / D;
    const bool is_q = head < r.n_heads;
    const bool is_k = !is_q && head < r.n_heads + r.n_kv_heads;
    const int kv_head = is_q ? 0 : (is_k ? head - r.n_heads : head - r.n_heads - r.n_kv_heads);
    const uint32_t t_head = t_row + h * D;
    const float* w = is_q ? r.q_norm_w : (is_k ? r.k_norm_w : nullptr);
    const bool wanted = is_q || r.write_cache;            // k and v of a layer that only reads a cache go nowhere
    // where the row goes: q into the output rows, k and v into their page of the cache
    __nv_bfloat16* dst = nullptr;
    if (live && pos_ok && wanted) {
      if (is_q) {
        dst = reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)row * p.ldy + col0;
      } else {
        const int seq = r.token_seq[row];
        const int slot = r.seq_slot[seq];
        const int logical = pos / kPageTokens;
        if (pos < 0 || logical >= r.table_stride) {
          report(p.status, kStatusPositionOutOfRange, row, pos, r.table_stride * kPageTokens);
        } else {
          const int page = r.page_table[(size_t)slot * r.table_stride + logical];
          if (page < 0 || page >= r.num_pages) {
            report(p.status, kStatusPageOutOfRange, row, page, r.num_pages);
          } else {
            const int off = pos % kPageTokens;
            dst = (is_k ? r.k_pages : r.v_pages) + (((size_t)page * r.n_kv_heads + kv_head) * kPageTokens + off) * D;
            // rows of the page beyond the sequence's last key must hold finite values: the sequence's last token of
            // this step clears the rest of its page when it starts the page or ends a multi-token step
            const int q_begin = r.seq_qstart[seq], q_end = r.seq_qstart[seq + 1];
            if (row + 1 == q_end && off + 1 < kPageTokens && (off == 0 || q_end - q_begin > 1)) {
              uint4* rest = reinterpret_cast<uint4*>(dst + D);
              const int n16 = (kPageTokens - 1 - off) * D / 8;
              for (int i = 0; i < n16; ++i) rest[i] = make_uint4(0, 0, 0, 0);
            }
          }
        }
      }
    }
    // the norm's scale: sum of squares over the head, in four chains added up in a fixed order
    float inv = 1.f;
    if (w != nullptr) {
      float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld32(t_head + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float x = bf16_round(v[j]);
          ss[j & 3] = fmaf(x, x, ss[j & 3]);
        }
      }
      inv = rsqrtf(((ss[0] + ss[1]) + (ss[2] + ss[3])) / (float)D + r.eps);
    }
    // features j and j + 64 together, 32 pairs at a time
#pragma unroll 1
    for (int c = 0; c < HALF; c += 32) {
      uint32_t a[32], b[32];
      __syncwarp();
      tmem_ld32(t_head + c, a);
      tmem_ld32(t_head + HALF + c, b);
      tmem_ld_wait();
      if (dst != nullptr) {
        uint32_t o1[16], o2[16];
        const bool rot = rotates && !(!is_q && !is_k);
        const float4* cs = rot ? reinterpret_cast<const float4*>(r.cos_table + (size_t)pos * HALF + c) : nullptr;
        const float4* sn = rot ? reinterpret_cast<const float4*>(r.sin_table + (size_t)pos * HALF + c) : nullptr;
        const float4* w1 = w ? reinterpret_cast<const float4*>(w + c) : nullptr;
        const float4* w2 = w ? reinterpret_cast<const float4*>(w + HALF + c) : nullptr;
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) {
          float x1[4], x2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            x1[e] = bf16_round(a[4 * q4 + e]);
            x2[e] = bf16_round(b[4 * q4 + e]);
          }
          if (w) {
            const float4 wa = w1[q4], wb = w2[q4];
            x1[0] = x1[0] * inv * wa.x; x1[1] = x1[1] * inv * wa.y; x1[2] = x1[2] * inv * wa.z; x1[3] = x1[3] * inv * wa.w;
            x2[0] = x2[0] * inv * wb.x; x2[1] = x2[1] * inv * wb.y; x2[2] = x2[2] * inv * wb.z; x2[3] = x2[3] * inv * wb.w;
          }
          float y1[4], y2[4];
          if (rot) {
            const float4 cv = cs[q4], sv = sn[q4];
            const float cc[4] = {cv.x, cv.y, cv.z, cv.w}, ss4[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              y1[e] = x1[e] * cc[e] - x2[e] * ss4[e];
              y2[e] = x2[e] * cc[e] + x1[e] * ss4[e];
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) { y1[e] = x1[e]; y2[e] = x2[e]; }
          }
          o1[2 * q4] = pack2(y1[0], y1[1]); o1[2 * q4 + 1] = pack2(y1[2], y1[3]);
          o2[2 * q4] = pack2(y2[0], y2[1]); o2[2 * q4 + 1] = pack2(y2[2], y2[3]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          reinterpret_cast<uint4*>(dst + c)[j] = make_uint4(o1[4 * j], o1[4 * j + 1], o1[4 * j + 2], o1[4 * j + 3]);
          reinterpret_cast<uint4*>(dst + HALF + c)[j] = make_uint4(o2[4 * j], o2[4 * j + 1], o2[4 * j + 2], o2[4 * j + 3]);
        }
      }
    }
  }
}

// ROPE: the instantiation that carries mode 3's epilogue (it needs 231 registers where the plain epilogues need 94;
// the plain products keep a kernel of their own).
template <bool ROPE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_umma2_kernel(Params p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap) {
  extern __shared__ char smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ volatile int failed;
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int k_blocks = p.K / BK;
  const int k_steps = (k_blocks + KBS - 1) / KBS;
  const int n_tiles_total = p.m_tiles * p.n_tiles;
  const int first_tile = (int)cluster_id_x(), tile_step = (int)n_clusters_x();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tma::mbar_init(&full_bar[s], 1);    // the leader's: one arrival (its producer), bytes of both blocks
      tma::mbar_init(&empty_bar[s], 1);   // one commit per phase, delivered to both blocks
    }
    for (int b = 0; b < 2; ++b) {
      tma::mbar_init(&acc_full[b], 1);    // one commit per phase, delivered to both blocks
      tma::mbar_init(&acc_empty[b], 8);   // the leader's: four epilogue warps of each block
    }
    failed = 0;
    tma::fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(&tmem_holder, kTmemCols);
  fence_before_sync();
  __syncthreads();
  cluster_sync();   // the peer's barriers exist before anything is sent to them
  fence_after_sync();
  const uint32_t tmem_base = tmem_holder;
  pdl_wait_block();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---- producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = first_tile; tile < n_tiles_total && !failed; tile += tile_step) {
        const int m0 = (tile % p.m_tiles) * (2 * BM) + (int)rank * BM;
        const int nt = tile / p.m_tiles;
        const int b_row = p.mode == 2 ? nt * BNH + (leader ? 0 : p.pair_offset) : nt * BN + (int)rank * BNH;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!tma::mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report(p.status, kStatusWaitTimedOut, 20, tile, ks);
            failed = 1;
            break;
          }
          char* sa = smem + stage * kStage;
          char* sb = sa + kBytesA;
          if (leader) tma::mbar_expect_tx(&full_bar[stage], 2 * kStage);
          const uint32_t bar = map_to_rank(tma::smem_addr(&full_bar[stage]), 0);
          load_3d_pair(sa, &amap, 0, m0, ks * KBS, bar);      // k blocks beyond K arrive as zeros and still count
          load_3d_pair(sb, &bmap, 0, b_row, ks * KBS, bar);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (leader only) ----
    if (leader && lane == 0) {
      const uint32_t idesc = instr_desc(2 * BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = first_tile; tile < n_tiles_total && !failed; tile += tile_step, ++it) {
        const int ab = it & 1;
        if (!tma::mbar_wait(&acc_empty[ab], ((it >> 1) & 1) ^ 1)) {
          report(p.status, kStatusWaitTimedOut, 21, tile, ab);
          failed = 1;
          break;
        }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!tma::mbar_wait(&full_bar[stage], phase)) {
            report(p.status, kStatusWaitTimedOut, 22, tile, ks);
            failed = 1;
            break;
          }
          fence_after_sync();
          const uint32_t sa = tma::smem_addr(smem + stage * kStage);
          const uint32_t sb = sa + kBytesA;
          const int n_kb = min(KBS, k_blocks - ks * KBS);
          for (int j = 0; j < n_kb; ++j)
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16_pair(d_tmem, smem_desc(sa + j * kTileA + k * 32), smem_desc(sb + j * kTileB + k * 32), idesc,
                             (ks > 0 || j > 0 || k > 0) ? 1u : 0u);
          umma_commit_both(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit_both(&acc_full[ab]);
      }
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 of their block ----
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = first_tile; tile < n_tiles_total && !failed; tile += tile_step, ++it) {
      const int ab = it & 1;
      const int m0 = (tile % p.m_tiles) * (2 * BM) + (int)rank * BM;
      const int n0 = (tile / p.m_tiles) * p.n_per_tile;
      if (!tma::mbar_wait(&acc_full[ab], (it >> 1) & 1)) {
        if (lane == 0) report(p.status, kStatusWaitTimedOut, 23, tile, ab);
        failed = 1;
        break;
      }
      fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ab * BN + ((uint32_t)(quarter * 32) << 16);
      if (ROPE) {
        rope_epilogue(p, row, n0, t_row);
      } else if (p.mode == 2) {
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
      // hand the accumulator back to the leader: one arrival per epilogue warp of either block
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(tma::smem_addr(&acc_empty[ab]), 0));
    }
  }
  // teardown: both blocks meet (neither may leave while the other still reads its shared memory or
  // signals its barriers), then the allocating warps free the tensor memory together
  fence_before_sync();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace umma2
}  // namespace pe

extern "C" int pe_gemm_umma2_supported(int M, int N, int K, int pair_offset) {
  if (M < 1 || N < 1 || K < 64 || (K % 64)) return 0;   // whole k blocks (the copies' 3-D view needs it)
  if (pair_offset > 0 && (N % 128 || pair_offset != N)) return 0;
  return 1;
}

namespace pe {
namespace umma2 {
static int launch_pair(Params p, const void* x, long long ldx, const void* w, int n_sms, cudaStream_t stream);
}
}

// The arguments of pe_gemm_umma (gemm_umma.cu); n_sms is rounded down to pairs; K a multiple of 64.
extern "C" int pe_gemm_umma2(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
                             int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream) {
  using namespace pe::umma2;
  if (M <= 0 || N <= 0) return PE_OK;
  if (!pe_gemm_umma2_supported(M, N, K, pair_offset) || n_sms < 2) return PE_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || (ldx * 2) % 16) return PE_ERR_BAD_ARGUMENT;
  Params p;
  p.M = M; p.N = N; p.K = K; p.y = y; p.ldy = ldy; p.status = status;
  p.mode = pair_offset > 0 ? 2 : (out_f32 ? 1 : 0);
  p.pair_offset = pair_offset;
  p.rope = RopeFuse();
  return launch_pair(p, x, ldx, w, n_sms, stream);
}

// 1 if pe_gemm_umma2_qkv_rope takes the layer: head size 128, the whole head rotated (or none of it).
extern "C" int pe_gemm_umma2_qkv_rope_supported(int M, int K, int n_heads, int n_kv_heads, int head_dim, int rotary_dim) {
  if (head_dim != 128 || n_heads < 1 || n_kv_heads < 0) return 0;
  if (rotary_dim != 0 && rotary_dim != head_dim) return 0;
  return pe_gemm_umma2_supported(M, (n_heads + 2 * n_kv_heads) * head_dim, K, 0);
}

// The fused q|k|v projection with the epilogue of csrc/rope_append.cu (see RopeFuse): qkv[:, :n_heads * 128] gets
// the normalised, rotated queries; keys and values go to the cache only (write_cache) and not to qkv.
// Arguments as pe_qk_norm_rope_append; rotary_dim 0 or cos_table null: no rotation.
extern "C" int pe_gemm_umma2_qkv_rope(const void* x, long long ldx, const void* w, void* qkv, long long ld, int M, int K,
                                      int n_heads, int n_kv_heads, int head_dim, const float* q_norm_w,
                                      const float* k_norm_w, float eps, const float* cos_table, const float* sin_table,
                                      int rotary_dim, int table_rows, const int* token_seq, const int* token_pos,
                                      const int* seq_slot, const int* seq_qstart, const int* page_table, int table_stride,
                                      int num_pages, void* k_pages, void* v_pages, int write_cache, int n_sms, int* status,
                                      cudaStream_t stream) {
  using namespace pe::umma2;
  if (M <= 0) return PE_OK;
  if (cos_table == nullptr) rotary_dim = 0;
  if (!pe_gemm_umma2_qkv_rope_supported(M, K, n_heads, n_kv_heads, head_dim, rotary_dim) || n_sms < 2) return PE_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || (ldx * 2) % 16 || ((uintptr_t)qkv % 16) || (ld * 2) % 16 ||
      ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || ((uintptr_t)q_norm_w % 16) || ((uintptr_t)k_norm_w % 16) ||
      ((uintptr_t)cos_table % 16) || ((uintptr_t)sin_table % 16))
    return PE_ERR_BAD_ARGUMENT;
  if (write_cache && (page_table == nullptr || k_pages == nullptr || v_pages == nullptr)) return PE_ERR_BAD_ARGUMENT;
  Params p;
  p.M = M; p.N = (n_heads + 2 * n_kv_heads) * head_dim; p.K = K; p.y = qkv; p.ldy = ld; p.status = status;
  p.mode = 3;
  p.pair_offset = 0;
  RopeFuse& r = p.rope;
  r.n_heads = n_heads; r.n_kv_heads = n_kv_heads; r.q_norm_w = q_norm_w; r.k_norm_w = k_norm_w; r.eps = eps;
  r.cos_table = rotary_dim > 0 ? cos_table : nullptr; r.sin_table = rotary_dim > 0 ? sin_table : nullptr;
  r.table_rows = table_rows; r.token_seq = token_seq; r.token_pos = token_pos; r.seq_slot = seq_slot;
  r.seq_qstart = seq_qstart; r.page_table = page_table; r.table_stride = table_stride; r.num_pages = num_pages;
  r.k_pages = (__nv_bfloat16*)k_pages; r.v_pages = (__nv_bfloat16*)v_pages; r.write_cache = write_cache;
  return launch_pair(p, x, ldx, w, n_sms, stream);
}

static int pe::umma2::launch_pair(Params p, const void* x, long long ldx, const void* w, int n_sms, cudaStream_t stream) {
  const int M = p.M, N = p.N, K = p.K, pair_offset = p.pair_offset;
  p.n_per_tile = pair_offset > 0 ? BNH : BN;
  p.m_tiles = (M + 2 * BM - 1) / (2 * BM);
  p.n_tiles = (N + p.n_per_tile - 1) / p.n_per_tile;
  CUtensorMap amap, bmap;
  const uint64_t w_rows = pair_offset > 0 ? 2ull * N : (uint64_t)N;
  int e = make_map_kblocks(&amap, x, K, M, ldx, BM, KBS);
  if (e == 0) e = make_map_kblocks(&bmap, w, K, w_rows, K, BNH, KBS);
  if (e != 0) return e < 0 ? e : PE_ERR_BAD_ARGUMENT;
  const size_t smem = 1024 + (size_t)STAGES * kStage;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_umma2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce == cudaSuccess)
      ce = cudaFuncSetAttribute(gemm_umma2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  const int pairs = tiles < n_sms / 2 ? tiles : n_sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pe::pdl_enabled() ? 2 : 1;
  cudaError_t ce = p.mode == 3 ? cudaLaunchKernelEx(&cfg, gemm_umma2_kernel<true>, p, amap, bmap)
                               : cudaLaunchKernelEx(&cfg, gemm_umma2_kernel<false>, p, amap, bmap);
  if (ce != cudaSuccess) return (int)ce;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
