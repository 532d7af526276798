// Causal grouped-query attention over the paged bfloat16 cache on the tensor cores (mma.sync
// m16n8k16, float32 accumulation), for head sizes 64 and 128 and groups of up to 16 query heads.
// Other shapes and the float32 mode use attention_generic.cu.
//
// Formulas as in attention_generic.cu (pygguf_engine/kv_cache.py:833, 2189-2192 masks; 756 head
// mapping; 836-861 online softmax; 273-282 merge of partial results).  Scores, the softmax state
// (m, l) and the output accumulator are float32; the probabilities are rounded to bfloat16 only as
// the tensor-core operand of the P.V product.
//
// Rows.  For one kv head, a "row" is a (query token, query head of the group) pair: row r is token
// r / group, head r % group.  All rows of a kv head share its keys and values, so the group's heads
// ride along in the M dimension of the MMA instead of re-reading K and V.
//   prefill: a block of 4 warps owns 64 consecutive rows of one (sequence, kv head) and walks the
//            64-key pages of that sequence up to its last row's position; each warp owns 16 rows.
//            K/V pages are double-buffered in shared memory.
//   decode:  one token per sequence, so a kv head has `group` rows (<= 16: one MMA row block).  A block
//            owns one (sequence, kv head, range of `split_keys` keys); its 4 warps each take 16 keys of
//            every 64-key page and are merged at the end; a second kernel merges the ranges.  Which
//            keys a partial result covers depends only on the sequence's own length.
// K/V pages travel from the cache to shared memory by TMA (cp.async.bulk.tensor, one elected thread,
// completion counted on an mbarrier): a page of one kv head is a [64 keys][head_dim] box of a 2-D
// tensor map over the layer's pages, split into 64-feature (128-byte) sub-tiles with the 128-byte
// swizzle, i.e. the 16-byte chunks of a row are XOR-ed with (row & 7).  That makes both the row-wise
// (K) and the transposed (V) ldmatrix reads conflict-free.  Rows of a page beyond the sequence's
// length are not read as zeros: the cache never holds a non-finite value there (the append kernel
// clears the rest of a page when it starts one), and their probabilities are exactly zero.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace pe {
namespace fa {

constexpr int BN = 64;  // keys per tile = one cache page

struct Args {
  const __nv_bfloat16* q; long long q_ld;
  __nv_bfloat16* out;     long long out_ld;
  int n_heads, n_kv_heads, group;
  float scale_log2;       // softmax scale * log2(e)
  int window;
  const int* seq_qstart; const int* seq_past; const int* seq_slot;
  const int* page_table; int table_stride; int num_pages;
  const __nv_bfloat16* k_pages; const __nv_bfloat16* v_pages;
  int* status;
  float* part_acc; float* part_lse; int split_keys, max_splits, min_range_keys;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (one instruction, about 2 ulp; exp2(-inf) = 0): the result is
// rounded to bfloat16 or summed into a float32 denominator, so this is within the path's precision.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of 16-byte chunk `chunk` of row `row` in a [ROWS][HD] bfloat16 tile stored as
// HD/64 sub-tiles of [ROWS][64] with the 128-byte swizzle (the layout TMA writes)
template <int HD, int ROWS = BN> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// One elected thread starts the copy of one page (64 keys of kv head `kvh`) of K and V into a stage;
// `bar` counts the bytes.
template <int HD>
__device__ __forceinline__ void issue_page(const Args& a, const CUtensorMap* kmap, const CUtensorMap* vmap, int slot,
                                           int kvh, int k0, char* stage, uint64_t* bar) {
  const int logical = k0 / BN;
  int page = -1;
  if (logical < a.table_stride) page = a.page_table[(size_t)slot * a.table_stride + logical];
  if (page < 0 || page >= a.num_pages) {
    report(a.status, kStatusPageOutOfRange, slot, page, k0);
    page = 0;
  }
  const int y = (page * a.n_kv_heads + kvh) * BN;
  tma::mbar_expect_tx(bar, 2 * BN * HD * 2);
#pragma unroll
  for (int sub = 0; sub < HD / 64; ++sub) {
    tma::load_2d(stage + sub * (BN * 128), kmap, sub * 64, y, bar);
    tma::load_2d(stage + BN * HD * 2 + sub * (BN * 128), vmap, sub * 64, y, bar);
  }
}

// A wait ran out: record it, give copies still in flight a last bounded chance to land, and leave.
__device__ __forceinline__ void give_up(const Args& a, uint64_t* bars, int n_bars, int where) {
  if (threadIdx.x == 0) report(a.status, kStatusWaitTimedOut, where, blockIdx.x, blockIdx.z);
  for (int s = 0; s < n_bars; ++s)
    for (int i = 0; i < 1000; ++i)
      if (tma::mbar_try_wait(&bars[s], 0) || tma::mbar_try_wait(&bars[s], 1)) break;
}

__device__ __forceinline__ char* align_1024(char* p) {
  return reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

// ---- prefill ---------------------------------------------------------------------------------------
// grid: (row tiles of 64, n_kv_heads, n_seqs); block: 128 threads.
template <int HD>
__global__ void __launch_bounds__(128, 3) prefill_kernel(Args a, const __grid_constant__ CUtensorMap kmap,
                                                      const __grid_constant__ CUtensorMap vmap) {
  extern __shared__ char smem_raw[];
  __shared__ uint64_t bars[2];
  pdl_wait_block();
  pdl_launch_dependents();
  char* smem = align_1024(smem_raw);
  constexpr int STAGE = 2 * BN * HD * 2;      // K and V tile
  constexpr int KS = HD / 16;                 // k-steps of Q.K^T
  constexpr int NO = HD / 8;                  // n-tiles of the output
  // Q is staged in the second K/V stage: its fragments are in registers before that stage is first filled
  char* q_s = smem + STAGE;                   // [64][HD] swizzled
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int q0 = a.seq_qstart[b], q_len = a.seq_qstart[b + 1] - q0, past = a.seq_past[b];
  const int group = a.group;
  const int n_rows = q_len * group;
  // late rows see the most keys: they go first, so that the longest blocks do not form the tail
  const int row0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * 64;
  if (row0 >= n_rows) return;
  const int slot = a.seq_slot[b];
  const int last_row = min(n_rows, row0 + 64) - 1;
  const int first_pos = past + row0 / group, last_pos = past + last_row / group;
  int k_begin = 0;
  if (a.window > 0) k_begin = max(0, first_pos - a.window + 1) / BN * BN;
  const int k_end = last_pos + 1;
  const int n_tiles = (k_end - k_begin + BN - 1) / BN;

  // first K/V page in flight, then stage Q
  if (tid == 0) {
    tma::mbar_init(&bars[0], 1);
    tma::mbar_init(&bars[1], 1);
    tma::fence_barrier_init();
    issue_page<HD>(a, &kmap, &vmap, slot, kvh, k_begin, smem, &bars[0]);
  }
  constexpr int CPR = HD / 8;
  for (int i = tid; i < 64 * CPR; i += 128) {
    const int r = i / CPR, chunk = i % CPR;
    const int row = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n_rows) {
      const int tok = row / group, head = kvh * group + row % group;
      v = *reinterpret_cast<const uint4*>(a.q + (size_t)(q0 + tok) * a.q_ld + (size_t)head * HD + chunk * 8);
    }
    *reinterpret_cast<uint4*>(q_s + tile_off<HD>(r, chunk)) = v;
  }
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    ldmatrix_x4(qf[ks], smem_u32(q_s) + tile_off<HD>(r, ks * 2 + (lane >> 4)));
  }
  __syncthreads();  // every warp has its Q fragments: the stage that held Q may now be filled with keys
  // this thread's two rows
  const int r_lo = row0 + warp * 16 + g, r_hi = r_lo + 8;
  const int pos_lo = past + r_lo / group, pos_hi = past + r_hi / group;   // rows beyond n_rows are never stored
  const int warp_last_pos = past + min(n_rows - 1, row0 + warp * 16 + 15) / group;
  const int warp_first_pos = past + min(n_rows - 1, row0 + warp * 16) / group;
  float o[NO][4];
#pragma unroll
  for (int n = 0; n < NO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    const int k0 = k_begin + it * BN;
    char* stage = smem + (it & 1) * STAGE;
    // next page into the other stage (everyone left it at the end of the last round)
    if (tid == 0 && it + 1 < n_tiles)
      issue_page<HD>(a, &kmap, &vmap, slot, kvh, k0 + BN, smem + ((it + 1) & 1) * STAGE, &bars[(it + 1) & 1]);
    if (!tma::mbar_wait(&bars[it & 1], (it >> 1) & 1)) {
      give_up(a, bars, 2, 1);
      return;
    }
    const bool skip = (k0 > warp_last_pos) || (a.window > 0 && k0 + BN - 1 <= warp_first_pos - a.window);
    if (!skip) {
      const uint32_t ks_base = smem_u32(stage), vs_base = ks_base + BN * HD * 2;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {  // pairs of 8-key n-tiles
          uint32_t kb[4];
          const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
          ldmatrix_x4(kb, ks_base + tile_off<HD>(key, ks * 2 + ((lane >> 3) & 1)));
          mma_bf16(s[np * 2], qf[ks], kb[0], kb[1]);
          mma_bf16(s[np * 2 + 1], qf[ks], kb[2], kb[3]);
        }
      }
      // scale, mask, running max
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
      // a page that lies wholly in the past of every row of this warp (and inside every window) needs no mask
      const bool full = (k0 + BN - 1 <= warp_first_pos) && (a.window <= 0 || k0 > warp_last_pos - a.window);
      if (full) {
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = s[n][e] * a.scale_log2;
            s[n][e] = v;
            if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
          }
        }
      } else {
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int kpos = k0 + n * 8 + 2 * t + (e & 1);
            const int qpos = (e < 2) ? pos_lo : pos_hi;
            bool vis = kpos <= qpos;
            if (a.window > 0) vis = vis && (kpos > qpos - a.window);
            const float v = vis ? s[n][e] * a.scale_log2 : -INFINITY;
            s[n][e] = v;
            if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
          }
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float al_lo = (m_lo == -INFINITY) ? 0.f : fast_exp2(m_lo - mn_lo);
      const float al_hi = (m_hi == -INFINITY) ? 0.f : fast_exp2(m_hi - mn_hi);
      const float base_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, base_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
      uint32_t pf[4][4];  // P as A operand: 4 k-steps of 16 keys
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float p0 = fast_exp2(s[n][0] - base_lo), p1 = fast_exp2(s[n][1] - base_lo);
        const float p2 = fast_exp2(s[n][2] - base_hi), p3 = fast_exp2(s[n][3] - base_hi);
        sum_lo += p0 + p1;
        sum_hi += p2 + p3;
        pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
      l_lo = l_lo * al_lo + sum_lo;
      l_hi = l_hi * al_hi + sum_hi;
      m_lo = mn_lo;
      m_hi = mn_hi;
#pragma unroll
      for (int n = 0; n < NO; ++n) {
        o[n][0] *= al_lo; o[n][1] *= al_lo; o[n][2] *= al_hi; o[n][3] *= al_hi;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {       // 16 keys per step
#pragma unroll
        for (int np = 0; np < NO / 2; ++np) {  // pairs of 8-feature n-tiles
          uint32_t vb[4];
          const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(vb, vs_base + tile_off<HD>(key, np * 2 + (lane >> 4)));
          mma_bf16(o[np * 2], pf[kk], vb[0], vb[1]);
          mma_bf16(o[np * 2 + 1], pf[kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();  // the stage may be overwritten in the next round
  }
  const float inv_lo = 1.f / fmaxf(l_lo, 1e-20f), inv_hi = 1.f / fmaxf(l_hi, 1e-20f);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? r_hi : r_lo;
    if (row >= n_rows) continue;
    const int tok = row / group, head = kvh * group + row % group;
    __nv_bfloat16* dst = a.out + (size_t)(q0 + tok) * a.out_ld + (size_t)head * HD;
    const float inv = half ? inv_hi : inv_lo;
#pragma unroll
    for (int n = 0; n < NO; ++n) {
      const uint32_t v = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = v;
    }
  }
}

// One warp folds its 16 keys (key0 .. key0+15 of the page that starts at position k0) into the
// running softmax state of the group's rows.  Keys outside [k_first, k_hi) are masked.
template <int HD>
__device__ __forceinline__ void decode_fold_page(uint32_t ks_base, uint32_t vs_base, int key0, int k0, int k_first,
                                                 int k_hi, float scale_log2, const uint32_t (&qf)[HD / 16][4],
                                                 float (&o)[HD / 8][4], float& m_lo, float& m_hi, float& l_lo,
                                                 float& l_hi, int lane) {
  constexpr int KS = HD / 16;
  constexpr int NO = HD / 8;
  const int t = lane & 3;
    if (k0 + key0 < k_hi && k0 + key0 + 15 >= k_first) {
  float s[2][4];
  s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    uint32_t kb[4];
    const int key = key0 + (lane & 7) + (lane >> 4) * 8;
    ldmatrix_x4(kb, ks_base + tile_off<HD>(key, ks * 2 + ((lane >> 3) & 1)));
    mma_bf16(s[0], qf[ks], kb[0], kb[1]);
    mma_bf16(s[1], qf[ks], kb[2], kb[3]);
  }
  float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kpos = k0 + key0 + n * 8 + 2 * t + (e & 1);
      const bool vis = kpos >= k_first && kpos < k_hi;
      const float v = vis ? s[n][e] * scale_log2 : -INFINITY;
      s[n][e] = v;
      if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
    }
  }
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
  const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
  const float al_lo = (m_lo == -INFINITY) ? 0.f : fast_exp2(m_lo - mn_lo);
  const float al_hi = (m_hi == -INFINITY) ? 0.f : fast_exp2(m_hi - mn_hi);
  const float base_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, base_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
  const float p00 = fast_exp2(s[0][0] - base_lo), p01 = fast_exp2(s[0][1] - base_lo);
  const float p02 = fast_exp2(s[0][2] - base_hi), p03 = fast_exp2(s[0][3] - base_hi);
  const float p10 = fast_exp2(s[1][0] - base_lo), p11 = fast_exp2(s[1][1] - base_lo);
  const float p12 = fast_exp2(s[1][2] - base_hi), p13 = fast_exp2(s[1][3] - base_hi);
  float sum_lo = p00 + p01 + p10 + p11, sum_hi = p02 + p03 + p12 + p13;
  sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
  sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
  sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
  sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
  l_lo = l_lo * al_lo + sum_lo;
  l_hi = l_hi * al_hi + sum_hi;
  m_lo = mn_lo;
  m_hi = mn_hi;
  uint32_t pf[4];
  pf[0] = pack_bf16(p00, p01); pf[1] = pack_bf16(p02, p03); pf[2] = pack_bf16(p10, p11); pf[3] = pack_bf16(p12, p13);
#pragma unroll
  for (int n = 0; n < NO; ++n) {
    o[n][0] *= al_lo; o[n][1] *= al_lo; o[n][2] *= al_hi; o[n][3] *= al_hi;
  }
#pragma unroll
  for (int np = 0; np < NO / 2; ++np) {
    uint32_t vb[4];
    const int key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8;
    ldmatrix_x4_trans(vb, vs_base + tile_off<HD>(key, np * 2 + (lane >> 4)));
    mma_bf16(o[np * 2], pf, vb[0], vb[1]);
    mma_bf16(o[np * 2 + 1], pf, vb[2], vb[3]);
  }
}
}

// ---- decode ------------------------------------------------------------------------------------------
// Keys per range of a sequence of `len` keys: the fixed split_keys, or (split_keys == 0) the
// sequence's own length shared out evenly over max_splits ranges, in whole pages, but no fewer than
// min_range_keys.  With even shares a grid sized for the longest possible sequence keeps all its
// blocks busy on shorter ones; the floor keeps a short sequence in a grid sized for a much longer
// one from being cut into ranges of a page or two (its spare blocks return at once).
__device__ __forceinline__ int range_keys(const Args& a, int len) {
  if (a.split_keys > 0) return a.split_keys;
  const int per = (len + a.max_splits - 1) / a.max_splits;
  return max(max(BN, a.min_range_keys), (per + BN - 1) / BN * BN);
}

// grid: (max_splits, n_kv_heads, n_seqs); block: 128 threads; STAGES pages in flight.
template <int HD, int STAGES>
__global__ void __launch_bounds__(128) decode_split_kernel(Args a, const __grid_constant__ CUtensorMap kmap,
                                                           const __grid_constant__ CUtensorMap vmap) {
  extern __shared__ char smem_raw[];
  __shared__ uint64_t bars[STAGES];
  // The batch description and every page but the sequence's last were written before the kernel that
  // precedes this one started, so they may be read before the dependency wait; the last page (it gets
  // this step's key) and the queries come from that kernel and are read after it.
  char* smem = align_1024(smem_raw);
  constexpr int STAGE = 2 * BN * HD * 2;
  constexpr int KS = HD / 16;
  constexpr int NO = HD / 8;
  char* q_s = smem + STAGES * STAGE;  // [16][HD] swizzled
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int b = blockIdx.z, kvh = blockIdx.y, split = blockIdx.x;
  const int group = a.group;
  const int tq = a.seq_qstart[b];
  const int len = a.seq_past[b] + 1;
  const int per_range = range_keys(a, len);
  const int k_lo = split * per_range, k_hi = min(len, k_lo + per_range);
  if (k_lo >= len) return;
  const int win_lo = a.window > 0 ? max(0, len - a.window) : 0;
  if (k_hi <= win_lo) return;
  const int slot = a.seq_slot[b];
  const int k_first = max(k_lo, win_lo);         // first visible key of this range
  const int k_begin = k_first / BN * BN;
  const int n_tiles = (k_hi - k_begin + BN - 1) / BN;
  const int last_page_k0 = (len - 1) / BN * BN;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) tma::mbar_init(&bars[s], 1);
    tma::fence_barrier_init();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
      if (s < n_tiles && k_begin + s * BN != last_page_k0)
        issue_page<HD>(a, &kmap, &vmap, slot, kvh, k_begin + s * BN, smem + s * STAGE, &bars[s]);
  }
  pdl_wait_block();
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
      if (s < n_tiles && k_begin + s * BN == last_page_k0)
        issue_page<HD>(a, &kmap, &vmap, slot, kvh, k_begin + s * BN, smem + s * STAGE, &bars[s]);
  }
  constexpr int CPR = HD / 8;
  for (int i = tid; i < 16 * CPR; i += 128) {
    const int r = i / CPR, chunk = i % CPR;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < group) v = *reinterpret_cast<const uint4*>(a.q + (size_t)tq * a.q_ld + (size_t)(kvh * group + r) * HD + chunk * 8);
    *reinterpret_cast<uint4*>(q_s + tile_off<HD, 16>(r, chunk)) = v;
  }
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
    ldmatrix_x4(qf[ks], smem_u32(q_s) + tile_off<HD, 16>(r, ks * 2 + (lane >> 4)));
  }
  float o[NO][4];
#pragma unroll
  for (int n = 0; n < NO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    // keep STAGES-1 pages in flight (the stage refilled here was released by the last round's barrier)
    const int nxt = it + STAGES - 1;
    if (tid == 0 && nxt < n_tiles)
      issue_page<HD>(a, &kmap, &vmap, slot, kvh, k_begin + nxt * BN, smem + (nxt % STAGES) * STAGE, &bars[nxt % STAGES]);
    if (!tma::mbar_wait(&bars[it % STAGES], (it / STAGES) & 1)) {
      give_up(a, bars, STAGES, 2);
      return;
    }
    const int k0 = k_begin + it * BN;
    decode_fold_page<HD>(smem_u32(smem + (it % STAGES) * STAGE), smem_u32(smem + (it % STAGES) * STAGE) + BN * HD * 2,
                         warp * 16, k0, k_first, k_hi, a.scale_log2, qf, o, m_lo, m_hi, l_lo, l_hi, lane);
    __syncthreads();
  }
  pdl_launch_dependents();
  // merge the four warps (fixed order) through shared memory laid over the stages
  float* ml = reinterpret_cast<float*>(smem);            // [4 warps][16 rows][2]
  float* acc = ml + 4 * 16 * 2;                          // [4 warps][16 rows][HD]
  if (t == 0) {
    ml[(warp * 16 + g) * 2] = m_lo;     ml[(warp * 16 + g) * 2 + 1] = l_lo;
    ml[(warp * 16 + g + 8) * 2] = m_hi; ml[(warp * 16 + g + 8) * 2 + 1] = l_hi;
  }
#pragma unroll
  for (int n = 0; n < NO; ++n) {
    float* r0 = acc + (size_t)(warp * 16 + g) * HD + n * 8 + 2 * t;
    float* r1 = acc + (size_t)(warp * 16 + g + 8) * HD + n * 8 + 2 * t;
    r0[0] = o[n][0]; r0[1] = o[n][1];
    r1[0] = o[n][2]; r1[1] = o[n][3];
  }
  __syncthreads();
  for (int i = tid; i < group * HD; i += 128) {
    const int r = i / HD, c = i - r * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml[(w * 16 + r) * 2]);
    float ll = 0.f, aa = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = ml[(w * 16 + r) * 2];
        const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mm);
        ll += ml[(w * 16 + r) * 2 + 1] * f;
        aa += acc[(size_t)(w * 16 + r) * HD + c] * f;
      }
    }
    const size_t pidx = ((size_t)b * a.n_heads + (kvh * group + r)) * a.max_splits + split;
    a.part_acc[pidx * HD + c] = (ll > 0.f) ? aa / ll : 0.f;
    // log-sum-exp in natural units, as the merge kernel expects: (m + log2 l) * ln 2
    if (c == 0) a.part_lse[pidx] = (ll > 0.f) ? (mm + log2f(ll)) * 0.6931471805599453f : -INFINITY;
  }
}

// grid: (n_heads, n_seqs): merge the ranges of one (sequence, head) (pygguf_engine/kv_cache.py:273-282).
template <int HD>
__global__ void decode_merge_kernel(Args a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y, h = blockIdx.x;
  const int tq = a.seq_qstart[b];
  const int len = a.seq_past[b] + 1;
  const int per_range = range_keys(a, len);
  int n_splits = (len + per_range - 1) / per_range;
  if (n_splits > a.max_splits) {
    // only with a fixed split_keys: the sequence is longer than split_keys * max_splits keys, for which the
    // split grid has no blocks and the scratch no room; say so and merge what was computed
    if (threadIdx.x == 0) report(a.status, kStatusPositionOutOfRange, b, len - 1, per_range * a.max_splits);
    n_splits = a.max_splits;
  }
  const int win_lo = a.window > 0 ? max(0, len - a.window) : 0;
  const int first = min(win_lo / per_range, n_splits);
  const size_t base = ((size_t)b * a.n_heads + h) * a.max_splits;
  __nv_bfloat16* o = a.out + (size_t)tq * a.out_ld + (size_t)h * HD;
  // Ranges are taken eight at a time: all their loads are issued before the first is used (this kernel
  // is short and a decode step waits for it once per layer), then they are folded into a running
  // maximum, denominator and sum, in range order.
  constexpr int G = 8;
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float mx = -INFINITY, denom = 0.f, v = 0.f;
    for (int s0 = first; s0 < n_splits; s0 += G) {
      float e[G], acc[G];
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const bool live = s0 + i < n_splits;
        e[i] = live ? a.part_lse[base + s0 + i] : -INFINITY;
        acc[i] = live ? a.part_acc[(base + s0 + i) * HD + c] : 0.f;
      }
      float m_new = mx;
#pragma unroll
      for (int i = 0; i < G; ++i) m_new = fmaxf(m_new, e[i]);
      if (m_new == -INFINITY) continue;
      const float keep = (mx == -INFINITY) ? 0.f : expf(mx - m_new);
      denom *= keep;
      v *= keep;
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const float w = (e[i] == -INFINITY) ? 0.f : expf(e[i] - m_new);
        denom += w;
        v = fmaf(w, acc[i], v);
      }
      mx = m_new;
    }
    o[c] = __float2bfloat16_rn(v / fmaxf(denom, 1e-20f));
  }
}

template <typename K>
static int opt_in(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

template <int HD>
static int launch(const Args& a, bool decode, int n_seqs, int max_q, cudaStream_t stream) {
  constexpr int STAGE = 2 * BN * HD * 2;
  CUtensorMap kmap, vmap;
  const uint64_t rows = (uint64_t)a.num_pages * a.n_kv_heads * BN;
  int me = tma::make_map_2d_bf16(&kmap, a.k_pages, HD, rows, HD, 64, BN);
  if (me == 0) me = tma::make_map_2d_bf16(&vmap, a.v_pages, HD, rows, HD, 64, BN);
  if (me != 0) return me < 0 ? me : PE_ERR_BAD_ARGUMENT;
  if (!decode) {
    const size_t smem = 1024 + 2 * STAGE;
    auto k = prefill_kernel<HD>;
    int e = opt_in(k, smem);
    if (e) return e;
    const long long tiles = ((long long)max_q * a.group + 63) / 64;
    dim3 grid((unsigned)tiles, a.n_kv_heads, n_seqs);
    if (grid.y > 65535 || grid.z > 65535) return PE_ERR_UNSUPPORTED_SIZE;
    pe::launch(k, grid, 128, smem, stream, a, kmap, vmap);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
  dim3 grid(a.max_splits, a.n_kv_heads, n_seqs);
  if (grid.y > 65535 || grid.z > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  auto go = [&](auto kern, int STAGES) -> int {
    size_t smem = STAGES * STAGE + 16 * HD * 2;
    const size_t merge = (4 * 16 * 2 + 4 * 16 * HD) * sizeof(float);
    if (merge > smem) smem = merge;
    smem += 1024;
    int e = opt_in(kern, smem);
    if (e) return e;
    pe::launch(kern, grid, 128, smem, stream, a, kmap, vmap);
    return 0;
  };
  // three stages: two blocks per SM, two pages in flight per block (measured best of 2, 3, 4)
  const int e = go(decode_split_kernel<HD, 3>, 3);
  if (e) return e;
  PE_LAUNCH_CHECK();
  // The merge starts when the split kernel has completed, not while it drains: with the early start a
  // decode step of the 8B shape took 4.32 instead of 4.03 ms at batch 8 and context 4,096 (3.59 / 3.49 ms
  // at 1,024, 4.92 / 4.74 at 8,192, 3.95 / 3.56 for 16 layers of the 32B shape), and never less, at batch
  // 1 to 64.  Why its waiting blocks cost that much is not known; switching the early start off for any
  // other kernel of the step gained nothing or lost.
  dim3 mgrid(a.n_heads, n_seqs);
  pe::launch_after(decode_merge_kernel<HD>, mgrid, HD >= 128 ? 128 : 64, 0, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

}  // namespace fa
}  // namespace pe

// Decode blocks that one SM holds at a time (shared memory bound): the caller sizes the number of
// ranges per sequence so that one wave of blocks covers the batch.
extern "C" int pe_attention_mma_decode_blocks_per_sm(int head_dim) {
  const size_t stage = 2 * (size_t)pe::fa::BN * head_dim * 2;
  const size_t smem = 3 * stage + 16 * (size_t)head_dim * 2 + 1024 + 1024;   // + the block's static and reserved part
  const int n = (int)((227 * 1024) / smem);
  return n < 1 ? 1 : n;
}

// 1 if this file's kernels take the shape (bfloat16 only), else 0: the caller then uses the generic path.
extern "C" int pe_attention_mma_supported(int head_dim, int n_heads, int n_kv_heads) {
  if (head_dim != 64 && head_dim != 128) return 0;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
  if (n_heads / n_kv_heads > 16) return 0;
  return 1;
}

extern "C" int pe_attention_mma(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs,
                                int max_q, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                const int* seq_qstart, const int* seq_past, const int* seq_slot, const int* page_table,
                                int table_stride, int num_pages, const void* k_pages, const void* v_pages,
                                float* scratch, int split_keys, int max_splits, int min_range_keys, int* status,
                                cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (!pe_attention_mma_supported(head_dim, n_heads, n_kv_heads)) return PE_ERR_UNSUPPORTED_SIZE;
  // 16-byte vector loads of q rows
  if ((q_ld * 2) % 16 || ((uintptr_t)q % 16) || (out_ld * 2) % 4 || ((uintptr_t)out % 4)) return PE_ERR_BAD_ARGUMENT;
  if (((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16)) return PE_ERR_BAD_ARGUMENT;
  pe::fa::Args a;
  a.q = (const __nv_bfloat16*)q; a.q_ld = q_ld; a.out = (__nv_bfloat16*)out; a.out_ld = out_ld;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.group = n_heads / n_kv_heads;
  a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
  a.seq_qstart = seq_qstart; a.seq_past = seq_past; a.seq_slot = seq_slot;
  a.page_table = page_table; a.table_stride = table_stride; a.num_pages = num_pages;
  a.k_pages = (const __nv_bfloat16*)k_pages; a.v_pages = (const __nv_bfloat16*)v_pages; a.status = status;
  a.part_acc = nullptr; a.part_lse = nullptr; a.split_keys = 0; a.max_splits = 0; a.min_range_keys = 0;
  if (decode) {
    if (!scratch || split_keys < 0 || split_keys % pe::fa::BN || max_splits <= 0) return PE_ERR_BAD_ARGUMENT;
    if (min_range_keys < 0 || min_range_keys % pe::fa::BN) return PE_ERR_BAD_ARGUMENT;
    a.split_keys = split_keys; a.max_splits = max_splits; a.min_range_keys = min_range_keys;
    a.part_acc = scratch;
    a.part_lse = scratch + (size_t)n_seqs * n_heads * max_splits * head_dim;
  }
  if (head_dim == 64) return pe::fa::launch<64>(a, decode != 0, n_seqs, max_q, stream);
  return pe::fa::launch<128>(a, decode != 0, n_seqs, max_q, stream);
}
