// Causal grouped-query attention over the paged cache, for every head size, group size and
// window, in float32 arithmetic (inputs float32 or bfloat16).  This is the exact path (the whole
// model in float32 runs through it) and the fallback for head sizes the tensor-core kernels refuse.
//
// Reference formulas: scores q.k * scale; key visible iff kpos <= qpos (pygguf_engine/kv_cache.py:833,
// 2192) and, with a window, kpos > qpos - window (2189-2190); query head h reads kv head h / group
// (756); online softmax m, l, acc in float32 (836-861, 2292-2305); split merge by log-sum-exp
// weights (273-282).
//
// Work split.  One warp owns one query token and up to 4 query heads of one kv head; lane j of the
// warp owns key j of the current 32-key tile for the scores and output features {lane, lane+32, ..}
// for the accumulation.  Prefill: a block of 8 warps (8 consecutive tokens of one sequence) shares
// each K/V tile through shared memory.  Decode: a block owns one (sequence, kv head, key range of
// `split_keys` positions); its warps take the 32-key tiles of the range in turn and merge at the
// end; a second kernel merges the ranges.  Which keys a partial result covers depends only on the
// sequence's own length, never on what else is in the batch.
#include "api.h"
#include "common.cuh"

namespace pe {

constexpr int kGT = 4;        // query heads per warp
constexpr int kTileKeys = 32; // keys per tile (one per lane)

struct AttnArgs {
  const void* q;  long long q_ld;     // token t, head h: q + t*q_ld + h*head_dim
  void* out;      long long out_ld;
  int n_heads, n_kv_heads, head_dim;
  float scale;
  int window;                         // <= 0: none
  const int* seq_qstart;              // [n_seqs + 1]
  const int* seq_past;                // [n_seqs] cached length before this step
  const int* seq_slot;                // [n_seqs]
  const int* page_table; int table_stride; int num_pages;
  const void* k_pages; const void* v_pages;   // [num_pages, n_kv_heads, 64, head_dim]
  int* status;
  // decode only
  float* part_acc;                    // [n_seqs, n_heads, max_splits, head_dim]
  float* part_lse;                    // [n_seqs, n_heads, max_splits]
  int split_keys, max_splits;
};

// Load keys [k0, k0+32) of kv head `kvh` of sequence slot `slot` into shared memory as float32.
// Rows at or beyond k_end are filled with zeros.  `nthreads` threads starting at `tid` cooperate.
template <typename T>
__device__ __forceinline__ void load_tile(const AttnArgs& a, int slot, int kvh, int k0, int k_end, float* Ks,
                                          float* Vs, int tid, int nthreads) {
  const int d = a.head_dim;
  const int logical = k0 / kPageTokens;
  int page = -1;
  if (logical < a.table_stride) page = a.page_table[(size_t)slot * a.table_stride + logical];
  const bool ok = page >= 0 && page < a.num_pages;
  if (!ok && tid == 0 && k0 < k_end) report(a.status, kStatusPageOutOfRange, slot, page, k0);
  const size_t base = (((size_t)(ok ? page : 0) * a.n_kv_heads + kvh) * kPageTokens + (k0 % kPageTokens)) * d;
  const T* kp = (const T*)a.k_pages + base;
  const T* vp = (const T*)a.v_pages + base;
  const int total = kTileKeys * d;
  for (int i = tid; i < total; i += nthreads) {
    const int r = i / d, c = i - r * d;
    const bool live = ok && (k0 + r) < k_end;
    Ks[r * (d + 1) + c] = live ? to_f32<T>(kp[i]) : 0.f;
    Vs[r * d + c] = live ? to_f32<T>(vp[i]) : 0.f;
  }
}

// One warp: fold the 32 keys of the tile in shared memory into (m, l, acc) of its query heads.
// `visible` says whether this lane's key takes part for this warp's query.
template <int DPL>
__device__ __forceinline__ void fold_tile(const float* qs /*[kGT][d]*/, const float* Ks, const float* Vs, int d,
                                          int n_heads_here, float scale, bool visible, int lane, float (&m)[kGT],
                                          float (&l)[kGT], float (&acc)[kGT][DPL]) {
  float s[kGT];
#pragma unroll
  for (int h = 0; h < kGT; ++h) s[h] = 0.f;
  const float* krow = Ks + lane * (d + 1);
  for (int c = 0; c < d; ++c) {
    const float kv = krow[c];
#pragma unroll
    for (int h = 0; h < kGT; ++h) s[h] = fmaf(qs[h * d + c], kv, s[h]);
  }
  float p[kGT];
#pragma unroll
  for (int h = 0; h < kGT; ++h) {
    const float sc = (visible && h < n_heads_here) ? s[h] * scale : -INFINITY;
    const float m_new = fmaxf(m[h], warp_max(sc));
    if (m_new == -INFINITY) {  // nothing visible yet for this head
      p[h] = 0.f;
      continue;
    }
    const float alpha = (m[h] == -INFINITY) ? 0.f : expf(m[h] - m_new);
    p[h] = (sc == -INFINITY) ? 0.f : expf(sc - m_new);
    l[h] = l[h] * alpha + warp_sum(p[h]);
    m[h] = m_new;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[h][i] *= alpha;
  }
  for (int j = 0; j < kTileKeys; ++j) {
    float pj[kGT];
#pragma unroll
    for (int h = 0; h < kGT; ++h) pj[h] = __shfl_sync(0xffffffffu, p[h], j);
    const float* vrow = Vs + j * d;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int c = lane + 32 * i;
      const float v = (c < d) ? vrow[c] : 0.f;
#pragma unroll
      for (int h = 0; h < kGT; ++h) acc[h][i] = fmaf(pj[h], v, acc[h][i]);
    }
  }
}

// ---- prefill -----------------------------------------------------------------------------------
// grid: (query tiles of 8 tokens, n_kv_heads * head chunks, n_seqs); block: 8 warps.
template <typename T, int DPL>
__global__ void __launch_bounds__(256) attn_prefill_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int W = 8;
  const int d = a.head_dim;
  float* Ks = smem;                          // [32][d+1]
  float* Vs = Ks + kTileKeys * (d + 1);      // [32][d]
  float* Qs = Vs + kTileKeys * d;            // [W][kGT][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int group = a.n_heads / a.n_kv_heads;
  const int chunks = (group + kGT - 1) / kGT;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int h0 = kvh * group + chunk * kGT;                 // first query head of this warp
  const int n_here = min(kGT, group - chunk * kGT);
  const int q0 = a.seq_qstart[b], q_len = a.seq_qstart[b + 1] - q0, past = a.seq_past[b];
  const int first = blockIdx.x * W;
  if (first >= q_len) return;
  const int slot = a.seq_slot[b];
  const int my_row = first + warp;
  const bool active = my_row < q_len;
  const int qpos = past + my_row;
  const int last_pos = past + min(q_len, first + W) - 1;
  // q of this warp into shared memory
  float* qs = Qs + warp * kGT * d;
  for (int i = lane; i < kGT * d; i += 32) {
    const int h = i / d, c = i - h * d;
    float v = 0.f;
    if (active && h < n_here) v = to_f32<T>(((const T*)a.q)[(size_t)(q0 + my_row) * a.q_ld + (size_t)(h0 + h) * d + c]);
    qs[i] = v;
  }
  float m[kGT], l[kGT], acc[kGT][DPL];
#pragma unroll
  for (int h = 0; h < kGT; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[h][i] = 0.f;
  }
  int k_begin = 0;
  if (a.window > 0) k_begin = max(0, (past + first) - a.window + 1) / kTileKeys * kTileKeys;
  const int k_end = last_pos + 1;
  for (int k0 = k_begin; k0 < k_end; k0 += kTileKeys) {
    __syncthreads();  // everyone is done with the previous tile (and q is written, first time)
    load_tile<T>(a, slot, kvh, k0, k_end, Ks, Vs, threadIdx.x, blockDim.x);
    __syncthreads();
    if (!active || k0 > qpos) continue;  // the whole tile lies in this query's future
    const int kpos = k0 + lane;
    bool visible = kpos <= qpos;
    if (a.window > 0) visible = visible && (kpos > qpos - a.window);
    if (a.window > 0 && k0 + kTileKeys - 1 <= qpos - a.window) continue;  // whole tile before the window
    fold_tile<DPL>(qs, Ks, Vs, d, n_here, a.scale, visible, lane, m, l, acc);
  }
  if (!active) return;
#pragma unroll
  for (int h = 0; h < kGT; ++h) {
    if (h >= n_here) continue;
    const float inv = 1.f / fmaxf(l[h], 1e-20f);
    T* o = (T*)a.out + (size_t)(q0 + my_row) * a.out_ld + (size_t)(h0 + h) * d;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int c = lane + 32 * i;
      if (c < d) o[c] = from_f32<T>(acc[h][i] * inv);
    }
  }
}

// ---- decode: one query token per sequence, keys split into ranges --------------------------------
// grid: (max_splits, n_kv_heads * head chunks, n_seqs); block: NW warps.
template <typename T, int DPL, int NW>
__global__ void __launch_bounds__(NW * 32) attn_decode_split_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  pdl_wait_block();
  pdl_launch_dependents();
  const int d = a.head_dim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_warp = kTileKeys * (d + 1) + kTileKeys * d;
  float* Ks = smem + warp * per_warp;
  float* Vs = Ks + kTileKeys * (d + 1);
  float* Qs = smem + NW * per_warp;              // [kGT][d], shared by the warps
  float* Ms = Qs + kGT * d;                      // [NW][kGT] m, then [NW][kGT] l
  float* Acc = Ms + 2 * NW * kGT;                // [NW][kGT][d]
  const int b = blockIdx.z, split = blockIdx.x;
  const int group = a.n_heads / a.n_kv_heads;
  const int chunks = (group + kGT - 1) / kGT;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int h0 = kvh * group + chunk * kGT;
  const int n_here = min(kGT, group - chunk * kGT);
  const int t = a.seq_qstart[b];                 // the sequence's single token of this step
  const int qpos = a.seq_past[b];                // its position; keys 0..qpos are in the cache
  const int len = qpos + 1;
  int k_lo = split * a.split_keys, k_hi = min(len, k_lo + a.split_keys);
  if (k_lo >= len) return;
  const int win_lo = a.window > 0 ? max(0, len - a.window) : 0;
  if (k_hi <= win_lo) return;                    // the whole range lies before the window
  const int slot = a.seq_slot[b];
  for (int i = threadIdx.x; i < kGT * d; i += blockDim.x) {
    const int h = i / d, c = i - h * d;
    Qs[i] = (h < n_here) ? to_f32<T>(((const T*)a.q)[(size_t)t * a.q_ld + (size_t)(h0 + h) * d + c]) : 0.f;
  }
  __syncthreads();
  float m[kGT], l[kGT], acc[kGT][DPL];
#pragma unroll
  for (int h = 0; h < kGT; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[h][i] = 0.f;
  }
  const int first_tile = max(k_lo, win_lo) / kTileKeys;
  const int last_tile = (k_hi - 1) / kTileKeys;
  for (int tile = first_tile + warp; tile <= last_tile; tile += NW) {
    const int k0 = tile * kTileKeys;
    load_tile<T>(a, slot, kvh, k0, k_hi, Ks, Vs, lane, 32);
    __syncwarp();
    const int kpos = k0 + lane;
    const bool visible = kpos >= max(k_lo, win_lo) && kpos < k_hi;
    fold_tile<DPL>(Qs, Ks, Vs, d, n_here, a.scale, visible, lane, m, l, acc);
    __syncwarp();
  }
  // merge the warps (fixed order: warp 0, 1, ..)
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < kGT; ++h) {
      Ms[warp * kGT + h] = m[h];
      Ms[NW * kGT + warp * kGT + h] = l[h];
    }
  }
#pragma unroll
  for (int h = 0; h < kGT; ++h)
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int c = lane + 32 * i;
      if (c < d) Acc[(warp * kGT + h) * d + c] = acc[h][i];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < n_here * d; i += blockDim.x) {
    const int h = i / d, c = i - h * d;
    float mm = -INFINITY;
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, Ms[w * kGT + h]);
    float ll = 0.f, aa = 0.f;
    if (mm != -INFINITY) {
      for (int w = 0; w < NW; ++w) {
        const float mw = Ms[w * kGT + h];
        const float f = (mw == -INFINITY) ? 0.f : expf(mw - mm);
        ll += Ms[NW * kGT + w * kGT + h] * f;
        aa += Acc[(w * kGT + h) * d + c] * f;
      }
    }
    const size_t pidx = ((size_t)b * a.n_heads + (h0 + h)) * a.max_splits + split;
    a.part_acc[pidx * d + c] = (ll > 0.f) ? aa / ll : 0.f;
    if (c == 0) a.part_lse[pidx] = (ll > 0.f) ? mm + logf(ll) : -INFINITY;
  }
}

// grid: (n_heads, n_seqs); merges the ranges that the split kernel wrote for this sequence.
template <typename T>
__global__ void attn_decode_combine_kernel(AttnArgs a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y, h = blockIdx.x;
  const int d = a.head_dim;
  const int t = a.seq_qstart[b];
  const int len = a.seq_past[b] + 1;
  int n_splits = (len + a.split_keys - 1) / a.split_keys;
  if (n_splits > a.max_splits) {
    // the sequence is longer than split_keys * max_splits keys: the split grid has no block for the ranges
    // beyond, and the scratch no room for them; say so and merge what was computed
    if (threadIdx.x == 0) report(a.status, kStatusPositionOutOfRange, b, len - 1, a.split_keys * a.max_splits);
    n_splits = a.max_splits;
  }
  const int win_lo = a.window > 0 ? max(0, len - a.window) : 0;
  const int first = min(win_lo / a.split_keys, n_splits);
  const size_t base = ((size_t)b * a.n_heads + h) * a.max_splits;
  float mx = -INFINITY;
  for (int s = first; s < n_splits; ++s) mx = fmaxf(mx, a.part_lse[base + s]);
  float denom = 0.f;
  for (int s = first; s < n_splits; ++s) {
    const float e = a.part_lse[base + s];
    denom += (e == -INFINITY) ? 0.f : expf(e - mx);
  }
  const float inv = 1.f / fmaxf(denom, 1e-20f);
  T* o = (T*)a.out + (size_t)t * a.out_ld + (size_t)h * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = 0.f;
    for (int s = first; s < n_splits; ++s) {
      const float e = a.part_lse[base + s];
      const float w = (e == -INFINITY) ? 0.f : expf(e - mx) * inv;
      v = fmaf(w, a.part_acc[(base + s) * d + c], v);
    }
    o[c] = from_f32<T>(v);
  }
}

template <typename K>
static int opt_in_smem(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

template <typename T, int DPL>
static int launch_prefill(const AttnArgs& a, int n_seqs, int max_q, cudaStream_t stream) {
  const int d = a.head_dim;
  const size_t smem = ((size_t)kTileKeys * (d + 1) + (size_t)kTileKeys * d + (size_t)8 * kGT * d) * sizeof(float);
  auto k = attn_prefill_kernel<T, DPL>;
  int e = opt_in_smem(k, smem);
  if (e) return e;
  const int group = a.n_heads / a.n_kv_heads;
  dim3 grid((max_q + 7) / 8, a.n_kv_heads * ((group + kGT - 1) / kGT), n_seqs);
  if (grid.y > 65535 || grid.z > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  pe::launch(k, grid, 256, smem, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

template <typename T, int DPL, int NW>
static int launch_decode(const AttnArgs& a, int n_seqs, cudaStream_t stream) {
  const int d = a.head_dim;
  const size_t smem = ((size_t)NW * (kTileKeys * (d + 1) + kTileKeys * d) + (size_t)kGT * d + 2 * NW * kGT +
                       (size_t)NW * kGT * d) * sizeof(float);
  auto k = attn_decode_split_kernel<T, DPL, NW>;
  int e = opt_in_smem(k, smem);
  if (e) return e;
  const int group = a.n_heads / a.n_kv_heads;
  dim3 grid(a.max_splits, a.n_kv_heads * ((group + kGT - 1) / kGT), n_seqs);
  if (grid.y > 65535 || grid.z > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  pe::launch(k, grid, NW * 32, smem, stream, a);
  PE_LAUNCH_CHECK();
  dim3 cgrid(a.n_heads, n_seqs);
  pe::launch(attn_decode_combine_kernel<T>, cgrid, 128, 0, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

template <typename T>
static int dispatch(const AttnArgs& a, int n_seqs, int max_q, bool decode, cudaStream_t stream) {
  const int d = a.head_dim;
  if (d > 512) return PE_ERR_UNSUPPORTED_SIZE;
  if (decode) {
    if (d <= 32) return launch_decode<T, 1, 4>(a, n_seqs, stream);
    if (d <= 64) return launch_decode<T, 2, 4>(a, n_seqs, stream);
    if (d <= 128) return launch_decode<T, 4, 4>(a, n_seqs, stream);
    if (d <= 256) return launch_decode<T, 8, 2>(a, n_seqs, stream);
    return launch_decode<T, 16, 1>(a, n_seqs, stream);
  }
  if (d <= 32) return launch_prefill<T, 1>(a, n_seqs, max_q, stream);
  if (d <= 64) return launch_prefill<T, 2>(a, n_seqs, max_q, stream);
  if (d <= 128) return launch_prefill<T, 4>(a, n_seqs, max_q, stream);
  if (d <= 256) return launch_prefill<T, 8>(a, n_seqs, max_q, stream);
  return launch_prefill<T, 16>(a, n_seqs, max_q, stream);
}

}  // namespace pe

// Scratch floats that the decode form needs: part_acc then part_lse.
extern "C" long long pe_attention_generic_scratch_floats(int n_seqs, int n_heads, int head_dim, int max_splits) {
  return (long long)n_seqs * n_heads * max_splits * (head_dim + 1);
}

// `decode` != 0: every sequence brings exactly one token (q row of sequence b is seq_qstart[b]).
extern "C" int pe_attention_generic(int dtype, int decode, const void* q, long long q_ld, void* out, long long out_ld,
                                    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale,
                                    int window, const int* seq_qstart, const int* seq_past, const int* seq_slot,
                                    const int* page_table, int table_stride, int num_pages, const void* k_pages,
                                    const void* v_pages, float* scratch, int split_keys, int max_splits, int* status,
                                    cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_heads % n_kv_heads) return PE_ERR_BAD_ARGUMENT;
  pe::AttnArgs a;
  a.q = q; a.q_ld = q_ld; a.out = out; a.out_ld = out_ld;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.scale = scale; a.window = window;
  a.seq_qstart = seq_qstart; a.seq_past = seq_past; a.seq_slot = seq_slot;
  a.page_table = page_table; a.table_stride = table_stride; a.num_pages = num_pages;
  a.k_pages = k_pages; a.v_pages = v_pages; a.status = status;
  a.part_acc = nullptr; a.part_lse = nullptr; a.split_keys = 0; a.max_splits = 0;
  if (decode) {
    if (!scratch || split_keys <= 0 || split_keys % pe::kTileKeys || max_splits <= 0) return PE_ERR_BAD_ARGUMENT;
    a.split_keys = split_keys; a.max_splits = max_splits;
    a.part_acc = scratch;
    a.part_lse = scratch + (size_t)n_seqs * n_heads * max_splits * head_dim;
  }
  if (dtype == PE_F32) return pe::dispatch<float>(a, n_seqs, max_q, decode != 0, stream);
  if (dtype == PE_BF16) return pe::dispatch<__nv_bfloat16>(a, n_seqs, max_q, decode != 0, stream);
  return PE_ERR_UNSUPPORTED_DTYPE;
}

// ---- the entry point that allocates nothing (see attention_noalloc.h) ----------------------------
#include "attention_noalloc.h"

#include <mutex>

namespace pe {

// Scratch for the partial results, inside the library image.  In host code this name is only a
// handle for the runtime's symbol table, never a device address: the address is looked up below.
static __device__ __align__(256) float g_noalloc_scratch[PE_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_noalloc_ptr[kMaxDevices] = {nullptr};
static std::mutex g_noalloc_mutex;

// Device address of the array on the current device; looked up once per device.
static int noalloc_scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return PE_ERR_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return PE_ERR_BAD_ARGUMENT;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_attention_decode_noalloc(int dtype, const void* q, long long q_ld, void* out, long long out_ld,
                                           int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale,
                                           int window, const int* seq_qstart, const int* seq_past, const int* seq_slot,
                                           const int* page_table, int table_stride, int num_pages, const void* k_pages,
                                           const void* v_pages, int split_keys, int max_splits, int* status,
                                           cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_heads % n_kv_heads) return PE_ERR_BAD_ARGUMENT;
  if (split_keys <= 0 || split_keys % pe::kTileKeys || max_splits <= 0) return PE_ERR_BAD_ARGUMENT;
  const long long need = (long long)n_seqs * n_heads * max_splits * (head_dim + 1);
  if (need > (long long)PE_NOALLOC_SCRATCH_FLOATS) return PE_ERR_SCRATCH_TOO_LARGE;
  float* scratch = nullptr;
  const int e = pe::noalloc_scratch_address(&scratch);
  if (e != PE_OK) return e;
  pe::AttnArgs a;
  a.q = q; a.q_ld = q_ld; a.out = out; a.out_ld = out_ld;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.scale = scale; a.window = window;
  a.seq_qstart = seq_qstart; a.seq_past = seq_past; a.seq_slot = seq_slot;
  a.page_table = page_table; a.table_stride = table_stride; a.num_pages = num_pages;
  a.k_pages = k_pages; a.v_pages = v_pages; a.status = status;
  a.split_keys = split_keys; a.max_splits = max_splits;
  a.part_acc = scratch;
  a.part_lse = scratch + (size_t)n_seqs * n_heads * max_splits * head_dim;
  if (dtype == PE_F32) return pe::dispatch<float>(a, n_seqs, 1, true, stream);
  if (dtype == PE_BF16) return pe::dispatch<__nv_bfloat16>(a, n_seqs, 1, true, stream);
  return PE_ERR_UNSUPPORTED_DTYPE;
}
