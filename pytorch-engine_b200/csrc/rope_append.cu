// Per-head q/k RMSNorm, rotary position encoding and the append of k, v to the paged cache, in one
// pass over the fused q|k|v projection; and the small kernel that expands the batch description
// into per-token sequence index and position.
//
// Reference formulas: q/k-norm over head_dim before RoPE, not on v (pygguf_engine/model.py:471-474);
// split-half rotation of the first rotary_dim features with position = cached length + row
// (pygguf_engine/model.py:232-241, 211-214); append at [P, P+S) (pygguf_engine/model.py:482-483);
// positions read from device memory (pygguf_engine/kv_cache.py:1847-1852).
#include "api.h"
#include "common.cuh"

namespace pe {

// token_seq[t] = index of the batch entry that token t belongs to; token_pos[t] = its position.
__global__ void batch_expand_kernel(const int* seq_qstart, const int* seq_past,
                                    int n_seqs, int* __restrict__ token_seq, int* __restrict__ token_pos) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  if (b >= n_seqs) return;
  const int q0 = seq_qstart[b], q1 = seq_qstart[b + 1], past = seq_past[b];
  for (int t = q0 + threadIdx.x; t < q1; t += blockDim.x) {
    token_seq[t] = b;
    token_pos[t] = past + (t - q0);
  }
}

struct RopeAppendArgs {
  void* qkv;            // [n_tokens, ld]; q heads, then k heads, then v heads; q and k are rewritten in place
  long long ld;
  int n_tokens, n_heads, n_kv_heads, head_dim;
  const float* q_norm_w;  // [head_dim] or null
  const float* k_norm_w;  // [head_dim] or null
  float eps;
  const float* cos_table;  // [table_rows, rotary_dim/2] or null
  const float* sin_table;
  int rotary_dim, table_rows;
  const int* token_seq;
  const int* token_pos;
  const int* seq_slot;
  const int* seq_qstart;   // [n_seqs + 1]
  const int* page_table;   // [slots, table_stride]
  int table_stride, num_pages;
  void* k_pages;           // [num_pages, n_kv_heads, 64, head_dim]
  void* v_pages;
  int write_cache;
  int* status;
};

template <typename T> __device__ __forceinline__ float2 load2(const T* p);
template <> __device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void store2(T* p, float2 v);
template <> __device__ __forceinline__ void store2<float>(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
template <> __device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
}

// PAIRS: every access covers two adjacent features (head size and half the rotary size even, rows
// aligned to two elements); otherwise one feature at a time.
template <typename T, bool PAIRS>
__global__ void qk_norm_rope_append_kernel(RopeAppendArgs a) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  const int total_heads = a.n_heads + 2 * a.n_kv_heads;
  const bool valid = t < a.n_tokens && head < total_heads;
  const int d = a.head_dim;
  const bool is_q = head < a.n_heads;
  const bool is_k = !is_q && head < a.n_heads + a.n_kv_heads;
  const int kv_head = is_q ? -1 : (is_k ? head - a.n_heads : head - a.n_heads - a.n_kv_heads);
  // Before the wait: what does not come from the kernel before this one.  The step's batch description
  // and the page table were complete before that kernel started, the angle tables and norm weights never
  // change; only the q|k|v rows have to be waited for.  In a decode step this kernel's latency is on the
  // critical path, and the chain token -> sequence -> slot -> page is three trips to memory.
  const bool to_cache = valid && !is_q && a.write_cache;
  int pos = 0, seq = 0, slot = 0, q_begin = 0, q_end = 0, page = -1;
  if (valid) pos = a.token_pos[t];
  if (to_cache) {
    seq = a.token_seq[t];
    slot = a.seq_slot[seq];
    q_begin = a.seq_qstart[seq];
    q_end = a.seq_qstart[seq + 1];
    if (pos >= 0 && pos / kPageTokens < a.table_stride)
      page = a.page_table[(size_t)slot * a.table_stride + pos / kPageTokens];
  }
  const float* w = is_q ? a.q_norm_w : a.k_norm_w;
  const int rot = a.cos_table ? a.rotary_dim : 0;
  const int half = rot / 2;
  const bool rotates = valid && (is_q || is_k);
  const bool pos_in_table = pos >= 0 && pos < a.table_rows;
  const float* cs = (rot > 0 && pos_in_table) ? a.cos_table + (size_t)pos * half : nullptr;
  const float* sn = (rot > 0 && pos_in_table) ? a.sin_table + (size_t)pos * half : nullptr;
  // the first pair of each lane (PAIRS): angles and weights are on their way before the wait
  float2 c_first = make_float2(1.f, 1.f), s_first = make_float2(0.f, 0.f);
  float2 w1_first = make_float2(1.f, 1.f), w2_first = make_float2(1.f, 1.f);
  if (PAIRS && rotates && lane * 2 < half) {
    if (cs) {
      c_first = *reinterpret_cast<const float2*>(cs + lane * 2);
      s_first = *reinterpret_cast<const float2*>(sn + lane * 2);
    }
    if (w) {
      w1_first = *reinterpret_cast<const float2*>(w + lane * 2);
      w2_first = *reinterpret_cast<const float2*>(w + lane * 2 + half);
    }
  }
  pdl_wait_block();
  pdl_launch_dependents();
  if (!valid) return;
  T* row = (T*)a.qkv + (size_t)t * a.ld + (size_t)head * d;

  // where this token's k/v row lies in the paged cache
  T* cache_row = nullptr;
  if (to_cache) {
    if (pos < 0 || pos / kPageTokens >= a.table_stride) {
      if (lane == 0) report(a.status, kStatusPositionOutOfRange, t, pos, a.table_stride * kPageTokens);
    } else if (page < 0 || page >= a.num_pages) {
      if (lane == 0) report(a.status, kStatusPageOutOfRange, t, page, a.num_pages);
    } else {
      T* base = (T*)(is_k ? a.k_pages : a.v_pages);
      const int off = pos % kPageTokens;
      cache_row = base + (((size_t)page * a.n_kv_heads + kv_head) * kPageTokens + off) * d;
      // Rows of a page beyond the sequence's last key must hold finite values (readers multiply them
      // by a probability of zero): the sequence's last token of this step clears the rest of its page
      // when it starts the page or ends a multi-token step; later single tokens find it cleared.
      if (t + 1 == q_end && off + 1 < kPageTokens && (off == 0 || q_end - q_begin > 1)) {
        T* rest = cache_row + d;
        const size_t n = (size_t)(kPageTokens - 1 - off) * d;
        if ((d * sizeof(T)) % 16 == 0) {
          uint4* r4 = reinterpret_cast<uint4*>(rest);
          const size_t n4 = n * sizeof(T) / 16;
          for (size_t i = lane; i < n4; i += 32) r4[i] = make_uint4(0, 0, 0, 0);
        } else {
          for (size_t i = lane; i < n; i += 32) rest[i] = from_f32<T>(0.f);
        }
      }
    }
  }

  if (!is_q && !is_k) {  // v: copy only
    if (cache_row) {
      if (PAIRS) {
        for (int c = lane * 2; c < d; c += 64) store2<T>(cache_row + c, load2<T>(row + c));
      } else {
        for (int c = lane; c < d; c += 32) cache_row[c] = row[c];
      }
    }
    return;
  }

  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    if (PAIRS) {
      for (int c = lane * 2; c < d; c += 64) {
        const float2 x = load2<T>(row + c);
        ss += x.x * x.x + x.y * x.y;
      }
    } else {
      for (int c = lane; c < d; c += 32) {
        const float x = to_f32<T>(row[c]);
        ss += x * x;
      }
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)d + a.eps);
  }
  // Norm and rotation are one float32 computation: nothing is rounded between them (the reference
  // rounds to its 16-bit type in between only because they are separate ops there).
  auto normed = [&](int c) -> float {
    float x = to_f32<T>(row[c]);
    if (w) x = x * inv * w[c];
    return x;
  };
  if (rot > 0 && !pos_in_table) {
    if (lane == 0) report(a.status, kStatusPositionOutOfRange, t, pos, a.table_rows);
    return;
  }
  if (PAIRS) {
    for (int j = lane * 2; j < half; j += 64) {
      const bool first = j == lane * 2;
      float2 x1 = load2<T>(row + j), x2 = load2<T>(row + j + half);
      if (w) {
        const float2 w1 = first ? w1_first : *reinterpret_cast<const float2*>(w + j);
        const float2 w2 = first ? w2_first : *reinterpret_cast<const float2*>(w + j + half);
        x1.x *= inv * w1.x; x1.y *= inv * w1.y; x2.x *= inv * w2.x; x2.y *= inv * w2.y;
      }
      const float2 c = first ? c_first : *reinterpret_cast<const float2*>(cs + j);
      const float2 sv = first ? s_first : *reinterpret_cast<const float2*>(sn + j);
      const float2 o1 = make_float2(x1.x * c.x - x2.x * sv.x, x1.y * c.y - x2.y * sv.y);
      const float2 o2 = make_float2(x2.x * c.x + x1.x * sv.x, x2.y * c.y + x1.y * sv.y);
      store2<T>(row + j, o1);
      store2<T>(row + j + half, o2);
      if (cache_row) {
        store2<T>(cache_row + j, o1);
        store2<T>(cache_row + j + half, o2);
      }
    }
    for (int c = rot + lane * 2; c < d; c += 64) {
      float2 x = load2<T>(row + c);
      if (w) {
        const float2 wv = *reinterpret_cast<const float2*>(w + c);
        x.x *= inv * wv.x; x.y *= inv * wv.y;
      }
      store2<T>(row + c, x);
      if (cache_row) store2<T>(cache_row + c, x);
    }
    return;
  }
  // rotated pairs (j, j + half): both are read before either is written
  for (int j = lane; j < half; j += 32) {
    const float x1 = normed(j), x2 = normed(j + half);
    const float c = cs[j], s = sn[j];
    const T o1 = from_f32<T>(x1 * c - x2 * s);
    const T o2 = from_f32<T>(x2 * c + x1 * s);
    row[j] = o1;
    row[j + half] = o2;
    if (cache_row) {
      cache_row[j] = o1;
      cache_row[j + half] = o2;
    }
  }
  // features beyond rotary_dim pass through (normalised only)
  for (int c = rot + lane; c < d; c += 32) {
    const T o = from_f32<T>(normed(c));
    row[c] = o;
    if (cache_row) cache_row[c] = o;
  }
}

// The same for bfloat16 rows with 16-byte accesses: head sizes that are multiples of 16 up to 256,
// the whole head rotated, everything 16-byte aligned.  A head takes head_dim / 8 lanes, so a warp
// holds several heads; the lane that holds features [8i, 8i + 8) of the first half trades its
// normalised values with the lane that holds the matching features of the second half.  A block
// takes TPB tokens and asks for all their rows and positions before it uses the first: a thread
// with one 16-byte load in flight at a time reached 2.3 TB/s on a 2,048-token step (54 MB moved in
// 23.6 us), which is the latency of one load after the other, not bandwidth.
template <int TPB>
__global__ void __launch_bounds__(256, 4) qk_norm_rope_append_vec8_kernel(RopeAppendArgs a, int lanes_per_head) {
  pdl_wait_block();
  pdl_launch_dependents();
  typedef __nv_bfloat16 T;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lph = lanes_per_head, heads_per_warp = 32 / lph;
  const int sub = lane / lph, li = lane - sub * lph;
  const int total_heads = a.n_heads + 2 * a.n_kv_heads;
  const int head = (blockIdx.y * (blockDim.x >> 5) + warp) * heads_per_warp + sub;
  const bool active = sub < heads_per_warp && head < total_heads;
  const int d = a.head_dim;
  const bool is_q = head < a.n_heads;
  const bool is_k = !is_q && head < a.n_heads + a.n_kv_heads;
  const bool is_v = !is_q && !is_k;
  const int kv_head = is_k ? head - a.n_heads : head - a.n_heads - a.n_kv_heads;
  const int half_l = lph >> 1;
  const bool second = li >= half_l;
  const int j = 8 * (second ? li - half_l : li);  // this lane's place in a row of the angle tables
  const int partner = lane + (second ? -half_l : half_l);
  const bool pow2 = (lph & (lph - 1)) == 0;
  const bool rotate = a.cos_table != nullptr && a.rotary_dim > 0;
  const float* w = is_q ? a.q_norm_w : a.k_norm_w;
  float wv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) wv[e] = 1.f;
  if (active && !is_v && w) {
    const float4 w0 = *reinterpret_cast<const float4*>(w + 8 * li), w1 = *reinterpret_cast<const float4*>(w + 8 * li + 4);
    wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
  }
  // every token's row and position first: independent loads, all in flight together
  uint4 raws[TPB];
  int poss[TPB];
#pragma unroll
  for (int i = 0; i < TPB; ++i) {
    const int t = blockIdx.x * TPB + i;
    raws[i] = make_uint4(0, 0, 0, 0);
    poss[i] = -1;
    if (t < a.n_tokens) {
      if (active) raws[i] = *reinterpret_cast<const uint4*>((const T*)a.qkv + (size_t)t * a.ld + (size_t)head * d + 8 * li);
      poss[i] = a.token_pos[t];
    }
  }
#pragma unroll
  for (int i = 0; i < TPB; ++i) {
    const int t = blockIdx.x * TPB + i;
    if (t >= a.n_tokens) break;
    T* row = (T*)a.qkv + (size_t)t * a.ld + (size_t)head * d + 8 * li;
    const uint4 raw = raws[i];
    const int pos = poss[i];
    T* cache_row = nullptr;
    if (active && !is_q && a.write_cache) {
      const int b = a.token_seq[t];
      const int slot = a.seq_slot[b];
      const int logical = pos / kPageTokens;
      if (pos < 0 || logical >= a.table_stride) {
        if (li == 0) report(a.status, kStatusPositionOutOfRange, t, pos, a.table_stride * kPageTokens);
      } else {
        const int page = a.page_table[(size_t)slot * a.table_stride + logical];
        if (page < 0 || page >= a.num_pages) {
          if (li == 0) report(a.status, kStatusPageOutOfRange, t, page, a.num_pages);
        } else {
          T* base = (T*)(is_k ? a.k_pages : a.v_pages);
          const int off = pos % kPageTokens;
          T* head_row = base + (((size_t)page * a.n_kv_heads + kv_head) * kPageTokens + off) * d;
          cache_row = head_row + 8 * li;
          // clear the rest of the page (see the kernel above for when and why)
          const int q_end = a.seq_qstart[b + 1];
          if (t + 1 == q_end && off + 1 < kPageTokens && (off == 0 || q_end - a.seq_qstart[b] > 1)) {
            uint4* r4 = reinterpret_cast<uint4*>(head_row + d);
            const size_t n4 = (size_t)(kPageTokens - 1 - off) * d / 8;
            for (size_t x = li; x < n4; x += lph) r4[x] = make_uint4(0, 0, 0, 0);
          }
        }
      }
    }
    float x[8];
    {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        x[2 * e] = f.x;
        x[2 * e + 1] = f.y;
      }
    }
    {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
      if (pow2) {
        for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      } else {
        float total = 0.f;
        for (int l = 0; l < lph; ++l) total += __shfl_sync(0xffffffffu, ss, (sub * lph + l) & 31);
        ss = total;
      }
      if (!is_v && w != nullptr) {
        const float inv = rsqrtf(ss / (float)d + a.eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x[e] * inv * wv[e];
      }
    }
    float other[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) other[e] = __shfl_sync(0xffffffffu, x[e], partner & 31);
    if (active && !is_v && rotate) {
      if (pos < 0 || pos >= a.table_rows) {
        if (li == 0) report(a.status, kStatusPositionOutOfRange, t, pos, a.table_rows);
        continue;
      }
      const float* cs = a.cos_table + (size_t)pos * (d / 2) + j;     // the tables stay in L2
      const float* sn = a.sin_table + (size_t)pos * (d / 2) + j;
      const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sn), s1 = *reinterpret_cast<const float4*>(sn + 4);
      const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = second ? x[e] * cv[e] + other[e] * sv[e] : x[e] * cv[e] - other[e] * sv[e];
    }
    if (!active) continue;
    uint4 out = raw;
    if (!is_v) {
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
      *reinterpret_cast<uint4*>(row) = out;
    }
    if (cache_row) *reinterpret_cast<uint4*>(cache_row) = out;
  }
}

}  // namespace pe

extern "C" int pe_batch_expand(const int* seq_qstart, const int* seq_past, int n_seqs, int* token_seq, int* token_pos,
                               cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  pe::launch(pe::batch_expand_kernel, n_seqs, 128, 0, stream, seq_qstart, seq_past, n_seqs, token_seq, token_pos);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_qk_norm_rope_append(int dtype, void* qkv, long long ld, int n_tokens, int n_heads, int n_kv_heads,
                                      int head_dim, const float* q_norm_w, const float* k_norm_w, float eps,
                                      const float* cos_table, const float* sin_table, int rotary_dim, int table_rows,
                                      const int* token_seq, const int* token_pos, const int* seq_slot,
                                      const int* seq_qstart, const int* page_table, int table_stride, int num_pages, void* k_pages,
                                      void* v_pages, int write_cache, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (head_dim <= 0 || n_heads <= 0 || n_kv_heads < 0) return PE_ERR_BAD_ARGUMENT;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return PE_ERR_UNSUPPORTED_SIZE;
  if (ld < (long long)(n_heads + 2 * n_kv_heads) * head_dim) return PE_ERR_BAD_ARGUMENT;
  pe::RopeAppendArgs a;
  a.qkv = qkv; a.ld = ld; a.n_tokens = n_tokens; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim;
  a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.eps = eps;
  a.cos_table = cos_table; a.sin_table = sin_table; a.rotary_dim = rotary_dim; a.table_rows = table_rows;
  a.token_seq = token_seq; a.token_pos = token_pos; a.seq_slot = seq_slot; a.seq_qstart = seq_qstart;
  a.page_table = page_table; a.table_stride = table_stride; a.num_pages = num_pages;
  a.k_pages = k_pages; a.v_pages = v_pages; a.write_cache = write_cache; a.status = status;
  const int warps = 4;
  const int total_heads = n_heads + 2 * n_kv_heads;
  dim3 grid(n_tokens, (total_heads + warps - 1) / warps);
  if (grid.y > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  // two features per access where everything is even and aligned (the usual case)
  const size_t esz = dtype == PE_F32 ? 4 : 2;
  const bool pairs = (head_dim % 2 == 0) && (rotary_dim % 4 == 0) && (ld % 2 == 0) && ((uintptr_t)qkv % (2 * esz) == 0) &&
                     ((uintptr_t)k_pages % (2 * esz) == 0) && ((uintptr_t)v_pages % (2 * esz) == 0) &&
                     ((uintptr_t)cos_table % 8 == 0) && ((uintptr_t)sin_table % 8 == 0) &&
                     ((uintptr_t)q_norm_w % 8 == 0) && ((uintptr_t)k_norm_w % 8 == 0);
  const bool vec8 = dtype == PE_BF16 && head_dim % 16 == 0 && head_dim <= 256 && (rotary_dim == head_dim || cos_table == nullptr) &&
                    ld % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 &&
                    (uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0 && (uintptr_t)q_norm_w % 16 == 0 &&
                    (uintptr_t)k_norm_w % 16 == 0;
  if (vec8 && n_tokens >= 256) {  // measured: with a few tokens (decode) the kernel above is the faster one
    constexpr int kTokensPerBlock = 4;
    const int lph = head_dim / 8, heads_per_block = 8 * (32 / lph);
    dim3 g((n_tokens + kTokensPerBlock - 1) / kTokensPerBlock, (total_heads + heads_per_block - 1) / heads_per_block);
    if (g.y > 65535) return PE_ERR_UNSUPPORTED_SIZE;
    pe::launch(pe::qk_norm_rope_append_vec8_kernel<kTokensPerBlock>, g, 256, 0, stream, a, lph);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
  if (dtype == PE_F32) {
    if (pairs) pe::launch(pe::qk_norm_rope_append_kernel<float, true>, grid, warps * 32, 0, stream, a);
    else pe::launch(pe::qk_norm_rope_append_kernel<float, false>, grid, warps * 32, 0, stream, a);
  } else if (dtype == PE_BF16) {
    if (pairs) pe::launch(pe::qk_norm_rope_append_kernel<__nv_bfloat16, true>, grid, warps * 32, 0, stream, a);
    else pe::launch(pe::qk_norm_rope_append_kernel<__nv_bfloat16, false>, grid, warps * 32, 0, stream, a);
  } else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
