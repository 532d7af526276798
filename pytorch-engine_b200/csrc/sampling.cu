// Token sampling over rows of float32 logits, one block per row, nothing sorted.
//
// Filter chain in the reference's order (pygguf_engine/engine.py:91-134): repetition penalty on the
// unique ids of the recent tokens (92-97, a kernel of its own below), greedy when the temperature is
// at most 1e-5 (99-100, 146-147), else logits / temperature (102), top-k (104-108), softmax (110),
// min-p against the largest probability (112-114), top-p dropping entries whose preceding mass
// exceeds it (116-124).  Each filter keeps the entries above a threshold value, so the kept set is
// found by bitwise search on the order-preserving integer image of the values (counts for top-k,
// probability mass for top-p) instead of a sort.  The draw is the Gumbel-max rule,
// argmax(value_i + G_i) over kept entries, with G_i = -log(-log u_i) and u_i from a counter-based
// generator keyed by (seed, request, step, vocabulary index): the drawn token does not depend on
// the batch a request runs in.  (The reference draws with torch.multinomial, engine.py:149.)
//
// Two kernels when the caller lends scratch memory and the row is greedy or has a small top-k: the
// first cuts every row into chunks of kChunk entries, one block each, and leaves each chunk's
// candidates (its own top-k, found by a threshold search on the ordered keys in shared memory; or
// its largest entry); the second runs the filter chain on the candidates of a row, which hold
// every entry that the row's top-k can keep.  A threshold search takes 8 sweeps of 4 bits with
// per-thread counters (no atomics, fixed summation order) instead of 32 sweeps of one bit.
#include "api.h"
#include "common.cuh"

namespace pe {

constexpr int kSampleThreads = 1024;
constexpr int kMaxCompact = 1024;
constexpr int kChunk = 4096;        // entries of a row per block of the first kernel
constexpr int kChunkThreads = 256;
constexpr int kMaxChunks = 64;
constexpr int kMaxCandidates = 3072;  // candidates of a row that the second kernel takes

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform_of(unsigned long long key, int index) {
  const unsigned long long bits = mix64(key + (unsigned long long)index) >> 40;  // 24 bits
  return ((float)bits + 0.5f) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ unsigned ordered_key(float v) {
  if (v != v) return 0u;  // NaN sorts lowest
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgBest {
  float v;
  int i;
};
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ ArgBest block_argbest(ArgBest x, ArgBest* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  ArgBest r = (lane < nwarps) ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y;
    y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, y);
  }
  return r;
}
__device__ int block_sum_int(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  int r = (lane < nwarps) ? scratch[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

// 16 sums at once over the block in a fixed order; every thread gets all of them.
template <typename T>
__device__ void block_sum16(T (&v)[16], T* scratch /* [33][16] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int b = 0; b < 16; ++b)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[b] += __shfl_xor_sync(0xffffffffu, v[b], o);
  __syncthreads();
  if (lane == 0)
#pragma unroll
    for (int b = 0; b < 16; ++b) scratch[warp * 16 + b] = v[b];
  __syncthreads();
  if (threadIdx.x < 16) {
    T r = T(0);
    for (int w = 0; w < nwarps; ++w) r += scratch[w * 16 + threadIdx.x];
    scratch[32 * 16 + threadIdx.x] = r;
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < 16; ++b) v[b] = scratch[32 * 16 + b];
}

// The largest key J such that the weight of the entries with key >= J reaches the target
// (STRICT: exceeds it), four bits of J per sweep.  `entry(i, key, weight)` yields entry i; entries
// of weight zero do not count.  The total weight must reach (exceed) the target.
template <bool STRICT, typename T, typename EntryFn>
__device__ unsigned search16(int n, T target, EntryFn entry, T* scratch) {
  unsigned prefix = 0u;
  T above = T(0);   // weight of the entries whose key is beyond every key with this prefix
  for (int shift = 28; shift >= 0; shift -= 4) {
    const unsigned hi_mask = shift == 28 ? 0u : (0xFFFFFFFFu << (shift + 4));
    T acc[16];
#pragma unroll
    for (int b = 0; b < 16; ++b) acc[b] = T(0);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      unsigned key;
      T w;
      entry(i, key, w);
      if ((key & hi_mask) != prefix) continue;
      const unsigned bin = (key >> shift) & 15u;
#pragma unroll
      for (int b = 0; b < 16; ++b) acc[b] += (bin == (unsigned)b) ? w : T(0);
    }
    block_sum16(acc, scratch);
    int b = 15;
    T run = above;
    for (; b > 0; --b) {
      const T t = run + acc[b];
      if (STRICT ? (t > target) : (t >= target)) break;
      run = t;
    }
    prefix |= (unsigned)b << shift;
    above = run;
  }
  return prefix;
}

struct SampleArgs {
  const float* logits;
  long long ld;
  int n_rows, vocab;
  float temperature;
  int top_k;
  float top_p, min_p;
  unsigned long long seed;
  const int* row_request;
  const int* row_step;
  int* out_tokens;
  // scratch of the two-kernel path (null: one kernel does everything)
  int n_chunks, cand_cap;     // chunks per row; room for candidates per chunk
  float* cand_val;            // [rows][chunks][cap] values / temperature, in index order
  int* cand_idx;              // [rows][chunks][cap]
  int* cand_cnt;              // [rows][chunks]; -1: more than cap entries tie for the chunk's top-k
};

__device__ __forceinline__ float scaled(float v, float mult) {
  v *= mult;
  return v == v ? v : -INFINITY;   // NaN sorts lowest
}

// First kernel of the two-kernel path.  grid: (chunks, rows).
__global__ void __launch_bounds__(kChunkThreads) sample_chunks_kernel(SampleArgs a) {
  __shared__ float vals[kChunk];
  __shared__ int red_i[33 * 16];
  __shared__ ArgBest red_b[32];
  __shared__ int scan[kChunkThreads];
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
  const int lo = chunk * kChunk, n = min(kChunk, a.vocab - lo);
  const float* src = a.logits + (size_t)row * a.ld + lo;
  const size_t slot = (size_t)row * a.n_chunks + chunk;
  float* out_val = a.cand_val + slot * a.cand_cap;
  int* out_idx = a.cand_idx + slot * a.cand_cap;
  const bool greedy = a.temperature <= 1e-5f;
  const float mult = greedy ? 1.0f : 1.0f / a.temperature;
  if (greedy || a.top_k <= 0) {
    // no filter: the row's draw is the best of its chunks' draws (value + Gumbel noise; greedy: value)
    const unsigned long long key =
        mix64(a.seed ^ mix64(((unsigned long long)(unsigned)a.row_request[row] << 32) | (unsigned)a.row_step[row]));
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < n; i += blockDim.x) {
      float v = scaled(src[i], mult);
      if (!greedy && v != -INFINITY) v += -logf(-logf(uniform_of(key, lo + i)));
      best = better(best, ArgBest{v, lo + i});
    }
    best = block_argbest(best, red_b);
    if (tid == 0) {
      out_val[0] = best.v;
      out_idx[0] = best.i;
      a.cand_cnt[slot] = 1;
    }
    return;
  }
  for (int i = tid; i < n; i += blockDim.x) vals[i] = scaled(src[i], mult);
  __syncthreads();
  const int k = min(a.top_k, n);
  const unsigned K = search16<false, int>(n, k, [&](int i, unsigned& key, int& w) { key = ordered_key(vals[i]); w = 1; }, red_i);
  // the entries with key >= K, in index order: each thread owns a contiguous run
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int i0 = min(n, tid * per), i1 = min(n, i0 + per);
  int mine = 0;
  for (int i = i0; i < i1; ++i) mine += ordered_key(vals[i]) >= K;
  scan[tid] = mine;
  __syncthreads();
  for (int o = 1; o < kChunkThreads; o <<= 1) {
    const int add = (tid >= o) ? scan[tid - o] : 0;
    __syncthreads();
    scan[tid] += add;
    __syncthreads();
  }
  const int total = scan[kChunkThreads - 1];
  if (total > a.cand_cap) {   // ties beyond the room: the second kernel reads the whole row instead
    if (tid == 0) a.cand_cnt[slot] = -1;
    return;
  }
  int pos = scan[tid] - mine;
  for (int i = i0; i < i1; ++i)
    if (ordered_key(vals[i]) >= K) {
      out_val[pos] = vals[i];
      out_idx[pos] = lo + i;
      ++pos;
    }
  if (tid == 0) a.cand_cnt[slot] = total;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(SampleArgs a) {
  __shared__ float red_f[33 * 16];
  __shared__ int red_i[33 * 16];
  __shared__ ArgBest red_b[32];
  __shared__ float c_val[kMaxCompact];
  __shared__ int c_idx[kMaxCompact];
  __shared__ int scan[kSampleThreads];
  __shared__ float l_val[kMaxCandidates];
  __shared__ int l_idx[kMaxCandidates];
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const float* src = a.logits + (size_t)row * a.ld;
  const int V = a.vocab;
  const bool greedy = a.temperature <= 1e-5f;

  // candidates: the whole row (values scaled on the fly), the chunks' candidates, or, after top-k,
  // a compact list
  const float* vals = src;
  const int* idxs = nullptr;
  float mult = greedy ? 1.0f : 1.0f / a.temperature;
  int n = V;
  if (a.cand_cnt != nullptr) {
    // gather the chunks' candidates (index order is kept); a chunk that overflowed sends us to the row
    const int* cnt = a.cand_cnt + (size_t)row * a.n_chunks;
    int total = 0;
    bool ok = true;
    for (int c = 0; c < a.n_chunks; ++c) {
      const int m = cnt[c];
      if (m < 0) ok = false;
      total += max(m, 0);
    }
    if (ok && total <= kMaxCandidates) {
      int base = 0;
      for (int c = 0; c < a.n_chunks; ++c) {
        const int m = cnt[c];
        const size_t slot = ((size_t)row * a.n_chunks + c) * a.cand_cap;
        for (int i = tid; i < m; i += blockDim.x) {
          l_val[base + i] = a.cand_val[slot + i];
          l_idx[base + i] = a.cand_idx[slot + i];
        }
        base += m;
      }
      __syncthreads();
      vals = l_val;
      idxs = l_idx;
      mult = 1.0f;
      n = total;
    }
  }

  const bool drawn_in_chunks = idxs != nullptr && a.top_k <= 0;   // the candidates are the chunks' finished draws
  if (greedy || drawn_in_chunks) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < n; i += blockDim.x) best = better(best, ArgBest{scaled(vals[i], mult), idxs ? idxs[i] : i});
    best = block_argbest(best, red_b);
    if (tid == 0) a.out_tokens[row] = best.i == 0x7fffffff ? 0 : best.i;
    return;
  }

  unsigned keep_key = 0u;  // entries with ordered_key(value) >= keep_key are kept

  // largest value
  float mx = -INFINITY;
  for (int i = tid; i < n; i += blockDim.x) mx = fmaxf(mx, scaled(vals[i], mult));
  mx = block_max(mx, red_f);

  if (a.top_k > 0 && a.top_k < V) {
    // k-th largest value: the largest key K with count(key >= K) >= k
    const unsigned K = search16<false, int>(
        n, min(a.top_k, n), [&](int i, unsigned& key, int& w) { key = ordered_key(scaled(vals[i], mult)); w = 1; }, red_i);
    keep_key = K;
    if (a.top_k <= kMaxCompact) {
      // compact the candidates in index order (deterministic): count, scan, write
      int mine = 0;
      for (int i = tid; i < n; i += blockDim.x) mine += ordered_key(scaled(vals[i], mult)) >= K;
      scan[tid] = mine;
      __syncthreads();
      for (int o = 1; o < kSampleThreads; o <<= 1) {
        const int add = (tid >= o) ? scan[tid - o] : 0;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
      }
      int pos = scan[tid] - mine;
      const int total = scan[kSampleThreads - 1];
      // a thread's entries are strided, so positions within the list follow (thread, index) order;
      // the list is a set here: nothing below depends on its order
      for (int i = tid; i < n; i += blockDim.x) {
        const float v = scaled(vals[i], mult);
        if (ordered_key(v) >= K) {
          if (pos < kMaxCompact) {
            c_val[pos] = v;
            c_idx[pos] = idxs ? idxs[i] : i;
          }
          ++pos;
        }
      }
      __syncthreads();
      vals = c_val;
      idxs = c_idx;
      mult = 1.0f;
      n = min(total, kMaxCompact);
    }
  }

  // softmax denominator over the kept entries, relative to the largest value
  float z = 0.f;
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = scaled(vals[i], mult);
    if (ordered_key(v) >= keep_key) z += expf(v - mx);
  }
  z = block_sum(z, red_f);

  if (a.min_p > 0.f) {
    // p_i < min_p * p_max  <=>  exp(v_i - max) < min_p   (p_max = 1 / z)
    // as a threshold on the value: v_i >= max + log(min_p)
    const float cut = mx + logf(a.min_p);
    const unsigned kc = ordered_key(cut);
    if (kc > keep_key) keep_key = kc;
  }

  if (a.top_p > 0.f && a.top_p < 1.f) {
    // keep entry i iff the mass of the kept entries with a larger value is <= top_p: the threshold
    // is the largest key J whose mass at or above it exceeds top_p (everything if none does, which
    // cannot be: the whole mass exceeds it)
    const float limit = a.top_p * z;
    const unsigned kk = keep_key;
    const unsigned J = search16<true, float>(
        n, limit,
        [&](int i, unsigned& key, float& w) {
          const float v = scaled(vals[i], mult);
          key = ordered_key(v);
          w = key >= kk ? expf(v - mx) : 0.f;
        },
        red_f);
    if (J > keep_key) keep_key = J;
  }

  // draw
  const unsigned long long key =
      mix64(a.seed ^ mix64(((unsigned long long)(unsigned)a.row_request[row] << 32) | (unsigned)a.row_step[row]));
  ArgBest best{-INFINITY, 0x7fffffff};
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = scaled(vals[i], mult);
    if (ordered_key(v) < keep_key || v == -INFINITY) continue;
    const int index = idxs ? idxs[i] : i;
    const float u = uniform_of(key, index);
    const float g = -logf(-logf(u));
    best = better(best, ArgBest{v + g, index});
  }
  best = block_argbest(best, red_b);
  if (tid == 0) {
    int tok = best.i;
    if (tok == 0x7fffffff) {  // nothing kept (all NaN): fall back to the first entry
      tok = 0;
    }
    a.out_tokens[row] = tok;
  }
}

// logits[row, id] for the unique ids among recent[row, 0..count): negative -> * penalty, else / penalty.
__global__ void repetition_penalty_kernel(float* logits, long long ld, int vocab, const int* recent, int recent_stride,
                                          const int* recent_count, float penalty) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int n = min(recent_count[row], recent_stride);
  const int* r = recent + (size_t)row * recent_stride;
  for (int t = threadIdx.x; t < n; t += blockDim.x) {
    const int id = r[t];
    if (id < 0 || id >= vocab) continue;
    bool first = true;
    for (int s = 0; s < t; ++s)
      if (r[s] == id) {
        first = false;
        break;
      }
    if (!first) continue;
    float* p = logits + (size_t)row * ld + id;
    const float v = *p;
    *p = v < 0.f ? v * penalty : v / penalty;
  }
}

}  // namespace pe

// Room for ties at a chunk's k-th value beyond its k candidates.
static bool unfiltered(float temperature, int top_k, float top_p, float min_p) {
  return temperature <= 1e-5f || ((top_k <= 0) && !(top_p > 0.f && top_p < 1.f) && !(min_p > 0.f));
}
static int cand_cap_of(float temperature, int top_k, float top_p, float min_p) {
  return unfiltered(temperature, top_k, top_p, min_p) ? 1 : top_k + 8;
}
static bool two_kernels(int vocab, float temperature, int top_k, float top_p, float min_p) {
  const int chunks = (vocab + pe::kChunk - 1) / pe::kChunk;
  if (chunks < 2 || chunks > pe::kMaxChunks) return false;
  if (unfiltered(temperature, top_k, top_p, min_p)) return true;
  return top_k > 0 && top_k < vocab && (long long)chunks * top_k <= pe::kMaxCandidates;
}

// Bytes of scratch with which pe_sample takes its two-kernel path for these settings (0: it has none).
extern "C" long long pe_sample_scratch_bytes(int n_rows, int vocab, float temperature, int top_k, float top_p, float min_p) {
  if (n_rows <= 0 || !two_kernels(vocab, temperature, top_k, top_p, min_p)) return 0;
  const long long chunks = (vocab + pe::kChunk - 1) / pe::kChunk;
  return (long long)n_rows * chunks * (cand_cap_of(temperature, top_k, top_p, min_p) * 8ll + 4ll);
}

// scratch: null, or at least pe_sample_scratch_bytes(...) bytes, 4-byte aligned.
extern "C" int pe_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k,
                         float top_p, float min_p, unsigned long long seed, const int* row_request, const int* row_step,
                         int* out_tokens, void* scratch, long long scratch_bytes, cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (vocab <= 0 || ld < vocab) return PE_ERR_BAD_ARGUMENT;
  pe::SampleArgs a;
  a.logits = logits; a.ld = ld; a.n_rows = n_rows; a.vocab = vocab; a.temperature = temperature; a.top_k = top_k;
  a.top_p = top_p; a.min_p = min_p; a.seed = seed; a.row_request = row_request; a.row_step = row_step;
  a.out_tokens = out_tokens;
  a.n_chunks = 0; a.cand_cap = 0; a.cand_val = nullptr; a.cand_idx = nullptr; a.cand_cnt = nullptr;
  const long long need = pe_sample_scratch_bytes(n_rows, vocab, temperature, top_k, top_p, min_p);
  if (scratch != nullptr && need > 0 && scratch_bytes >= need && ((uintptr_t)scratch % 4) == 0) {
    a.n_chunks = (vocab + pe::kChunk - 1) / pe::kChunk;
    a.cand_cap = cand_cap_of(temperature, top_k, top_p, min_p);
    const size_t slots = (size_t)n_rows * a.n_chunks;
    a.cand_val = reinterpret_cast<float*>(scratch);
    a.cand_idx = reinterpret_cast<int*>(a.cand_val + slots * a.cand_cap);
    a.cand_cnt = a.cand_idx + slots * a.cand_cap;
    pe::launch(pe::sample_chunks_kernel, dim3(a.n_chunks, n_rows), pe::kChunkThreads, 0, stream, a);
    PE_LAUNCH_CHECK();
  }
  pe::launch(pe::sample_kernel, n_rows, pe::kSampleThreads, 0, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_repetition_penalty(float* logits, long long ld, int n_rows, int vocab, const int* recent,
                                     int recent_stride, const int* recent_count, float penalty, cudaStream_t stream) {
  if (n_rows <= 0 || penalty == 1.0f) return PE_OK;
  if (penalty <= 0.f) return PE_ERR_BAD_ARGUMENT;
  pe::launch(pe::repetition_penalty_kernel, n_rows, 256, 0, stream, logits, ld, vocab, recent, recent_stride, recent_count, penalty);
  PE_LAUNCH_CHECK();
  return PE_OK;
}
