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
#include "common.cuh"

namespace pe {

constexpr int kSampleThreads = 1024;
constexpr int kMaxCompact = 1024;

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
};

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(SampleArgs a) {
  __shared__ float red_f[32];
  __shared__ int red_i[32];
  __shared__ ArgBest red_b[32];
  __shared__ float c_val[kMaxCompact];
  __shared__ int c_idx[kMaxCompact];
  __shared__ int scan[kSampleThreads];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const float* src = a.logits + (size_t)row * a.ld;
  const int V = a.vocab;

  if (a.temperature <= 1e-5f) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < V; i += blockDim.x) {
      float v = src[i];
      if (v != v) v = -INFINITY;
      best = better(best, ArgBest{v, i});
    }
    best = block_argbest(best, red_b);
    if (tid == 0) a.out_tokens[row] = best.i == 0x7fffffff ? 0 : best.i;
    return;
  }

  const float inv_t = 1.0f / a.temperature;
  // candidates: the whole row (values scaled on the fly) or, after top-k, a compact list
  const float* vals = src;
  const int* idxs = nullptr;
  float mult = inv_t;
  int n = V;
  unsigned keep_key = 0u;  // entries with ordered_key(value) >= keep_key are kept

  // largest value
  float mx = -INFINITY;
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = vals[i] * mult;
    if (v == v) mx = fmaxf(mx, v);
  }
  mx = block_max(mx, red_f);

  if (a.top_k > 0 && a.top_k < V) {
    // k-th largest value: largest key K with count(key >= K) >= k
    unsigned K = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = K | (1u << bit);
      int cnt = 0;
      for (int i = tid; i < n; i += blockDim.x) cnt += ordered_key(vals[i] * mult) >= cand;
      cnt = block_sum_int(cnt, red_i);
      if (cnt >= a.top_k) K = cand;
    }
    keep_key = K;
    if (a.top_k <= kMaxCompact) {
      // compact the candidates in index order (deterministic): count, scan, write
      int mine = 0;
      for (int i = tid; i < n; i += blockDim.x) mine += ordered_key(vals[i] * mult) >= K;
      scan[tid] = mine;
      __syncthreads();
      // inclusive scan over the block's threads (Hillis-Steele)
      for (int o = 1; o < kSampleThreads; o <<= 1) {
        const int add = (tid >= o) ? scan[tid - o] : 0;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
      }
      int pos = scan[tid] - mine;
      const int total = scan[kSampleThreads - 1];
      for (int i = tid; i < n; i += blockDim.x) {
        const float v = vals[i] * mult;
        if (ordered_key(v) >= K) {
          if (pos < kMaxCompact) {
            c_val[pos] = v;
            c_idx[pos] = i;
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
    const float v = vals[i] * mult;
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
    // keep entry i iff the mass of kept entries with a larger value is <= top_p.
    // P(K): mass of entries with key > K is <= top_p.  Find the largest K with P false.
    const float limit = a.top_p * z;
    auto mass_above = [&](unsigned K) -> float {
      float s = 0.f;
      for (int i = tid; i < n; i += blockDim.x) {
        const float v = vals[i] * mult;
        const unsigned k = ordered_key(v);
        if (k > K && k >= keep_key) s += expf(v - mx);
      }
      return block_sum(s, red_f);
    };
    if (!(mass_above(0u) <= limit)) {
      unsigned K = 0u;
      for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = K | (1u << bit);
        if (!(mass_above(cand) <= limit)) K = cand;
      }
      if (K + 1u > keep_key) keep_key = K + 1u;
    }
  }

  // draw
  const unsigned long long key =
      mix64(a.seed ^ mix64(((unsigned long long)(unsigned)a.row_request[row] << 32) | (unsigned)a.row_step[row]));
  ArgBest best{-INFINITY, 0x7fffffff};
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = vals[i] * mult;
    if (ordered_key(v) < keep_key || !(v == v)) continue;
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
  pdl_wait();
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

extern "C" int pe_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k,
                         float top_p, float min_p, unsigned long long seed, const int* row_request, const int* row_step,
                         int* out_tokens, cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (vocab <= 0 || ld < vocab) return PE_ERR_BAD_ARGUMENT;
  pe::SampleArgs a;
  a.logits = logits; a.ld = ld; a.n_rows = n_rows; a.vocab = vocab; a.temperature = temperature; a.top_k = top_k;
  a.top_p = top_p; a.min_p = min_p; a.seed = seed; a.row_request = row_request; a.row_step = row_step;
  a.out_tokens = out_tokens;
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
