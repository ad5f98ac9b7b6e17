// Sampling on the device: logit edits (penalties, stop-token masking) and the draw
// (greedy / temperature / top-k / top-p / exponential race), one block per logits row.
//
// Order and formulas follow turingserve/sampling/sampler.py:45-107 and
// turingserve/sampling/penalties.py:20-45:
//   bad row (a NaN or +inf logit; -inf marks a masked entry) -> flagged; greedy -> first index of the maximum;
//   otherwise scaled = logits / temperature; keep the top_k largest; p = softmax over the kept;
//   walking down in value, an entry is dropped once the mass before it reaches top_p (the first is
//   always kept); p = softmax over what remains; token = argmax(p / E), E ~ Exp(1).
// Where the reference sorts, this kernel finds the two value thresholds by radix selection over
// order-preserving integer keys (four 8-bit passes each), so equal values are kept or dropped
// together.  E comes from Philox4x32-10 keyed by the request's seed, counter = (vocabulary index,
// number of tokens the request has drawn so far).
#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                      uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

// E ~ Exp(1) for vocabulary entry i of a request's `drawn`-th draw.
__device__ __forceinline__ float exponential(uint64_t seed, uint64_t drawn, uint32_t i) {
  const uint32_t r = philox_first_word(i, (uint32_t)drawn, (uint32_t)(drawn >> 32), 0u,
                                       (uint32_t)seed, (uint32_t)(seed >> 32));
  const float u = ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f);    // (0, 1)
  return -logf(u);
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ Best block_best(Best x, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  Best t = scratch[lane < nw ? lane : 0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = better(t, y);
  }
  return t;
}

// The draw is the last kernel of a step and its output the one thing the host waits for: the
// first block copies the status words of the kernels with bounded waits out beside the tokens, so
// that a block that gave up somewhere in the step is seen with the step's own tokens.
__device__ __forceinline__ void report_status(bool mine, const TsStatusPtrs& src, int* __restrict__ out) {
  if (mine && out != nullptr && threadIdx.x < TS_STATUS_WORDS)
    out[threadIdx.x] = src.p[threadIdx.x] != nullptr ? *reinterpret_cast<const volatile int*>(src.p[threadIdx.x]) : 0;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ tokens, int* __restrict__ bad_out, const float* __restrict__ logits,
              const float* __restrict__ fparams, const long long* __restrict__ iparams, int V,
              const TsStatusPtrs status_src, int* __restrict__ status_out) {
  pdl_launch_dependents();
  pdl_wait();
  report_status(blockIdx.x == 0, status_src, status_out);
  __shared__ Best best_s[32];
  __shared__ float red_s[32];
  __shared__ int cnt_s[256];
  __shared__ float mass_s[256];
  __shared__ uint32_t sel_prefix;
  __shared__ float sel_above;
  __shared__ int sel_k;
  __shared__ int any_bad;

  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * V;
  const float temp = fparams[row * 2 + 0], top_p = fparams[row * 2 + 1];
  const long long top_k = iparams[row * 4 + 0];
  const uint64_t seed = (uint64_t)iparams[row * 4 + 1], drawn = (uint64_t)iparams[row * 4 + 2];

  if (threadIdx.x == 0) any_bad = 0;
  __syncthreads();
  Best b{-INFINITY, 0x7fffffff};
  bool bad = false;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (isnan(v) || v == INFINITY) bad = true;       // -inf is a masked entry, not a fault
    b = better(b, Best{v, i});
  }
  if (bad) any_bad = 1;
  b = block_best(b, best_s);        // has __syncthreads inside: any_bad is visible after it
  if (any_bad) {
    if (threadIdx.x == 0) {
      tokens[row] = 0;
      bad_out[row] = 1;
    }
    return;
  }
  if (threadIdx.x == 0) bad_out[row] = 0;
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) tokens[row] = b.i;
    return;
  }
  const float m = b.v / temp;
  uint32_t keep_from = 0u;          // entries with order_key >= keep_from are kept

  if (top_k > 0 && top_k < V) {     // exact key of the top_k-th largest value
    if (threadIdx.x == 0) {
      sel_prefix = 0u;
      sel_k = (int)top_k;
    }
    uint32_t mask = 0u;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (threadIdx.x < 256) cnt_s[threadIdx.x] = 0;
      __syncthreads();
      const uint32_t prefix = sel_prefix;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const uint32_t k = order_key(x[i] / temp);
        if ((k & mask) == prefix) atomicAdd(&cnt_s[(k >> shift) & 255u], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int k = sel_k, chosen = 0;
        for (int bin = 255; bin >= 0; --bin) {
          if (k <= cnt_s[bin]) {
            chosen = bin;
            break;
          }
          k -= cnt_s[bin];
        }
        sel_k = k;
        sel_prefix = prefix | ((uint32_t)chosen << shift);
      }
      mask |= 255u << shift;
      __syncthreads();
    }
    keep_from = sel_prefix;
  }

  if (top_p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float s = x[i] / temp;
      if (order_key(s) >= keep_from) z += expf(s - m);
    }
    z = block_sum(z, red_s);
    const float limit = top_p * z;
    if (threadIdx.x == 0) {
      sel_prefix = 0u;
      sel_above = 0.f;
    }
    uint32_t mask = 0u;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (threadIdx.x < 256) {
        cnt_s[threadIdx.x] = 0;
        mass_s[threadIdx.x] = 0.f;
      }
      __syncthreads();
      const uint32_t prefix = sel_prefix;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float s = x[i] / temp;
        const uint32_t k = order_key(s);
        if (k >= keep_from && (k & mask) == prefix) {
          atomicAdd(&cnt_s[(k >> shift) & 255u], 1);
          atomicAdd(&mass_s[(k >> shift) & 255u], expf(s - m));
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        float above = sel_above, above_chosen = sel_above;
        int chosen = 255;
        for (int bin = 255; bin >= 0; --bin) {
          if (cnt_s[bin] == 0) continue;
          if (!(above < limit)) break;
          chosen = bin;
          above_chosen = above;
          above += mass_s[bin];
        }
        sel_above = above_chosen;
        sel_prefix = prefix | ((uint32_t)chosen << shift);
      }
      mask |= 255u << shift;
      __syncthreads();
    }
    keep_from = max(keep_from, sel_prefix);
  }

  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float s = x[i] / temp;
    if (order_key(s) >= keep_from) z += expf(s - m);
  }
  z = block_sum(z, red_s);
  Best w{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float s = x[i] / temp;
    if (order_key(s) < keep_from) continue;
    const float p = expf(s - m) / z;
    w = better(w, Best{p / exponential(seed, drawn, (uint32_t)i), i});
  }
  w = block_best(w, best_s);
  if (threadIdx.x == 0) tokens[row] = w.i;
}

// Greedy rows only: the row's vocabulary is cut into gridDim.x parts, one block each, so that a
// handful of rows still reads at the speed of many SMs; the block that finishes last for a row
// (a ticket counter: nobody waits) picks among the parts' candidates.  Same result as
// sample_kernel with temperature 0: first index of the maximum, or token 0 and the bad flag when the
// row holds a NaN or +inf.
constexpr int GREEDY_THREADS = 256;

__global__ void __launch_bounds__(GREEDY_THREADS)
sample_greedy_kernel(int* __restrict__ tokens, int* __restrict__ bad_out, const float* __restrict__ logits, int V,
                     float* __restrict__ part_v, int* __restrict__ part_i, int* __restrict__ counters,
                     const TsStatusPtrs status_src, int* __restrict__ status_out) {
  pdl_launch_dependents();
  pdl_wait();
  report_status(blockIdx.x == 0 && blockIdx.y == 0, status_src, status_out);
  __shared__ Best best_s[32];
  __shared__ int any_bad;
  __shared__ int is_last;
  const int row = blockIdx.y, part = blockIdx.x, P = gridDim.x;
  const float* x = logits + (size_t)row * V;
  const int len = (V + P - 1) / P;
  const int lo = part * len, hi = min(V, lo + len);
  if (threadIdx.x == 0) any_bad = 0;
  __syncthreads();
  Best b{-INFINITY, 0x7fffffff};
  bool bad = false;
  for (int i = lo + threadIdx.x; i < hi; i += GREEDY_THREADS) {
    const float v = x[i];
    if (isnan(v) || v == INFINITY) bad = true;
    b = better(b, Best{v, i});
  }
  if (bad) any_bad = 1;
  b = block_best(b, best_s);
  if (threadIdx.x == 0) {
    part_v[row * P + part] = b.v;
    part_i[row * P + part] = any_bad ? -1 : b.i;          // -1: this part saw a bad value
    __threadfence();
    const int ticket = atomicAdd(&counters[row], 1);
    is_last = (ticket == P - 1);
    if (is_last) counters[row] = 0;                        // ready for the next launch
  }
  __syncthreads();
  if (!is_last || threadIdx.x >= 32) return;
  __threadfence();
  Best w{-INFINITY, 0x7fffffff};
  bool row_bad = false;
  for (int p = threadIdx.x; p < P; p += 32) {
    const float v = __ldcg(part_v + row * P + p);
    const int i = __ldcg(part_i + row * P + p);
    if (i < 0) row_bad = true;
    else w = better(w, Best{v, i});
  }
  row_bad = __any_sync(0xffffffffu, row_bad);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, w.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, w.i, o);
    w = better(w, y);
  }
  if (threadIdx.x == 0) {
    tokens[row] = row_bad ? 0 : w.i;
    bad_out[row] = row_bad ? 1 : 0;
  }
}

// Logit edits.  meta[row] = {a, b, c, d}: ids[a:b] prompt tokens, ids[b:c] output tokens (both
// empty when the row has no penalties), ids[c:d] tokens to mask to -inf.  pen[row] = {repetition,
// presence, frequency}.  seen = prompt or output: logit > 0 ? logit / rep : logit * rep; then
// logit -= frequency * count_in_output; then logit -= presence * (count_in_output > 0).
__global__ void penalize_kernel(float* __restrict__ logits, const int* __restrict__ ids,
                                const int* __restrict__ meta, const float* __restrict__ pen, int V) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ uint32_t bits[];           // [2][ceil(V/32)]: seen, seen-in-output
  const int words = (V + 31) / 32;
  uint32_t* seen = bits;
  uint32_t* seen_out = bits + words;
  const int row = blockIdx.x;
  float* x = logits + (size_t)row * V;
  const int a = meta[row * 8 + 0], b = meta[row * 8 + 1], c = meta[row * 8 + 2], d = meta[row * 8 + 3];
  const float rep = pen[row * 4 + 0], presence = pen[row * 4 + 1], frequency = pen[row * 4 + 2];
  for (int i = threadIdx.x; i < 2 * words; i += blockDim.x) bits[i] = 0u;
  __syncthreads();
  for (int i = a + threadIdx.x; i < c; i += blockDim.x) {
    const int t = ids[i];
    if (t < 0 || t >= V) continue;
    const uint32_t bit = 1u << (t & 31);
    const uint32_t old = atomicOr(&seen[t >> 5], bit);
    if (!(old & bit)) {                        // first sighting: repetition penalty, once
      const float v = x[t];
      x[t] = v > 0.f ? v / rep : v * rep;
    }
  }
  __syncthreads();
  for (int i = b + threadIdx.x; i < c; i += blockDim.x) {
    const int t = ids[i];
    if (t < 0 || t >= V) continue;
    const uint32_t bit = 1u << (t & 31);
    const uint32_t old = atomicOr(&seen_out[t >> 5], bit);
    if (!(old & bit)) {
      int count = 0;
      for (int j = b; j < c; ++j) count += (ids[j] == t);
      float v = x[t];
      v = v - frequency * (float)count;
      v = v - presence * 1.0f;
      x[t] = v;
    }
  }
  __syncthreads();
  for (int i = c + threadIdx.x; i < d; i += blockDim.x) {
    const int t = ids[i];
    if (t >= 0 && t < V) x[t] = -INFINITY;
  }
}

}  // namespace

// out[0:S] tokens, out[S:2S] bad flags; status_out (may be null): TS_STATUS_WORDS ints that receive
// the status words of the kernels with bounded waits as they stand when the draw runs.
TS_API int ts_sample(int* out, const float* logits, const float* fparams, const long long* iparams, int S,
                     int V, int* status_out, void* stream) {
  if (S <= 0) return 0;
  if (V <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_sample: vocabulary %d", V);
  ts_launch(sample_kernel, dim3(S), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, out, out + S, logits, fparams, iparams, V,
            ts_status_ptrs(), status_out);
  TS_LAUNCH_CHECK();
}

// Parts a row is cut into by ts_sample_greedy: scratch holds 2 * S * parts 4-byte words, counters S
// ints that are zero on entry (the kernel leaves them zero).
TS_API int ts_sample_greedy_parts(int V) {
  const int p = (V + 4095) / 4096;
  return p < 1 ? 1 : (p > 64 ? 64 : p);
}

// Every row greedy: out[0:S] tokens, out[S:2S] bad flags, as ts_sample with temperature 0 gives them.
TS_API int ts_sample_greedy(int* out, const float* logits, int S, int V, void* scratch, int* counters, int* status_out,
                            void* stream) {
  if (S <= 0) return 0;
  if (V <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_sample_greedy: vocabulary %d", V);
  if (S > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_sample_greedy: %d rows", S);
  if (scratch == nullptr || counters == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_sample_greedy: scratch and counters are needed");
  const int P = ts_sample_greedy_parts(V);
  float* pv = (float*)scratch;
  int* pi = (int*)scratch + (size_t)S * P;
  ts_launch(sample_greedy_kernel, dim3(P, S), dim3(GREEDY_THREADS), 0, (cudaStream_t)stream, out, out + S, logits, V, pv, pi, counters,
            ts_status_ptrs(), status_out);
  TS_LAUNCH_CHECK();
}

TS_API int ts_penalize(float* logits, const int* ids, const int* meta, const float* pen, int S, int V,
                       void* stream) {
  if (S <= 0) return 0;
  const size_t smem = 2 * (size_t)((V + 31) / 32) * sizeof(uint32_t);
  if (smem > 200 * 1024) TS_REFUSE(TS_ERR_LIMIT, "ts_penalize: vocabulary %d too large", V);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(penalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_penalize: %s", cudaGetErrorString(e));
    configured = smem;
  }
  ts_launch(penalize_kernel, dim3(S), dim3(256), smem, (cudaStream_t)stream, logits, ids, meta, pen, V);
  TS_LAUNCH_CHECK();
}
