// Row-wise and element-wise kernels: embedding gather, (residual +) RMSNorm, SiLU*mul,
// rotary encoding fused with the key/value cache write, row gather.
//
// Numerics follow the reference's op twins (turingserve/ops/reference.py:13-57) with the
// model-dtype rounding points of its Triton kernels (turingserve/ops/triton_rmsnorm.py:10-27,
// triton_silu_mul.py:10-18, triton_rope.py:10-24, triton_kv_write.py:10-25): statistics, the
// rotation and the activation are computed in 32-bit and rounded once.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Embedding: out[t, :] = table[ids[t], :]   (turingserve/model/qwen2.py:41)
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* src = table + (size_t)id * hidden;
  T* dst = out + (size_t)t * hidden;
  const int bytes = hidden * (int)sizeof(T);
  if ((bytes & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

TS_API int ts_embedding(void* out, const void* table, const int* ids, int T, int hidden, int vocab,
                        int dtype, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    ts_launch(embedding_kernel<float>, dim3(T), dim3(128), 0, s, (float*)out, (const float*)table, ids, hidden, vocab);
  else if (dtype == TS_BF16)
    ts_launch(embedding_kernel<bf16>, dim3(T), dim3(128), 0, s, (bf16*)out, (const bf16*)table, ids, hidden, vocab);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_embedding: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// Row gather: out[s, :] = x[rows[s], :]
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x,
                                   const int* __restrict__ rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const T* src = x + (size_t)rows[blockIdx.x] * width;
  T* dst = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

TS_API int ts_gather_rows(void* out, const void* x, const int* rows, int S, int width, int dtype,
                          void* stream) {
  if (S <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    ts_launch(gather_rows_kernel<float>, dim3(S), dim3(256), 0, s, (float*)out, (const float*)x, rows, width);
  else if (dtype == TS_BF16)
    ts_launch(gather_rows_kernel<bf16>, dim3(S), dim3(256), 0, s, (bf16*)out, (const bf16*)x, rows, width);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_gather_rows: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// RMSNorm, optionally with the residual add in front:
//   r = x (+ residual, rounded to T and stored back);  y = w * T(r32 * rsqrt(mean(r32^2) + eps))
// (turingserve/ops/reference.py:13-23).  One block per row; the row is read twice, the second
// time from cache.  WT is the scale's type: T, or float when the checkpoint stores it in 32-bit.
template <typename T, typename WT>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x, T* residual,
                               const WT* __restrict__ w, float eps, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f(x[base + i]);
    if (residual != nullptr) {
      v = round_to<T>(v + to_f(residual[base + i]));
      residual[base + i] = from_f<T>(v);
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  const T* src = residual != nullptr ? residual : x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float y = round_to<T>(to_f(src[base + i]) * rstd);
    out[base + i] = from_f<T>(to_f(w[i]) * y);
  }
}

// Latency-lean variant for rows whose length is a multiple of one 16-byte vector: every thread
// loads its vectors once, keeps them in registers across the reduction, and writes once.
template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<bf16> { static constexpr int N = 8; };

template <typename T, int N> __device__ __forceinline__ void load_vec(const T* p, float (&f)[N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = to_f(e[i]);
}
template <typename T, int N> __device__ __forceinline__ void store_vec(T* p, const float (&f)[N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = from_f<T>(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

template <typename T, typename WT, int CHUNKS>
__global__ void rmsnorm_vec_kernel(T* __restrict__ out, const T* __restrict__ x, T* residual,
                                   const WT* __restrict__ w, float eps, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float v[CHUNKS][N];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * N;
    if (i < hidden) {
      load_vec<T, N>(x + base + i, v[c]);
      if (residual != nullptr) {
        float r[N];
        load_vec<T, N>(residual + base + i, r);
#pragma unroll
        for (int k = 0; k < N; ++k) v[c][k] = round_to<T>(v[c][k] + r[k]);
        store_vec<T, N>(residual + base + i, v[c]);
      }
#pragma unroll
      for (int k = 0; k < N; ++k) ss += v[c][k] * v[c][k];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * N;
    if (i < hidden) {
      float y[N];
#pragma unroll
      for (int k = 0; k < N; ++k) y[k] = to_f(w[i + k]) * round_to<T>(v[c][k] * rstd);
      store_vec<T, N>(out + base + i, y);
    }
  }
}

template <typename T, typename WT>
bool launch_rmsnorm_vec(T* out, const T* x, T* residual, const WT* w, float eps, int rows, int hidden, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  if (hidden % N) return false;
  if (((uintptr_t)out | (uintptr_t)x | (uintptr_t)residual) & 15) return false;
  const int vecs = hidden / N;
  auto threads_for = [&](int chunks) { return ((vecs + chunks - 1) / chunks + 31) / 32 * 32; };
  if (threads_for(1) <= 1024)
    ts_launch(rmsnorm_vec_kernel<T, WT, 1>, dim3(rows), dim3(threads_for(1)), 0, s, out, x, residual, w, eps, hidden);
  else if (threads_for(2) <= 1024)
    ts_launch(rmsnorm_vec_kernel<T, WT, 2>, dim3(rows), dim3(threads_for(2)), 0, s, out, x, residual, w, eps, hidden);
  else if (threads_for(4) <= 1024)
    ts_launch(rmsnorm_vec_kernel<T, WT, 4>, dim3(rows), dim3(threads_for(4)), 0, s, out, x, residual, w, eps, hidden);
  else
    return false;
  return true;
}

TS_API int ts_rmsnorm(void* out, const void* x, void* residual, const void* w, float eps, int T,
                      int hidden, int dtype, int w_dtype, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  bool done = false;
  if (dtype == TS_F32 && w_dtype == TS_F32)
    done = launch_rmsnorm_vec<float, float>((float*)out, (const float*)x, (float*)residual, (const float*)w, eps, T, hidden, s);
  else if (dtype == TS_BF16 && w_dtype == TS_BF16)
    done = launch_rmsnorm_vec<bf16, bf16>((bf16*)out, (const bf16*)x, (bf16*)residual, (const bf16*)w, eps, T, hidden, s);
  else if (dtype == TS_BF16 && w_dtype == TS_F32)
    done = launch_rmsnorm_vec<bf16, float>((bf16*)out, (const bf16*)x, (bf16*)residual, (const float*)w, eps, T, hidden, s);
  if (done) {
    TS_LAUNCH_CHECK();
  }
  if (dtype == TS_F32 && w_dtype == TS_F32)
    ts_launch(rmsnorm_kernel<float, float>, dim3(T), dim3(threads), 0, s, (float*)out, (const float*)x, (float*)residual,
                                                       (const float*)w, eps, hidden);
  else if (dtype == TS_BF16 && w_dtype == TS_BF16)
    ts_launch(rmsnorm_kernel<bf16, bf16>, dim3(T), dim3(threads), 0, s, (bf16*)out, (const bf16*)x, (bf16*)residual,
                                                     (const bf16*)w, eps, hidden);
  else if (dtype == TS_BF16 && w_dtype == TS_F32)
    ts_launch(rmsnorm_kernel<bf16, float>, dim3(T), dim3(threads), 0, s, (bf16*)out, (const bf16*)x, (bf16*)residual,
                                                      (const float*)w, eps, hidden);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_rmsnorm: dtype %d with scale dtype %d", dtype, w_dtype);
  TS_LAUNCH_CHECK();
}

// The same norm, fed by a product that was left unreduced: x[row] = sum over splits (ascending) of
// part[s, row, :] + bias, rounded to bfloat16 as the product's own epilogue would have done; then
// residual add and norm as above.  Saves the separate reduction kernel after a split-K product.
template <typename WT, int CHUNKS>
__global__ void __launch_bounds__(256) reduce_rmsnorm_kernel(bf16* __restrict__ out, const float* __restrict__ part, int splits,
                                      size_t split_stride, const bf16* __restrict__ bias, bf16* residual,
                                      const WT* __restrict__ w, float eps, int hidden) {
  pdl_launch_dependents();
  // the scale and the bias are weights: their trip to memory overlaps the product's tail (the widest
  // rows, which have no registers to spare, fetch them where they are used instead)
  constexpr bool EARLY = CHUNKS < 8;
  float wv[EARLY ? CHUNKS : 1][8], bv[EARLY ? CHUNKS : 1][8];
  auto load_scale_bias = [&](int i, float (&ws)[8], float (&bs)[8]) {
#pragma unroll
    for (int k = 0; k < 8; k += Vec16<WT>::N) {
      float t[Vec16<WT>::N];
      load_vec<WT, Vec16<WT>::N>(w + i + k, t);
#pragma unroll
      for (int j = 0; j < Vec16<WT>::N; ++j) ws[k + j] = t[j];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) bs[k] = 0.f;
    if (bias != nullptr) load_vec<bf16, 8>(bias + i, bs);
  };
  if constexpr (EARLY) {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = (c * blockDim.x + threadIdx.x) * 8;
      if (i < hidden) load_scale_bias(i, wv[c], bv[c]);
    }
  }
  pdl_wait();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float v[CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    if (i < hidden) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (splits <= 16) {
        // all loads first (one round trip), then the sums in ascending split order
        float4 a[16], b[16];
#pragma unroll
        for (int sp = 0; sp < 16; ++sp)
          if (sp < splits) {
            a[sp] = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * split_stride + base + i));
            b[sp] = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * split_stride + base + i + 4));
          }
#pragma unroll
        for (int sp = 0; sp < 16; ++sp)
          if (sp < splits) {
            acc[0] += a[sp].x; acc[1] += a[sp].y; acc[2] += a[sp].z; acc[3] += a[sp].w;
            acc[4] += b[sp].x; acc[5] += b[sp].y; acc[6] += b[sp].z; acc[7] += b[sp].w;
          }
      } else {
        for (int sp = 0; sp < splits; ++sp) {
          const float4 a = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * split_stride + base + i));
          const float4 b = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * split_stride + base + i + 4));
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
          acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[c][k] = acc[k];
      if constexpr (EARLY) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] += bv[c][k];
      } else if (bias != nullptr) {
        float bl[8];
        load_vec<bf16, 8>(bias + i, bl);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] += bl[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[c][k] = round_to<bf16>(v[c][k]);
      if (residual != nullptr) {
        float r[8];
        load_vec<bf16, 8>(residual + base + i, r);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] = round_to<bf16>(v[c][k] + r[k]);
        store_vec<bf16, 8>(residual + base + i, v[c]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[c][k] * v[c][k];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    if (i < hidden) {
      float y[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        y[k] = (EARLY ? wv[EARLY ? c : 0][k] : to_f(w[i + k])) * round_to<bf16>(v[c][k] * rstd);
      store_vec<bf16, 8>(out + base + i, y);
    }
  }
}

// part: float [splits, T, hidden].  bfloat16 rows whose length is a multiple of 8 only.
TS_API int ts_reduce_rmsnorm(void* out, const float* part, int splits, const void* bias, void* residual,
                             const void* w, float eps, int T, int hidden, int w_dtype, void* stream) {
  if (T <= 0) return 0;
  if (hidden % 8 || splits < 1) TS_REFUSE(TS_ERR_SHAPE, "ts_reduce_rmsnorm: hidden %d, splits %d", hidden, splits);
  cudaStream_t s = (cudaStream_t)stream;
  const int vecs = hidden / 8;
  const size_t stride = (size_t)T * hidden;
  auto threads_for = [&](int chunks) { return ((vecs + chunks - 1) / chunks + 31) / 32 * 32; };
#define TS_RR(WT, CH) ts_launch(reduce_rmsnorm_kernel<WT, CH>, dim3(T), dim3(threads_for(CH)), 0, s, (bf16*)out, part, \
                                splits, stride, (const bf16*)bias, (bf16*)residual, (const WT*)w, eps, hidden)
  // at most 256 threads per row (the kernel keeps up to 16 partial sums per thread in registers)
  if (w_dtype == TS_BF16) {
    if (threads_for(1) <= 256) TS_RR(bf16, 1);
    else if (threads_for(2) <= 256) TS_RR(bf16, 2);
    else if (threads_for(4) <= 256) TS_RR(bf16, 4);
    else if (threads_for(8) <= 256) TS_RR(bf16, 8);
    else TS_REFUSE(TS_ERR_LIMIT, "ts_reduce_rmsnorm: hidden %d too large", hidden);
  } else if (w_dtype == TS_F32) {
    if (threads_for(1) <= 256) TS_RR(float, 1);
    else if (threads_for(2) <= 256) TS_RR(float, 2);
    else if (threads_for(4) <= 256) TS_RR(float, 4);
    else if (threads_for(8) <= 256) TS_RR(float, 8);
    else TS_REFUSE(TS_ERR_LIMIT, "ts_reduce_rmsnorm: hidden %d too large", hidden);
  } else {
    TS_REFUSE(TS_ERR_DTYPE, "ts_reduce_rmsnorm: scale dtype %d", w_dtype);
  }
#undef TS_RR
  TS_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// SiLU*mul: out[t, i] = T(silu(g_i)) * u_i (turingserve/ops/reference.py:26-28; rounding as
// triton_silu_mul.py:15-18).  Layout of gu[t]: group = 0: [g(0..I) | u(0..I)]; group = 64: blocks
// of 128 columns, each the 64 gates j*64.. then the 64 ups j*64.. (what a product with
// block-interleaved weight rows gives; the few-token tensor-core product applies the activation to
// such a tile in its own epilogue).
__device__ __forceinline__ size_t gate_col(int i, int group) { return group ? (size_t)(i / group) * 2 * group + i % group : (size_t)i; }

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, size_t total, int group) {
  pdl_launch_dependents();
  pdl_wait();
  const int up_off = group ? group : inter;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const size_t gc = t * 2 * inter + gate_col(i, group);
    const float g = to_f(gu[gc]);
    const float u = to_f(gu[gc + up_off]);
    const float s = round_to<T>(silu_for<T>(g));
    out[idx] = from_f<T>(s * u);
  }
}

// Vector variant: one thread takes 16 bytes of gate and 16 bytes of up.
template <typename T>
__global__ void silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, int vec_per_row,
                                    unsigned total_vecs, int group) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int N = Vec16<T>::N;
  const int up_off = group ? group : inter;
  for (unsigned v = blockIdx.x * blockDim.x + threadIdx.x; v < total_vecs; v += gridDim.x * blockDim.x) {
    const unsigned t = v / vec_per_row;
    const int i = (int)(v - t * vec_per_row) * N;
    float g[N], u[N], o[N];
    const size_t gc = (size_t)t * 2 * inter + gate_col(i, group);
    load_vec<T, N>(gu + gc, g);
    load_vec<T, N>(gu + gc + up_off, u);
#pragma unroll
    for (int k = 0; k < N; ++k) o[k] = round_to<T>(silu_for<T>(g[k])) * u[k];
    store_vec<T, N>(out + (size_t)t * inter + i, o);
  }
}

TS_API int ts_silu_mul_ex(void* out, const void* gu, int T, int inter, int group, int dtype, void* stream);

TS_API int ts_silu_mul(void* out, const void* gu, int T, int inter, int dtype, void* stream) {
  return ts_silu_mul_ex(out, gu, T, inter, 0, dtype, stream);
}

// group: 0, or the block size of an interleaved layout (a multiple of 8 that divides inter).
TS_API int ts_silu_mul_ex(void* out, const void* gu, int T, int inter, int group, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (group < 0 || (group > 0 && (inter % group != 0 || group % 8 != 0)))
    TS_REFUSE(TS_ERR_SHAPE, "ts_silu_mul: blocks of %d columns for a width of %d", group, inter);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t total = (size_t)T * inter;
  const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  {
    const int n = dtype == TS_F32 ? 4 : 8;
    const size_t vecs = total / n;
    if ((dtype == TS_F32 || dtype == TS_BF16) && inter % n == 0 && vecs < 0xffffffffull &&
        ((((uintptr_t)out | (uintptr_t)gu) & 15) == 0)) {
      const int vb = (int)((vecs + 255) / 256 > 148 * 32 ? 148 * 32 : (vecs + 255) / 256);
      if (dtype == TS_F32)
        ts_launch(silu_mul_vec_kernel<float>, dim3(vb), dim3(256), 0, s, (float*)out, (const float*)gu, inter, inter / n, (unsigned)vecs, group);
      else
        ts_launch(silu_mul_vec_kernel<bf16>, dim3(vb), dim3(256), 0, s, (bf16*)out, (const bf16*)gu, inter, inter / n, (unsigned)vecs, group);
      TS_LAUNCH_CHECK();
    }
  }
  if (dtype == TS_F32)
    ts_launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)out, (const float*)gu, inter, total, group);
  else if (dtype == TS_BF16)
    ts_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (bf16*)out, (const bf16*)gu, inter, total, group);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_silu_mul: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// Rotary encoding of q and k in place in qkv[T, (H+2KVH)*D], fused with the cache write of the
// rotated k and of v.  Rotate-half over the first `rot` dims of each head:
//   o[i] = x[i]*c - x[i+rot/2]*s,  o[i+rot/2] = x[i+rot/2]*c + x[i]*s,   c,s = T(table[pos, i])
// (turingserve/ops/reference.py:31-42).  Cache layout per run: [pages, KVH, page, D]; slot < 0
// skips the write (reference.py:50-57).  k_cache == nullptr: rotate only (a run that reads
// another run's cache).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     const int* __restrict__ slots, int H, int KVH, int D, int rot,
                                     int page) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = (k_cache != nullptr) ? slots[t] : -1;
  const int half = rot / 2;
  T* row = qkv + (size_t)t * (H + 2 * KVH) * D;
  size_t cache_base = 0;
  if (slot >= 0) cache_base = ((size_t)(slot / page) * KVH * page + (size_t)(slot % page)) * D;
  const size_t head_stride = (size_t)page * D;
  // q and k heads: pairs (i, i+half) for i < half, untouched dims rot..D-1
  const int pair_items = (H + KVH) * (D - half);   // per head: half pairs + (D - rot) pass-through
  for (int idx = threadIdx.x; idx < pair_items; idx += blockDim.x) {
    const int head = idx / (D - half);
    const int i = idx % (D - half);
    T* x = row + (size_t)head * D;
    const bool is_k = head >= H;
    T* kdst = (is_k && slot >= 0) ? k_cache + cache_base + (size_t)(head - H) * head_stride : nullptr;
    if (i < half) {
      const float c = round_to<T>(cos_t[(size_t)pos * half + i]);
      const float s = round_to<T>(sin_t[(size_t)pos * half + i]);
      const float x1 = to_f(x[i]), x2 = to_f(x[i + half]);
      const T o1 = from_f<T>(x1 * c - x2 * s);
      const T o2 = from_f<T>(x2 * c + x1 * s);
      x[i] = o1;
      x[i + half] = o2;
      if (kdst != nullptr) {
        kdst[i] = o1;
        kdst[i + half] = o2;
      }
    } else {
      const int d = rot + (i - half);
      if (kdst != nullptr) kdst[d] = x[d];
    }
  }
  if (slot >= 0) {
    const T* v = row + (size_t)(H + KVH) * D;
    for (int idx = threadIdx.x; idx < KVH * D; idx += blockDim.x) {
      const int head = idx / D, d = idx % D;
      v_cache[cache_base + (size_t)head * head_stride + d] = v[idx];
    }
  }
}

// Latency-lean variant for bfloat16 when half the rotary width is a multiple of 8: one thread
// rotates 8 pairs (two 16-byte vectors) or copies one 16-byte vector of v.
//
// With `part` set, the q/k/v product arrives unreduced: the value of column c of token t is
// sum over splits (ascending) of part[s, t, c] + bias[c], rounded to bfloat16 as the product's own
// epilogue would have rounded it; the kernel then writes q, k and v into qkv as well.
template <bool PART>
__device__ __forceinline__ void load_qkv8(const bf16* row, int col, const float* part, int splits, size_t split_stride,
                                          size_t part_row, const bf16* bias, float (&f)[8]) {
  if constexpr (!PART) {
    load_vec<bf16, 8>(row + col, f);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = 0.f;
    // eight splits' loads at a time (one round trip per eight), sums in ascending split order
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float4 a[8], b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < splits) {
          a[u] = __ldcg(reinterpret_cast<const float4*>(part + (size_t)(s0 + u) * split_stride + part_row + col));
          b[u] = __ldcg(reinterpret_cast<const float4*>(part + (size_t)(s0 + u) * split_stride + part_row + col + 4));
        }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < splits) {
          f[0] += a[u].x; f[1] += a[u].y; f[2] += a[u].z; f[3] += a[u].w;
          f[4] += b[u].x; f[5] += b[u].y; f[6] += b[u].z; f[7] += b[u].w;
        }
    }
    if (bias != nullptr) {
      float bv[8];
      load_vec<bf16, 8>(bias + col, bv);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += bv[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = round_to<bf16>(f[k]);
  }
}

// PART: the product arrives unreduced (`part` set).  A kernel of its own, because the partial sums
// held in registers would otherwise limit the plain kernel to a few resident warps (250 registers
// against 40: a 2,048-token portion took 22 us instead of 6).
template <bool PART>
__global__ void rope_kv_write_vec_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                         const int* __restrict__ slots, int H, int KVH, int D, int rot, int page,
                                         const float* __restrict__ part, int splits, size_t split_stride,
                                         const bf16* __restrict__ bias, int lph) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const size_t part_row = (size_t)t * (H + 2 * KVH) * D;
  // The step's index arrays come from the host before the step's first kernel: no kernel writes
  // them, so they are read ahead of the wait for the preceding kernel.
  const int pos = positions[t];
  const int slot = (k_cache != nullptr) ? slots[t] : -1;
  pdl_wait();
  const int half = rot / 2;
  const int hv = half / 8;                          // vectors per half
  const int pv = (D - rot) / 8;                     // pass-through vectors per head
  bf16* row = qkv + (size_t)t * (H + 2 * KVH) * D;
  size_t cache_base = 0;
  if (slot >= 0) cache_base = ((size_t)(slot / page) * KVH * page + (size_t)(slot % page)) * D;
  const size_t head_stride = (size_t)page * D;
  const int per_head = hv + pv;
  // `lph` lanes per head (q heads, k heads, then v heads): a whole warp where a few tokens must
  // spread over many blocks (and each lane has several partial sums to fetch), else just enough
  // lanes for a head's vectors so that no lane idles over a long prompt portion.
  const int hpw = 32 / lph;                                       // heads per warp
  const int head = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * hpw + (threadIdx.x & 31) / lph;
  const int lane = (threadIdx.x & 31) % lph;
  if (head >= H + 2 * KVH) return;
  if (head < H + KVH) {
    bf16* x = row + (size_t)head * D;
    bf16* kdst = (head >= H && slot >= 0) ? k_cache + cache_base + (size_t)(head - H) * head_stride : nullptr;
    for (int j = lane; j < per_head; j += lph) {
      if (j < hv) {
        const int i = j * 8;
        float x1[8], x2[8], o1[8], o2[8];
        load_qkv8<PART>(row, head * D + i, part, splits, split_stride, part_row, bias, x1);
        load_qkv8<PART>(row, head * D + i + half, part, splits, split_stride, part_row, bias, x2);
        const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i);
        const float4 c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i);
        const float4 s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i + 4);
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float c = round_to<bf16>(cs[k]), sv = round_to<bf16>(sn[k]);
          o1[k] = x1[k] * c - x2[k] * sv;
          o2[k] = x2[k] * c + x1[k] * sv;
        }
        store_vec<bf16, 8>(x + i, o1);
        store_vec<bf16, 8>(x + i + half, o2);
        if (kdst != nullptr) {
          store_vec<bf16, 8>(kdst + i, o1);
          store_vec<bf16, 8>(kdst + i + half, o2);
        }
      } else if (kdst != nullptr || PART) {
        const int d = rot + (j - hv) * 8;
        float pass[8];
        load_qkv8<PART>(row, head * D + d, part, splits, split_stride, part_row, bias, pass);
        if (PART) store_vec<bf16, 8>(x + d, pass);
        if (kdst != nullptr) store_vec<bf16, 8>(kdst + d, pass);
      }
    }
  } else if (slot >= 0 || PART) {
    const int vh = head - H - KVH;
    for (int j = lane; j < D / 8; j += lph) {
      const int d = j * 8;
      const int col = (H + KVH) * D + vh * D + d;
      float vv[8];
      load_qkv8<PART>(row, col, part, splits, split_stride, part_row, bias, vv);
      if (PART) store_vec<bf16, 8>(row + col, vv);
      if (slot >= 0) store_vec<bf16, 8>(v_cache + cache_base + (size_t)vh * head_stride + d, vv);
    }
  }
}

TS_API int ts_rope_kv_write_ex(void* qkv, const int* positions, const float* cos_t, const float* sin_t,
                               void* k_cache, void* v_cache, const int* slots, int T, int H, int KVH, int D, int rot,
                               int page, int dtype, const float* part, int splits, const void* bias, void* stream);

TS_API int ts_rope_kv_write(void* qkv, const int* positions, const float* cos_t, const float* sin_t,
                            void* k_cache, void* v_cache, const int* slots, int T, int H, int KVH,
                            int D, int rot, int page, int dtype, void* stream) {
  return ts_rope_kv_write_ex(qkv, positions, cos_t, sin_t, k_cache, v_cache, slots, T, H, KVH, D, rot, page, dtype,
                             nullptr, 0, nullptr, stream);
}

// Whether the kernel that also finishes an unreduced q/k/v product takes the shape.
TS_API int ts_rope_kv_write_fused_supported(int D, int rot, int dtype) {
  return dtype == TS_BF16 && rot > 0 && ((rot / 2) % 8) == 0 && (D % 8) == 0;
}

// `part` (float [splits, T, (H+2KVH)*D]) set: qkv is an OUTPUT too; see rope_kv_write_vec_kernel.
TS_API int ts_rope_kv_write_ex(void* qkv, const int* positions, const float* cos_t, const float* sin_t,
                               void* k_cache, void* v_cache, const int* slots, int T, int H, int KVH, int D, int rot,
                               int page, int dtype, const float* part, int splits, const void* bias, void* stream) {
  if (T <= 0) return 0;
  if (part != nullptr && !ts_rope_kv_write_fused_supported(D, rot, dtype))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_rope_kv_write: unreduced input with head_dim %d, rotary_dim %d", D, rot);
  if (rot < 0 || rot > D || (rot & 1)) TS_REFUSE(TS_ERR_SHAPE, "ts_rope_kv_write: rotary_dim %d for head_dim %d", rot, D);
  if (rot > 0 && (cos_t == nullptr || sin_t == nullptr)) TS_REFUSE(TS_ERR_SHAPE, "ts_rope_kv_write: tables missing");
  cudaStream_t s = (cudaStream_t)stream;
  const int half = rot / 2;
  const bool aligned = ((((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0);
  if (dtype == TS_BF16 && rot > 0 && (half % 8) == 0 && (D % 8) == 0 && aligned) {
    const int heads = H + 2 * KVH;
    int lph = 32;                                                  // lanes per head, a power of two
    if (T > 64) {
      const int vecs = half / 8 + (D - rot) / 8;                  // of a rotated head; a value head takes two turns
      lph = 1;
      while (lph < vecs && lph < 32) lph *= 2;
    }
    const int head_warps = ceil_div(heads, 32 / lph);
    const int warps = head_warps >= 4 ? 4 : head_warps;
    const dim3 grid(T, ceil_div(head_warps, warps)), block(warps * 32);
    const size_t stride = (size_t)T * (H + 2 * KVH) * D;
    if (part != nullptr)
      ts_launch(rope_kv_write_vec_kernel<true>, grid, block, 0, s, (bf16*)qkv, positions, cos_t, sin_t, (bf16*)k_cache,
                (bf16*)v_cache, slots, H, KVH, D, rot, page, part, splits, stride, (const bf16*)bias, lph);
    else
      ts_launch(rope_kv_write_vec_kernel<false>, grid, block, 0, s, (bf16*)qkv, positions, cos_t, sin_t, (bf16*)k_cache,
                (bf16*)v_cache, slots, H, KVH, D, rot, page, part, splits, stride, (const bf16*)bias, lph);
    TS_LAUNCH_CHECK();
  }
  if (part != nullptr) TS_REFUSE(TS_ERR_ALIGN, "ts_rope_kv_write: unreduced input needs 16-byte aligned buffers");
  if (dtype == TS_F32)
    ts_launch(rope_kv_write_kernel<float>, dim3(T), dim3(256), 0, s, (float*)qkv, positions, cos_t, sin_t, (float*)k_cache,
                                                  (float*)v_cache, slots, H, KVH, D, rot, page);
  else if (dtype == TS_BF16)
    ts_launch(rope_kv_write_kernel<bf16>, dim3(T), dim3(256), 0, s, (bf16*)qkv, positions, cos_t, sin_t, (bf16*)k_cache,
                                                 (bf16*)v_cache, slots, H, KVH, D, rot, page);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_rope_kv_write: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// Token feedback: ids[rows[i]] = tokens[src[i]].  Lets a decode step take its input ids straight
// from the previous step's sampler output on the device, so that the host can launch it before
// it has read those tokens.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ rows, const int* __restrict__ src,
                                   const int* __restrict__ tokens, int n, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    int t = tokens[src[i]];
    t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
    ids[rows[i]] = t;
  }
}

TS_API int ts_feed_tokens(int* ids, const int* rows, const int* src, const int* tokens, int n, int vocab, void* stream) {
  if (n <= 0) return 0;
  ts_launch(feed_tokens_kernel, dim3(ceil_div(n, 128)), dim3(128), 0, (cudaStream_t)stream, ids, rows, src, tokens, n, vocab);
  TS_LAUNCH_CHECK();
}
