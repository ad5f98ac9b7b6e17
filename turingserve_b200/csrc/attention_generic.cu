// Paged grouped-query attention, any sizes, 32-bit arithmetic: the engine's attention for the
// float32 path and for every shape the tensor-core kernels do not take.
//
// Semantics (turingserve/ops/reference.py:60-77,94-111): for request b with q_len new tokens and
// context seq_len (after the write), query token t at position p = seq_len - q_len + t sees keys
// j <= p (bottom-right causal mask), and with a window w only j >= p - w + 1; query head h reads
// kv head h / G; scores = q.k * scale; softmax and the weighted sum in 32-bit; a request with
// seq_len 0 gives zeros.  Keys and values come from the cache through the block table.
//
// Work split: one block per (tile of ROWS query rows, kv head, request), where a "row" is one
// (token, head-in-group) pair, so the G heads of a group share each key/value tile.  Keys are
// taken 32 at a time: lane j scores key j (full dot product over D from shared memory), the warp
// does the online-softmax update, then each lane accumulates its D/32 output dims.
#include "common.cuh"

namespace {

constexpr int ROWS = 16;     // query rows per block
constexpr int KT = 32;       // keys per tile (one per lane)
constexpr int NWARPS = 4;
constexpr int RPW = ROWS / NWARPS;
constexpr int MAX_DPL = 8;   // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(NWARPS * 32)
attention_generic_kernel(T* __restrict__ out, const T* __restrict__ qkv, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, const int* __restrict__ block_tables,
                         const int* __restrict__ q_start, const int* __restrict__ seq_lens,
                         int table_width, int H, int KVH, int D, int page, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = H / KVH;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int seq_len = seq_lens[b];
  const int row0 = blockIdx.x * ROWS;
  const int n_rows = q_len * G;
  if (row0 >= n_rows) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dpl = (D + 31) / 32;
  const int prefix = seq_len - q_len;
  const int qkv_stride = (H + 2 * KVH) * D;

  float* q_s = smem;                         // [ROWS][D]
  float* k_s = q_s + ROWS * D;               // [KT][D+1]
  float* v_s = k_s + KT * (D + 1);           // [KT][D]
  __shared__ size_t key_off[KT];

  // stage the query rows
  for (int idx = threadIdx.x; idx < ROWS * D; idx += blockDim.x) {
    const int r = idx / D, d = idx % D;
    const int row = row0 + r;
    float v = 0.f;
    if (row < n_rows) {
      const int t = row / G, g = row % G;
      v = to_f(qkv[(size_t)(qs + t) * qkv_stride + (size_t)(kvh * G + g) * D + d]);
    }
    q_s[idx] = v;
  }

  const int last_row = min(row0 + ROWS, n_rows) - 1;
  const int t_lo = row0 / G, t_hi = last_row / G;
  const int j_hi = prefix + t_hi;                                   // last key any row of the tile sees
  const int j_lo = window > 0 ? max(0, prefix + t_lo - window + 1) : 0;

  float m[RPW], l[RPW], acc[RPW][MAX_DPL];
  int p_row[RPW], lo_row[RPW];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) acc[r][i] = 0.f;
    const int row = row0 + warp * RPW + r;
    const int t = row / G;
    p_row[r] = (row < n_rows) ? prefix + t : -1;
    lo_row[r] = (window > 0) ? max(0, p_row[r] - window + 1) : 0;
  }

  if (seq_len > 0 && j_hi >= 0) {
    for (int j0 = j_lo; j0 <= j_hi; j0 += KT) {
      __syncthreads();
      if (threadIdx.x < KT) {
        const int j = j0 + threadIdx.x;
        size_t off = 0;
        if (j <= j_hi) {
          const int pg = block_tables[(size_t)b * table_width + j / page];
          off = (((size_t)pg * KVH + kvh) * page + (size_t)(j % page)) * D;
        }
        key_off[threadIdx.x] = off;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < KT * D; idx += blockDim.x) {
        const int kk = idx / D, d = idx % D;
        float kv = 0.f, vv = 0.f;
        if (j0 + kk <= j_hi) {
          kv = to_f(k_cache[key_off[kk] + d]);
          vv = to_f(v_cache[key_off[kk] + d]);
        }
        k_s[kk * (D + 1) + d] = kv;
        v_s[kk * D + d] = vv;
      }
      __syncthreads();
      const int j = j0 + lane;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        if (p_row[r] < j0) continue;                 // whole tile is in this row's future (warp-uniform)
        const float* qr = q_s + (warp * RPW + r) * D;
        const float* kr = k_s + lane * (D + 1);
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
        s *= scale;
        const bool ok = (j <= p_row[r]) && (j >= lo_row[r]);
        s = ok ? s : -INFINITY;
        const float m_new = fmaxf(m[r], warp_max(s));
        if (m_new == -INFINITY) continue;            // nothing visible yet (warp-uniform)
        const float p = ok ? expf(s - m_new) : 0.f;
        const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
        l[r] = l[r] * corr + warp_sum(p);
        m[r] = m_new;
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) acc[r][i] *= corr;
        for (int kk = 0; kk < KT; ++kk) {
          const float pk = __shfl_sync(0xffffffffu, p, kk);
          const float* vr = v_s + kk * D;
#pragma unroll
          for (int i = 0; i < MAX_DPL; ++i) {
            const int d = lane + 32 * i;
            if (i < dpl && d < D) acc[r][i] = fmaf(pk, vr[d], acc[r][i]);
          }
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int row = row0 + warp * RPW + r;
    if (row >= n_rows) continue;
    const int t = row / G, g = row % G;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    T* o = out + (size_t)(qs + t) * H * D + (size_t)(kvh * G + g) * D;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) {
      const int d = lane + 32 * i;
      if (i < dpl && d < D) o[d] = from_f<T>(acc[r][i] * inv);
    }
  }
}

template <typename T>
int launch(void* out, const void* qkv, const void* k_cache, const void* v_cache, const int* block_tables,
           const int* q_start, const int* seq_lens, int B, int table_width, int max_q_len, int H, int KVH,
           int D, int page, float scale, int window, cudaStream_t s) {
  const int G = H / KVH;
  const size_t smem = sizeof(float) * ((size_t)ROWS * D + (size_t)KT * (D + 1) + (size_t)KT * D);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  dim3 grid(ceil_div(max_q_len * G, ROWS), KVH, B);
  ts_launch(attention_generic_kernel<T>, dim3(grid), dim3(NWARPS * 32), smem, s, 
      (T*)out, (const T*)qkv, (const T*)k_cache, (const T*)v_cache, block_tables, q_start, seq_lens,
      table_width, H, KVH, D, page, scale, window);
  TS_LAUNCH_CHECK();
}

}  // namespace

// window <= 0: no window.
TS_API int ts_attention_generic(void* out, const void* qkv, const void* k_cache, const void* v_cache,
                                const int* block_tables, const int* q_start, const int* seq_lens, int B,
                                int table_width, int max_q_len, int H, int KVH, int D, int page,
                                float scale, int window, int dtype, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (KVH <= 0 || H % KVH) TS_REFUSE(TS_ERR_SHAPE, "ts_attention: %d heads over %d kv heads", H, KVH);
  if (D <= 0 || D > 32 * MAX_DPL) TS_REFUSE(TS_ERR_LIMIT, "ts_attention: head_dim %d (limit %d)", D, 32 * MAX_DPL);
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention: %d requests / %d kv heads per launch", B, KVH);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    return launch<float>(out, qkv, k_cache, v_cache, block_tables, q_start, seq_lens, B, table_width,
                         max_q_len, H, KVH, D, page, scale, window, s);
  if (dtype == TS_BF16)
    return launch<bf16>(out, qkv, k_cache, v_cache, block_tables, q_start, seq_lens, B, table_width,
                        max_q_len, H, KVH, D, page, scale, window, s);
  TS_REFUSE(TS_ERR_DTYPE, "ts_attention: dtype %d", dtype);
}
