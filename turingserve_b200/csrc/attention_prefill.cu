// Paged grouped-query attention for PROMPT PORTIONS in bfloat16: any number of new tokens per
// request, attending to the cache (earlier portions plus the new tokens, written just before).
//
// Counterpart of the reference's varlen paged causal FlashAttention kernel
// (turingserve/ops/triton_prefill_attention.py:17-79: prefix = seq_len - q_len, keys
// j <= prefix + i, probabilities rounded to the model dtype before the second product);
// semantics as turingserve/ops/reference.py:60-77,94-111, plus an optional window.
//
// Work split: one block per (tile of 64 query ROWS, kv head, request), where a row is one
// (token, head-in-group) pair: the G query heads of a kv head ride in the same tile and share
// every key/value tile, so keys and values are fetched once per group, not once per head.
// Each of the 4 warps owns 16 rows (one m16n8k16 row block).  Keys are streamed 64 at a time
// through a 3-stage cp.async pipeline into XOR-swizzled shared memory; scores, the online
// softmax and the output accumulator are 32-bit.  Tiles are issued longest-first (the last rows
// of a prompt see the most keys).
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int PF_WARPS = 4;
constexpr int PF_ROWS = PF_WARPS * 16;   // query rows per block
constexpr int PF_TILE = 64;              // keys per pipeline stage
constexpr int PF_STAGES = 3;
constexpr int PF_PAGES_S = 2048;        // block-table entries a block keeps in shared memory
constexpr float PF_LOG2E = 1.4426950408889634f;

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ qkv, const bf16* __restrict__ k_cache,
                         const bf16* __restrict__ v_cache, const int* __restrict__ block_tables,
                         const int* __restrict__ q_start, const int* __restrict__ seq_lens, int table_width,
                         int H, int KVH, int page, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CH = D / 8, KS = D / 16, NT = D / 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = H / KVH;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int seq_len = seq_lens[b];
  const int n_rows = q_len * G;
  const int n_row_tiles = (n_rows + PF_ROWS - 1) / PF_ROWS;
  if ((int)blockIdx.x >= n_row_tiles) return;
  const int row0 = (n_row_tiles - 1 - blockIdx.x) * PF_ROWS;       // longest tiles first
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int prefix = seq_len - q_len;
  const int qkv_stride = (H + 2 * KVH) * D;

  unsigned char* k_s = smem;
  unsigned char* v_s = smem + PF_STAGES * PF_TILE * D * 2;

  // this thread's two rows
  int pos[2];
  const bf16* qptr[2];
  bf16* optr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + warp * 16 + (lane >> 2) + 8 * r;
    if (row < n_rows) {
      const int t = row / G, g = row % G;
      pos[r] = prefix + t;
      qptr[r] = qkv + (size_t)(qs + t) * qkv_stride + (size_t)(kvh * G + g) * D;
      optr[r] = out + (size_t)(qs + t) * H * D + (size_t)(kvh * G + g) * D;
    } else {
      pos[r] = -1;                                                 // sees nothing, writes nothing
      qptr[r] = nullptr;
      optr[r] = nullptr;
    }
  }
  unsigned qf[KS][4];
  {
    const int kc = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int k = ks * 16 + kc;
      qf[ks][0] = qptr[0] ? *reinterpret_cast<const unsigned*>(qptr[0] + k) : 0u;
      qf[ks][1] = qptr[1] ? *reinterpret_cast<const unsigned*>(qptr[1] + k) : 0u;
      qf[ks][2] = qptr[0] ? *reinterpret_cast<const unsigned*>(qptr[0] + k + 8) : 0u;
      qf[ks][3] = qptr[1] ? *reinterpret_cast<const unsigned*>(qptr[1] + k + 8) : 0u;
    }
  }

  // keys any row of the block can see
  const int last_row = min(row0 + PF_ROWS, n_rows) - 1;
  const int j_hi = prefix + last_row / G;
  const int j_lo = window > 0 ? max(0, prefix + row0 / G - window + 1) : 0;
  const int n_tiles = (seq_len > 0 && j_hi >= j_lo) ? (j_hi - j_lo) / PF_TILE + 1 : 0;
  // rows of this warp: first and last position (warp-uniform), to skip tiles wholly outside
  const int w_first = row0 + warp * 16, w_last = min(w_first + 15, n_rows - 1);
  const int w_pos_lo = prefix + w_first / G, w_pos_hi = (w_first < n_rows) ? prefix + w_last / G : -1;

  // this block's part of the block table, once, in shared memory (no dependent global load per key)
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;      // pages of 2^k tokens: no division
  __shared__ int pages_s[PF_PAGES_S];
  const int page_first = j_lo / page;
  const int n_pages = n_tiles > 0 ? j_hi / page - page_first + 1 : 0;
  const bool pages_staged = n_pages <= PF_PAGES_S;
  if (pages_staged) {
    for (int i = threadIdx.x; i < n_pages; i += PF_WARPS * 32)
      pages_s[i] = block_tables[(size_t)b * table_width + page_first + i];
    __syncthreads();
  }

  auto load_tile = [&](int tile, int stage) {
    const int j0 = j_lo + tile * PF_TILE;
    unsigned char* ks_ = k_s + stage * PF_TILE * D * 2;
    unsigned char* vs_ = v_s + stage * PF_TILE * D * 2;
    for (int idx = threadIdx.x; idx < PF_TILE * CH; idx += PF_WARPS * 32) {
      const int key = idx / CH, c = idx % CH;
      const int j = j0 + key;
      const bool ok = j <= j_hi;
      size_t off = 0;
      if (ok) {
        const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page);
        const int pg = pages_staged ? pages_s[lp - page_first] : block_tables[(size_t)b * table_width + lp];
        off = (((size_t)pg * KVH + kvh) * page + (size_t)(j - lp * page)) * D + c * 8;
      }
      cp_async_16(ks_ + swz<D>(key, c), k_cache + off, ok);
      cp_async_16(vs_ + swz<D>(key, c), v_cache + off, ok);
    }
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sc = scale * PF_LOG2E;

#pragma unroll
  for (int s = 0; s < PF_STAGES - 1; ++s) {
    if (s < n_tiles) load_tile(s, s);
    cp_async_commit();
  }
  for (int t = 0; t < n_tiles; ++t) {
    if (t + PF_STAGES - 1 < n_tiles) load_tile(t + PF_STAGES - 1, (t + PF_STAGES - 1) % PF_STAGES);
    cp_async_commit();
    cp_async_wait<PF_STAGES - 1>();
    __syncthreads();
    const unsigned char* ks_ = k_s + (t % PF_STAGES) * PF_TILE * D * 2;
    const unsigned char* vs_ = v_s + (t % PF_STAGES) * PF_TILE * D * 2;
    const int j0 = j_lo + t * PF_TILE;
    const bool in_future = j0 > w_pos_hi;                                          // warp-uniform
    const bool in_past = window > 0 && (j0 + PF_TILE - 1) < (w_pos_lo - window + 1);
    if (!in_future && !in_past) {
      float s_acc[PF_TILE / 8][4];
#pragma unroll
      for (int nt = 0; nt < PF_TILE / 8; ++nt) s_acc[nt][0] = s_acc[nt][1] = s_acc[nt][2] = s_acc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < PF_TILE / 16; ++np) {                // pairs of 8-key n-tiles
          const int mat = lane >> 3, r = lane & 7;
          const int key = np * 16 + (mat >> 1) * 8 + r;
          const int c = ks * 2 + (mat & 1);
          unsigned b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, ks_ + swz<D>(key, c));
          mma_bf16(s_acc[2 * np], qf[ks], b0, b1);
          mma_bf16(s_acc[2 * np + 1], qf[ks], b2, b3);
        }
      }
      // mask + online softmax
      const bool need_mask = (j0 + PF_TILE - 1 > w_pos_lo) || (window > 0) || (j0 + PF_TILE - 1 > j_hi);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < PF_TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s_acc[nt][e] * sc;
          if (need_mask) {
            const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            const int p = pos[e >> 1];
            const bool ok = (j <= p) && (window <= 0 || j > p - window);
            v = ok ? v : -INFINITY;
          }
          s_acc[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;             // a row that has seen nothing yet
        corr[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < PF_TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s_acc[nt][e] - m_use[e >> 1]);
          s_acc[nt][e] = p;
          rs[e >> 1] += p;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        l_run[r] = l_run[r] * corr[r] + rs[r];
      }
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      // O += P . V, 16 keys (one k-step) at a time
#pragma unroll
      for (int kk = 0; kk < PF_TILE / 16; ++kk) {
        unsigned pf[4];
        pf[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
        pf[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
        pf[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
        pf[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
        for (int i = 0; i < NT; i += 2) {
          const int mat = lane >> 3, r = lane & 7;
          const int key = kk * 16 + (mat & 1) * 8 + r;
          const int c = i + (mat >> 1);
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + swz<D>(key, c));
          mma_bf16(o[i], pf, b0, b1);
          mma_bf16(o[i + 1], pf, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (optr[r] == nullptr) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<__nv_bfloat162*>(optr[r] + d) =
          __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
  }
}

template <int D>
int launch_prefill(bf16* out, const bf16* qkv, const bf16* k_cache, const bf16* v_cache, const int* block_tables,
                   const int* q_start, const int* seq_lens, int B, int table_width, int max_q_len, int H, int KVH,
                   int page, float scale, int window, cudaStream_t s) {
  const size_t smem = (size_t)2 * PF_STAGES * PF_TILE * D * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int G = H / KVH;
  dim3 grid(ceil_div(max_q_len * G, PF_ROWS), KVH, B);
  ts_launch(attention_prefill_kernel<D>, dim3(grid), dim3(PF_WARPS * 32), smem, s, out, qkv, k_cache, v_cache, block_tables, q_start,
                                                              seq_lens, table_width, H, KVH, page, scale, window);
  TS_LAUNCH_CHECK();
}

}  // namespace

TS_API int ts_attention_prefill_supported(int H, int KVH, int D, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && (D == 64 || D == 128);
}

TS_API int ts_attention_prefill(void* out, const void* qkv, const void* k_cache, const void* v_cache,
                                const int* block_tables, const int* q_start, const int* seq_lens, int B,
                                int table_width, int max_q_len, int H, int KVH, int D, int page, float scale,
                                int window, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (!ts_attention_prefill_supported(H, KVH, D, TS_BF16))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_prefill: H=%d KVH=%d D=%d is not taken by this kernel", H, KVH, D);
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_prefill: %d requests / %d kv heads", B, KVH);
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 64)
    return launch_prefill<64>((bf16*)out, (const bf16*)qkv, (const bf16*)k_cache, (const bf16*)v_cache, block_tables,
                              q_start, seq_lens, B, table_width, max_q_len, H, KVH, page, scale, window, s);
  return launch_prefill<128>((bf16*)out, (const bf16*)qkv, (const bf16*)k_cache, (const bf16*)v_cache, block_tables,
                             q_start, seq_lens, B, table_width, max_q_len, H, KVH, page, scale, window, s);
}
