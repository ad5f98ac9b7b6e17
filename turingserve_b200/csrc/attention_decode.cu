// Paged grouped-query DECODE attention in bfloat16 (one new token per request), split over the
// keys so that a small batch still fills the GPU.
//
// Counterpart of the reference's split-K flash-decoding kernels
// (turingserve/ops/triton_decode_attention.py:101-163: partial (m, l, acc) per partition, then a
// reduce kernel) and of its grouped kernel (:60-95: the G query heads of a kv head share every
// key/value tile).  Semantics as turingserve/ops/reference.py:60-77,94-111 for q_len = 1.
//
// Work split: one block per (key split, kv head, request); 4 warps.  The block streams its share
// of the keys in tiles of 64 through a 3-stage cp.async pipeline into XOR-swizzled shared memory;
// warp w owns keys 16w..16w+15 of every tile.  The G query heads sit in the 16 rows of one
// mma.sync m16n8k16 tile (rows >= G are zero), scores and the softmax state are 32-bit, the
// probabilities are rounded to bfloat16 for the second product as the reference does
// (triton_prefill_attention.py:58).  Warps keep independent online-softmax states over disjoint
// keys and merge them through shared memory at the end; with more than one split the block
// writes an unnormalised partial (m, l, acc) to scratch, and the block that finishes last for a
// (request, kv head) merges the partials (no second launch, no waiting: a ticket counter).  With 2,
// 4 or 8 splits (16 in a launch of few blocks) the splits are one thread-block cluster instead: the
// partial stays in shared memory and every block sums its share of the output out of its peers'.
#include <mutex>

#include "common.cuh"
#include "mma_utils.cuh"
#include "no_alloc.h"

namespace {

constexpr int DEC_STAGES = 3;
// WARPS warps a block, 16 keys of every tile each: 4 (tiles of 64 keys, two blocks an SM), or 8 (tiles of
// 128 keys, one block an SM) where 8 splits of 8 warps can be one cluster per (request, kv head) and all
// clusters fit the chip: the same keys per warp as 16 splits of 4 warps, half the partial results, and
// those merged through the cluster's shared memory instead of scratch, a fence and a ticket.
constexpr int PAGES_S = 1024;       // block-table entries a block keeps in shared memory
constexpr float LOG2E = 1.4426950408889634f;

// Thread-block clusters: the splits of one (request, kv head) are the blocks of one cluster and read
// each other's merged states from shared memory.
// CLUSTER: the grid's x dimension (the splits) is one cluster; nsplit is then a power of two <= 16.
template <int D, bool CLUSTER, int DEC_WARPS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(bf16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                        const bf16* __restrict__ qkv, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, const int* __restrict__ block_tables,
                        const int* __restrict__ q_start, const int* __restrict__ seq_lens, int table_width,
                        int H, int KVH, int page, float scale, int window, int nsplit, int* __restrict__ counters) {
  // Everything up to pdl_wait() reads only what no kernel of this step writes: the step's index
  // arrays (copied from the host before the step's first kernel) and cache rows of earlier steps.
  // The one row this step writes, the new token's at seq_len - 1, is fetched after the wait.
  pdl_launch_dependents();
  constexpr int DEC_TILE = 16 * DEC_WARPS;        // keys per pipeline stage
  constexpr int CH = D / 8;                       // 16-byte chunks per row
  constexpr int KS = D / 16;                      // k-steps of the score product
  constexpr int NT = D / 8;                       // n-tiles of the output
  extern __shared__ __align__(128) unsigned char smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = H / KVH;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq_len = seq_lens[b];
  const int row_q = q_start[b];                   // the request's single query token
  const int lo = (window > 0) ? max(0, seq_len - window) : 0;
  const int span = max(seq_len - lo, 0);
  int chunk = (span + nsplit - 1) / nsplit;
  chunk = (chunk + DEC_TILE - 1) / DEC_TILE * DEC_TILE;
  const int k_begin = lo + split * chunk;
  const int k_end = min(seq_len, k_begin + chunk);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + DEC_TILE - 1) / DEC_TILE : 0;

  unsigned char* k_s = smem;                                       // [STAGES][TILE][D] bf16
  unsigned char* v_s = smem + DEC_STAGES * DEC_TILE * D * 2;

  // The block's share of the block table goes to shared memory once: the copies below then need no
  // dependent global load per key.
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;      // pages of 2^k tokens: no division
  __shared__ int pages_s[PAGES_S];
  const int page_first = k_begin / page;
  const int n_pages = k_end > k_begin ? (k_end - 1) / page - page_first + 1 : 0;
  const bool pages_staged = n_pages <= PAGES_S;
  if (pages_staged) {
    for (int i = threadIdx.x; i < n_pages; i += DEC_WARPS * 32)
      pages_s[i] = block_tables[(size_t)b * table_width + page_first + i];
    __syncthreads();
  }

  // `skip`: a key whose row is left alone (no copy, no zero fill), to be fetched later.  Two copies
  // into the same shared-memory bytes would land in no defined order.
  auto load_tile = [&](int tile, int stage, int skip) {
    const int j0 = k_begin + tile * DEC_TILE;
    unsigned char* ks_ = k_s + stage * DEC_TILE * D * 2;
    unsigned char* vs_ = v_s + stage * DEC_TILE * D * 2;
    for (int idx = threadIdx.x; idx < DEC_TILE * CH; idx += DEC_WARPS * 32) {
      const int key = idx / CH, c = idx % CH;
      const int j = j0 + key;
      if (j == skip) continue;
      const bool ok = j < k_end;
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

  // First tiles of the pipeline, without the new token's row.
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < n_tiles) load_tile(s, s, seq_len - 1);
    cp_async_commit();
  }
  pdl_wait();
  // The new token's row, if it lies in a tile fetched above; later tiles take it with them.
  const int new_tile = (k_end == seq_len && n_tiles > 0) ? (seq_len - 1 - k_begin) / DEC_TILE : -1;
  const bool patch = new_tile >= 0 && new_tile < DEC_STAGES - 1;       // block-uniform
  if (patch && threadIdx.x < CH) {
    const int j = seq_len - 1, key = j - k_begin - new_tile * DEC_TILE, c = threadIdx.x;
    const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page);
    const int pg = pages_staged ? pages_s[lp - page_first] : block_tables[(size_t)b * table_width + lp];
    const size_t off = (((size_t)pg * KVH + kvh) * page + (size_t)(j - lp * page)) * D + c * 8;
    cp_async_16(k_s + new_tile * DEC_TILE * D * 2 + swz<D>(key, c), k_cache + off, true);
    cp_async_16(v_s + new_tile * DEC_TILE * D * 2 + swz<D>(key, c), v_cache + off, true);
  }
  if (patch) cp_async_commit();

  // query fragments: rows 0..G-1 of the group, zero above
  unsigned qf[KS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, kc = (lane & 3) * 2;
    const bf16* qbase = qkv + (size_t)row_q * (H + 2 * KVH) * D + (size_t)kvh * G * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int k = ks * 16 + kc;
      qf[ks][0] = r0 < G ? *reinterpret_cast<const unsigned*>(qbase + r0 * D + k) : 0u;
      qf[ks][1] = r1 < G ? *reinterpret_cast<const unsigned*>(qbase + r1 * D + k) : 0u;
      qf[ks][2] = r0 < G ? *reinterpret_cast<const unsigned*>(qbase + r0 * D + k + 8) : 0u;
      qf[ks][3] = r1 < G ? *reinterpret_cast<const unsigned*>(qbase + r1 * D + k + 8) : 0u;
    }
  }

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sc = scale * LOG2E;

  for (int t = 0; t < n_tiles; ++t) {
    if (t + DEC_STAGES - 1 < n_tiles) load_tile(t + DEC_STAGES - 1, (t + DEC_STAGES - 1) % DEC_STAGES, -1);
    cp_async_commit();
    // Groups, oldest first: the STAGES-1 first tiles, the patch group if there is one, then one per
    // iteration.  The patched tile needs the patch group too, hence the full wait up to it.
    if (patch && t <= new_tile) cp_async_wait<0>();
    else cp_async_wait<DEC_STAGES - 1>();
    __syncthreads();
    const unsigned char* ks_ = k_s + (t % DEC_STAGES) * DEC_TILE * D * 2;
    const unsigned char* vs_ = v_s + (t % DEC_STAGES) * DEC_TILE * D * 2;
    const int key0 = warp * 16;                                    // this warp's keys in the tile
    const int j_base = k_begin + t * DEC_TILE + key0;
    if (j_base < k_end) {                                          // warp-uniform
      // scores S[16 x 16] = Q . K^T
      float s_acc[2][4] = {};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        // matrices: (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
        const int mat = lane >> 3, r = lane & 7;
        const int key = key0 + (mat >> 1) * 8 + r;
        const int c = ks * 2 + (mat & 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks_ + swz<D>(key, c));
        mma_bf16(s_acc[0], qf[ks], b0, b1);
        mma_bf16(s_acc[1], qf[ks], b2, b3);
      }
      // mask, online softmax (rows lane/4 and lane/4 + 8; columns (lane%4)*2 + {0,1} of each n-tile)
      float p[2][4];
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j_base + nt * 8 + (lane & 3) * 2 + (e & 1);
          const float v = j < k_end ? s_acc[nt][e] * sc : -INFINITY;
          s_acc[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);                // finite: the warp has >= 1 valid key
        corr[r] = exp2f(m_run[r] - m_new);                         // exp2(-inf) = 0 on the first tile
        m_run[r] = m_new;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[nt][e] = exp2f(s_acc[nt][e] - m_run[e >> 1]);
          rs[e >> 1] += p[nt][e];
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
      // P as the A operand of the second product (16 rows x 16 keys)
      unsigned pf[4];
      pf[0] = pack_bf16(p[0][0], p[0][1]);
      pf[1] = pack_bf16(p[0][2], p[0][3]);
      pf[2] = pack_bf16(p[1][0], p[1][1]);
      pf[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
      for (int i = 0; i < NT; i += 2) {
        // matrices: (keys 0-7, d tile i), (keys 8-15, d tile i), (keys 0-7, d tile i+1), (keys 8-15, d tile i+1)
        const int mat = lane >> 3, r = lane & 7;
        const int key = key0 + (mat & 1) * 8 + r;
        const int c = i + (mat >> 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + swz<D>(key, c));
        mma_bf16(o[i], pf, b0, b1);
        mma_bf16(o[i + 1], pf, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps' states through shared memory (the stage buffers are free now)
  float* m_s = reinterpret_cast<float*>(smem);                     // [WARPS][16]
  float* l_s = m_s + DEC_WARPS * 16;                               // [WARPS][16]
  float* o_s = l_s + DEC_WARPS * 16;                               // [WARPS][16][D]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    if ((lane & 3) == 0) {
      m_s[warp * 16 + r0] = m_run[0];
      m_s[warp * 16 + r1] = m_run[1];
      l_s[warp * 16 + r0] = l_run[0];
      l_s[warp * 16 + r1] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      float* a = o_s + ((size_t)warp * 16 + r0) * D + d;
      float* c = o_s + ((size_t)warp * 16 + r1) * D + d;
      a[0] = o[i][0];
      a[1] = o[i][1];
      c[0] = o[i][2];
      c[1] = o[i][3];
    }
  }
  __syncthreads();
  // each warp's weight 2^(m_w - M) and the block's (M, L), once per head; then 16 bytes a thread
  float* f_s = o_s + DEC_WARPS * 16 * D;                           // [WARPS][16]
  float* M_s = f_s + DEC_WARPS * 16;                               // [16]
  float* L_s = M_s + 16;                                           // [16]
  float* c_acc = L_s + 16;                                         // [G][D], read by the cluster's blocks
  if ((int)threadIdx.x < DEC_WARPS * G) {
    const int v = threadIdx.x / G, g = threadIdx.x % G;
    float M = -INFINITY;
#pragma unroll
    for (int u = 0; u < DEC_WARPS; ++u) M = fmaxf(M, m_s[u * 16 + g]);
    const float mv = m_s[v * 16 + g];
    f_s[v * 16 + g] = (mv == -INFINITY) ? 0.f : exp2f(mv - M);     // a warp without a key weighs nothing
    if (v == 0) {
      float L = 0.f;
#pragma unroll
      for (int u = 0; u < DEC_WARPS; ++u) {
        const float mu = m_s[u * 16 + g];
        if (mu != -INFINITY) L += l_s[u * 16 + g] * exp2f(mu - M);
      }
      M_s[g] = M;
      L_s[g] = L;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * (D / 4); idx += DEC_WARPS * 32) {
    const int g = idx / (D / 4), d = (idx % (D / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int v = 0; v < DEC_WARPS; ++v) {
      const float f = f_s[v * 16 + g];
      const float4 x = *reinterpret_cast<const float4*>(o_s + ((size_t)v * 16 + g) * D + d);
      acc.x += x.x * f; acc.y += x.y * f; acc.z += x.z * f; acc.w += x.w * f;
    }
    const int h = kvh * G + g;
    if (nsplit == 1) {
      const float L = L_s[g], inv = L > 0.f ? 1.f / L : 0.f;
      bf16* op = out + (size_t)row_q * H * D + (size_t)h * D + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    } else if (CLUSTER) {
      *reinterpret_cast<float4*>(c_acc + g * D + d) = acc;
    } else {
      const size_t pi = ((size_t)b * H + h) * nsplit + split;
      *reinterpret_cast<float4*>(part_acc + pi * D + d) = acc;
      if (d == 0) *reinterpret_cast<float2*>(part_ml + pi * 2) = make_float2(M_s[g], L_s[g]);
    }
  }
  if (nsplit == 1) return;

  if constexpr (CLUSTER) {
    // Block r of the cluster finishes the 16-byte pieces r, r + nsplit, ... of the output; the
    // nsplit lanes of a group each fetch one split's state of that piece and sum by butterfly:
    //   out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
    cluster_sync_all();
    constexpr int QD = D / 4;
    const int pieces = G * QD, rank = split;
    const int mine = pieces > rank ? (pieces - rank + nsplit - 1) / nsplit : 0;
    const int total = mine * nsplit;
    const int shift = 31 - __clz(nsplit);
    for (int p0 = 0; p0 < total; p0 += DEC_WARPS * 32) {           // block-uniform trip count
      const int p = p0 + threadIdx.x;
      const bool valid = p < total;
      const int s2 = p & (nsplit - 1);
      const int piece = valid ? rank + ((p >> shift) << shift) : 0;
      const int g = piece / QD, d = (piece % QD) * 4;
      float m = -INFINITY, l = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid) {
        m = ld_peer_f32(peer_shared(M_s + g, s2));
        l = ld_peer_f32(peer_shared(L_s + g, s2));
        acc = ld_peer_v4(peer_shared(c_acc + g * D + d, s2));
      }
      float M = m;
      for (int x = 1; x < nsplit; x <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, x));
      const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
      l *= f;
      acc.x *= f; acc.y *= f; acc.z *= f; acc.w *= f;
      for (int x = 1; x < nsplit; x <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, x);
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, x);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, x);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, x);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, x);
      }
      if (valid && s2 == 0) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* op = out + (size_t)row_q * H * D + (size_t)(kvh * G + g) * D + d;
        *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
      }
    }
    cluster_sync_all();                                            // no block leaves while a peer still reads it
    return;
  }

  // The block that finishes last for this (request, kv head) merges all splits, in split order:
  //   out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&counters[b * KVH + kvh], 1);
    is_last = (ticket == nsplit - 1);
    if (is_last) counters[b * KVH + kvh] = 0;                      // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // weights of every (head, split): w = 2^(m_s - M) / sum_s l_s 2^(m_s - M), staged in shared memory
  float* w_s = reinterpret_cast<float*>(smem);                     // [G][nsplit]
  float* m_all = w_s + G * nsplit;                                 // [G][nsplit]
  float* l_all = m_all + G * nsplit;                               // [G][nsplit]
  for (int idx = threadIdx.x; idx < G * nsplit; idx += DEC_WARPS * 32) {
    const int g = idx / nsplit, s2 = idx % nsplit;
    const size_t pi = ((size_t)b * H + kvh * G + g) * nsplit + s2;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + pi * 2));
    m_all[idx] = ml.x;
    l_all[idx] = ml.y;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * nsplit; idx += DEC_WARPS * 32) {
    const int g = idx / nsplit;
    float M = -INFINITY, L = 0.f;
    for (int s2 = 0; s2 < nsplit; ++s2) M = fmaxf(M, m_all[g * nsplit + s2]);
    if (M > -INFINITY)
      for (int s2 = 0; s2 < nsplit; ++s2) L += l_all[g * nsplit + s2] * exp2f(m_all[g * nsplit + s2] - M);
    w_s[idx] = (L > 0.f) ? exp2f(m_all[idx] - M) / L : 0.f;
  }
  __syncthreads();
  // out[g, d..d+3] = sum_s w[g, s] * acc[g, s, d..d+3]: independent 16-byte loads, split order
  for (int idx = threadIdx.x; idx < G * (D / 4); idx += DEC_WARPS * 32) {
    const int g = idx / (D / 4), d = (idx % (D / 4)) * 4;
    const int h = kvh * G + g;
    const float* src = part_acc + (((size_t)b * H + h) * nsplit) * D + d;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int s2 = 0; s2 < nsplit; ++s2) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)s2 * D));
      const float w = w_s[g * nsplit + s2];
      acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
    }
    bf16* o = out + (size_t)row_q * H * D + (size_t)h * D + d;
    *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(acc.x, acc.y);
    *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(acc.z, acc.w);
  }
}

// How many clusters of `nsplit` blocks of this kernel the device holds at once (asked once per size);
// 0 when the splits cannot be one cluster (not 2, 4, 8 or 16 of them, or the device refuses).
template <int D, int DEC_WARPS>
int cluster_ok(int nsplit, size_t smem) {
  static int known[5] = {-1, -1, -1, -1, -1};                      // by log2(nsplit)
  if (nsplit < 2 || nsplit > 16 || (nsplit & (nsplit - 1))) return 0;
  int idx = 0;
  while ((1 << idx) < nsplit) ++idx;
  if (known[idx] < 0) {
    known[idx] = 0;
    auto kernel = attention_decode_kernel<D, true, DEC_WARPS>;
    bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
    if (ok && nsplit > 8)
      ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    if (ok) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(nsplit, 1, 1);
      cfg.blockDim = dim3(DEC_WARPS * 32);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = (unsigned)nsplit;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1) known[idx] = clusters;
    }
    cudaGetLastError();                                            // a refusal above is an answer, not an error
  }
  return known[idx];
}

template <int D, int DEC_WARPS>
int launch_decode(bf16* out, float* part_acc, float* part_ml, const bf16* qkv, const bf16* k_cache,
                  const bf16* v_cache, const int* block_tables, const int* q_start, const int* seq_lens, int B,
                  int table_width, int H, int KVH, int page, float scale, int window, int nsplit, int* counters,
                  cudaStream_t s) {
  constexpr int DEC_TILE = 16 * DEC_WARPS;
  const size_t stage_bytes = (size_t)2 * DEC_STAGES * DEC_TILE * D * 2;
  const size_t merge_bytes = sizeof(float) * ((size_t)3 * DEC_WARPS * 16 + 32 + (size_t)(DEC_WARPS + 1) * 16 * D);
  const size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, false, DEC_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_kernel<D, true, DEC_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  // Clusters only while all of them fit the chip at once: a launch whose clusters come in two waves
  // loses more than the merge gains (16 clusters of 16 blocks: a step a sixth slower than with the
  // ticket; they fit few places on the chip).  Clusters of 16 only while there are a handful.
  if (ts_clusters_enabled() && (nsplit <= 8 || B * KVH <= 4) && B * KVH <= cluster_ok<D, DEC_WARPS>(nsplit, smem))
    ts_launch_cluster(attention_decode_kernel<D, true, DEC_WARPS>, dim3(nsplit, 1, 1), dim3(nsplit, KVH, B), dim3(DEC_WARPS * 32), smem, s,
        out, part_acc, part_ml, qkv, k_cache, v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, page,
        scale, window, nsplit, counters);
  else
    ts_launch(attention_decode_kernel<D, false, DEC_WARPS>, dim3(nsplit, KVH, B), dim3(DEC_WARPS * 32), smem, s,
        out, part_acc, part_ml, qkv, k_cache, v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, page,
        scale, window, nsplit, counters);
  TS_LAUNCH_CHECK();
}

}  // namespace

static int g_wide_blocks = 2;
// The blocks of 8 warps: 2 = whenever they fit one per SM, 1 = only where they merge as clusters, 0 = never
// (for measurements).
TS_API void ts_set_decode_wide(int on) { g_wide_blocks = on; }
static int ts_num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 1;
  }
  return sms;
}

// How many clusters of 8 blocks of 8 warps (head size 128) the device holds at once: the most (request,
// kv head) pairs the wide blocks serve.
TS_API int ts_attention_decode_wide_clusters() { return cluster_ok<128, 8>(8, (size_t)2 * DEC_STAGES * 128 * 128 * 2); }

// Whether this kernel takes the shape (else the caller uses the generic kernel).
TS_API int ts_attention_decode_supported(int H, int KVH, int D, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && H / KVH <= 16 && (D == 64 || D == 128);
}

// Scratch needed for `nsplit` splits, in floats: acc [B, H, nsplit, D] then ml [B, H, nsplit, 2].
TS_API long long ts_attention_decode_scratch_floats(int B, int H, int D, int nsplit) {
  return nsplit > 1 ? (long long)B * H * nsplit * (D + 2) : 0;
}

// One query token per request (rows q_start[b]); `scratch` holds ts_attention_decode_scratch_floats()
// floats when nsplit > 1, and `counters` B * KVH ints that are zero on entry (the kernel leaves them
// zero).  window <= 0: none.
TS_API int ts_attention_decode(void* out, void* scratch, int* counters, const void* qkv, const void* k_cache, const void* v_cache,
                               const int* block_tables, const int* q_start, const int* seq_lens, int B,
                               int table_width, int H, int KVH, int D, int page, float scale, int window,
                               int nsplit, void* stream) {
  if (B <= 0) return 0;
  if (!ts_attention_decode_supported(H, KVH, D, TS_BF16))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_decode: H=%d KVH=%d D=%d is not taken by this kernel", H, KVH, D);
  if (nsplit < 1 || nsplit > 128 || B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode: nsplit=%d B=%d", nsplit, B);
  if (nsplit > 1 && (scratch == nullptr || counters == nullptr))
    TS_REFUSE(TS_ERR_SHAPE, "ts_attention_decode: %d splits need scratch and counters", nsplit);
  float* acc = (float*)scratch;
  float* ml = acc ? acc + (size_t)B * H * nsplit * D : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  // Few (request, kv head) pairs cut into 16 or more: half as many splits of 8 warps instead (as many as
  // fit one block per SM, at least 8), tiles of 128 keys: half the partial results to merge for the same
  // keys per warp (1.416 -> 1.394 ms a decode step at batch 8, 1.333 -> 1.272 ms at batch 4).  Merged as
  // one cluster a pair where the count is 8 and all clusters fit the chip at once (15 on this device), else
  // through scratch and the ticket.
  if (g_wide_blocks && nsplit >= 16) {
    const size_t wide_smem = (size_t)2 * DEC_STAGES * 128 * D * 2;
    int ws = (nsplit + 1) / 2;
    if (ws > ts_num_sms() / (B * KVH)) ws = ts_num_sms() / (B * KVH);
    const int clusters = D == 128 ? cluster_ok<128, 8>(8, wide_smem) : cluster_ok<64, 8>(8, wide_smem);
    const bool fits = ws >= 8 && (g_wide_blocks == 2 || (ws == 8 && ts_clusters_enabled() && B * KVH <= clusters));
    if (fits && D == 128)
      return launch_decode<128, 8>((bf16*)out, acc, ml, (const bf16*)qkv, (const bf16*)k_cache, (const bf16*)v_cache,
                                   block_tables, q_start, seq_lens, B, table_width, H, KVH, page, scale, window, ws, counters, s);
    if (fits)
      return launch_decode<64, 8>((bf16*)out, acc, ml, (const bf16*)qkv, (const bf16*)k_cache, (const bf16*)v_cache,
                                  block_tables, q_start, seq_lens, B, table_width, H, KVH, page, scale, window, ws, counters, s);
  }
  if (D == 64)
    return launch_decode<64, 4>((bf16*)out, acc, ml, (const bf16*)qkv, (const bf16*)k_cache, (const bf16*)v_cache,
                             block_tables, q_start, seq_lens, B, table_width, H, KVH, page, scale, window, nsplit, counters, s);
  return launch_decode<128, 4>((bf16*)out, acc, ml, (const bf16*)qkv, (const bf16*)k_cache, (const bf16*)v_cache,
                            block_tables, q_start, seq_lens, B, table_width, H, KVH, page, scale, window, nsplit, counters, s);
}

// ---- the entry point that allocates nothing (see no_alloc.h) -------------------------------------
// Scratch in the library image.  In host code this name is only a handle for the symbol, not a
// device address: the address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float g_static_scratch[TS_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_counters[TS_STATIC_COUNTERS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {};
int* g_counters_addr[MAX_DEVICES] = {};
std::mutex g_static_setup;          // two host threads may make a device's first call at the same time
}  // namespace

TS_API int ts_attention_decode_static(void* out, const void* qkv, const void* k_cache, const void* v_cache,
                                      const int* block_tables, const int* q_start, const int* seq_lens, int B,
                                      int table_width, int H, int KVH, int D, int page, float scale, int window,
                                      int nsplit, void* stream) {
  if (B <= 0) return 0;
  if (nsplit < 1) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_static: nsplit=%d", nsplit);
  const long long need = ts_attention_decode_scratch_floats(B, H, D, nsplit);
  if (need > TS_STATIC_SCRATCH_FLOATS || (long long)B * KVH > TS_STATIC_COUNTERS)
    TS_REFUSE(TS_ERR_LIMIT,
              "ts_attention_decode_static: B=%d H=%d D=%d nsplit=%d needs %lld scratch floats and %lld counters; "
              "the fixed array holds %d and %d",
              B, H, D, nsplit, need, (long long)B * KVH, TS_STATIC_SCRATCH_FLOATS, TS_STATIC_COUNTERS);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= MAX_DEVICES) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_static: device %d", dev);
  {
    std::lock_guard<std::mutex> lock(g_static_setup);
    if (g_scratch_addr[dev] == nullptr) {              // set-up, once per device, with that device current
    float* sp = nullptr;
    int* cp = nullptr;
    e = cudaGetSymbolAddress((void**)&sp, g_static_scratch);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_decode_static: scratch address: %s", cudaGetErrorString(e));
    e = cudaGetSymbolAddress((void**)&cp, g_static_counters);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_decode_static: counters address: %s", cudaGetErrorString(e));
    g_counters_addr[dev] = cp;
    g_scratch_addr[dev] = sp;
    }
  }
  if (nsplit > 1) {
    // the ticket counters must start at zero whatever an earlier (perhaps aborted) call left behind
    e = cudaMemsetAsync(g_counters_addr[dev], 0, sizeof(int) * (size_t)B * KVH, (cudaStream_t)stream);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_decode_static: clearing counters: %s", cudaGetErrorString(e));
  }
  return ts_attention_decode(out, g_scratch_addr[dev], g_counters_addr[dev], qkv, k_cache, v_cache, block_tables,
                             q_start, seq_lens, B, table_width, H, KVH, D, page, scale, window, nsplit, stream);
}
