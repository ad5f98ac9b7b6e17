// Paged grouped-query attention for PROMPT PORTIONS on the 5th-generation tensor cores:
// S = Q.K^T and O += P.V are tcgen05.mma products with their accumulators in tensor memory;
// key/value tiles come from the paged cache by TMA (one box per page or 64 keys, and half head; with
// pages shorter than a tile, ONE box per half head where the tile's pages happen to lie one after the
// other in the pool, which a request's pages do until the pool has been through many requests);
// P never leaves tensor memory (the second product reads its A operand from there).  Same
// semantics as attention_prefill.cu (the reference's turingserve/ops/triton_prefill_attention.py:17-79
// and turingserve/ops/reference.py:60-77,94-111, plus the optional window); bfloat16, head size 128,
// pages that are a multiple of 16 tokens.
//
// One block = 128 query ROWS (a row is one (token, head-in-group) pair of one kv head, so a
// group shares its key/value tiles).  Warps 0-3: thread r owns row r and tensor-memory lane r.
// Warp 4 (one lane) issues the products, warp 5 (one lane) the TMA loads: keys into a ring of
// three stages, values into a ring of two.  S has two buffers in tensor memory, so the score
// product of tile t+1 runs while the softmax warps work on tile t:
//   warp 4   : S(t)[128x64] = Q[128x128] . K(t)[64x128]^T      (issued two tiles ahead of P)
//   warps 0-3: read S(t) from tensor memory, mask, online softmax in 32-bit, write P(t) (bfloat16
//              pairs) over the first half of S(t)'s own columns; arrive on a barrier
//   warp 4   : O[128x128] += P(t)[128x64] . V(t)[64x128]   (P from tensor memory, V MN-major as TMA
//              left it), then S(t+2) into the buffer P(t) leaves
// The running maximum that the exponentials refer to moves only when a row's true maximum has
// grown by more than 2^8 since (P stays below 2^8, 32-bit sums keep their scale): then, and only
// then, O is rescaled in tensor memory, after the product before it has finished.  Two blocks
// share an SM.  Every barrier wait is bounded; a block that gives up records where, stops, and
// frees its tensor memory.
#include <utility>
#include <vector>

#include "common.cuh"
#include "tc_utils.cuh"

namespace {

using namespace tc;

constexpr int TQ = 128;            // query rows per block = TMEM lanes
constexpr int TK = 64;             // keys per tile
constexpr int HD = 128;            // head size
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int BOX_ROWS = 16;       // keys per TMA box at least: 64, 32 or 16, the largest that divides the page
constexpr uint32_t Q_BYTES = TQ * HD * 2;                 // 2 halves x [128 rows][128 B]
constexpr uint32_t KV_TILE_BYTES = TK * HD * 2;           // 2 halves x [64 keys][128 B]
constexpr uint32_t HALF_K = TK * 128;                     // bytes between the two 64-column halves of a K/V tile
constexpr uint32_t HALF_Q = TQ * 128;
constexpr uint32_t TMEM_COLS = 256;                       // S (and, over its first half, P as bf16 pairs): columns 0..63
constexpr uint32_t S_COL = 0, S_BUF = 64, O_COL = 128;    // and 64..127, O: 128..255
constexpr float RESCALE_STEP = 8.f;                       // log2 of how far a maximum may run ahead of its reference
constexpr float LOG2E_F = 1.4426950408889634f;

__device__ int g_attn_status = 0;   // 0 = fine; otherwise the wait that ran out

// Shared-memory descriptor for an MN-major operand ([k rows][64 elements = 128 B], 128-byte swizzle):
// 8-row groups along K are 1024 B apart (SBO), the next 64 elements along MN are `lbo` bytes away.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct AttnArgs {
  bf16* out;
  const bf16* qkv;
  const int* block_tables;
  const int* q_start;
  const int* seq_lens;
  int table_width, H, KVH, page, box;
  int run;                 // pages per tile when a tile is several pages (then the run maps are valid), else 0
  float scale;
  int window;
  int* status;
};

// D[tmem] (+)= A[tmem] . B[smem]: the A operand (here P) is read from tensor memory.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}

// A 4-D box (64 columns, a page's rows, one kv head, `run` pages that follow one another in the pool).
__device__ __forceinline__ void tma_load_run(void* dst, const CUtensorMap* map, int x, int kvh, int page0, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(0), "r"(kvh), "r"(page0) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr int ATT_THREADS = TQ + 64;      // warps 0-3: one query row per thread; warp 4: product issue; warp 5: TMA

__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            const __grid_constant__ CUtensorMap k_run_map, const __grid_constant__ CUtensorMap v_run_map,
                            const AttnArgs a) {
  pdl_launch_dependents();
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_s = smem;                               // [2][128][128 B]
  unsigned char* k_s = q_s + Q_BYTES;                      // [K_STAGES][2][64][128 B]
  unsigned char* v_s = k_s + K_STAGES * KV_TILE_BYTES;     // [V_STAGES][2][64][128 B]
  uint64_t* full_k = reinterpret_cast<uint64_t*>(v_s + V_STAGES * KV_TILE_BYTES);
  uint64_t* empty_k = full_k + K_STAGES;
  uint64_t* full_v = empty_k + K_STAGES;
  uint64_t* empty_v = full_v + V_STAGES;
  uint64_t* bar_s = empty_v + V_STAGES;                    // [2]: S in that buffer (and every product issued before it) is complete
  // [2]: all 128 rows have consumed S(t) and written P(t), t & 1 choosing the barrier: a warp that is
  // done with tile t may go on to tile t+1 (its S is there already), and its arrivals for t+1 must not
  // count towards tile t, which a slower warp has yet to finish
  uint64_t* bar_p = bar_s + 2;
  uint64_t* bar_pv = bar_p + 2;                            // an O product is complete
  uint64_t* bar_o = bar_pv + 1;                            // the last O product is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = a.H / a.KVH;
  const int qs = a.q_start[b];
  const int q_len = a.q_start[b + 1] - qs;
  const int seq_len = a.seq_lens[b];
  const int n_rows = q_len * G;
  const int n_row_tiles = (n_rows + TQ - 1) / TQ;
  if ((int)blockIdx.x >= n_row_tiles) return;
  const int row0 = (n_row_tiles - 1 - blockIdx.x) * TQ;     // longest tiles first
  const int tid = threadIdx.x, warp = tid >> 5;
  const int prefix = seq_len - q_len;

  if ((smem_u32(smem) & 1023u) != 0) {                       // the swizzled tiles need 1024-byte alignment
    if (tid == 0) atomicCAS(a.status, 0, 9);
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&full_k[s], 1);
      mbar_init(&empty_k[s], 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(&full_v[s], 1);
      mbar_init(&empty_v[s], 1);
    }
    mbar_init(&bar_s[0], 1);
    mbar_init(&bar_s[1], 1);
    mbar_init(&bar_p[0], TQ);
    mbar_init(&bar_p[1], TQ);
    mbar_init(bar_pv, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // key range of the block, its start aligned down to a TMA box
  const int last_row = min(row0 + TQ, n_rows) - 1;
  const int j_hi = prefix + last_row / G;
  int j_lo = a.window > 0 ? max(0, prefix + row0 / G - a.window + 1) : 0;
  const int box = a.box;
  j_lo &= ~(box - 1);
  const int n_tiles = (seq_len > 0 && j_hi >= j_lo) ? (j_hi - j_lo) / TK + 1 : 0;

  // a softmax thread's row
  const int row = row0 + tid;
  const bool row_ok = tid < TQ && row < n_rows;
  const int tok = row_ok ? row / G : 0, g = row_ok ? row % G : 0;
  const int pos = row_ok ? prefix + tok : -1;

  pdl_wait();                                               // q/k/v of this step are written by earlier kernels

  // Q rows -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c of row r at c ^ (r & 7))
  if (tid < TQ) {
    const bf16* src = a.qkv + (size_t)(qs + tok) * (a.H + 2 * a.KVH) * HD + (size_t)(kvh * G + g) * HD;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row_ok) v = *reinterpret_cast<const uint4*>(src + c * 8);
      const int half = c >> 3, cc = c & 7;
      *reinterpret_cast<uint4*>(q_s + half * HALF_Q + tid * 128 + ((cc ^ (tid & 7)) << 4)) = v;
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 5) {
    // ================= producer: TMA loads, one lane =================
    if ((tid & 31) == 0 && n_tiles > 0) {
      // The page ids of a tile whose pages are shorter than the tile (2 or 4 of them), kept in registers
      // and read two tiles ahead: a table entry fetched where it is used would put a trip to memory
      // into every tile of the one thread that issues the copies.
      struct TilePages { int p[4]; };
      const int run = a.run;
      const int* tab_row = a.block_tables + (size_t)b * a.table_width;
      auto pages_of = [&](int t) {
        TilePages tp;
        const int lp0 = (j_lo + t * TK) / a.page;
#pragma unroll
        for (int i = 0; i < 4; ++i) tp.p[i] = (i < run && t < n_tiles && lp0 + i < a.table_width) ? tab_row[lp0 + i] : -1;
        return tp;
      };
      auto load = [&](const CUtensorMap* map, const CUtensorMap* run_map, unsigned char* dst, uint64_t* bar, int t,
                      const TilePages& tp) {
        mbar_expect_tx(bar, KV_TILE_BYTES);
        const int j0 = j_lo + t * TK;
        if (run > 1) {
          // A TMA copy costs the unit about the same whatever it brings: where the tile's pages follow
          // one another in the pool (page ids p, p + 1, ...), one 4-D box per half head brings them all.
          bool in_a_row = tp.p[0] >= 0;
#pragma unroll
          for (int i = 1; i < 4; ++i) in_a_row = in_a_row && (i >= run || tp.p[i] == tp.p[0] + i);
          if (in_a_row) {
#pragma unroll
            for (int half = 0; half < 2; ++half) tma_load_run(dst + half * HALF_K, run_map, half * 64, kvh, tp.p[0], bar);
            return;
          }
          // a box is a page here: one 2-D box per page and half head
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (i >= run) break;
            const int y = (max(tp.p[i], 0) * a.KVH + kvh) * a.page;
#pragma unroll
            for (int half = 0; half < 2; ++half) tma_load_2d(dst + half * HALF_K + i * a.page * 128, map, half * 64, y, bar);
          }
          return;
        }
        // one TMA box per (`box` keys, 64 columns)
        for (int bx = 0; bx < TK / box; ++bx) {
          const int j = j0 + bx * box;
          const int lp = j / a.page;
          const int pg = lp < a.table_width ? tab_row[lp] : 0;
          const int y = (pg * a.KVH + kvh) * a.page + (j - lp * a.page);
#pragma unroll
          for (int half = 0; half < 2; ++half) tma_load_2d(dst + half * HALF_K + bx * box * 128, map, half * 64, y, bar);
        }
      };
      // keys are needed two softmax rounds before the values of the same tile: K(t+1) goes before V(t)
      bool ok = true;
      TilePages cur = pages_of(0), nxt = pages_of(1);
      load(&k_map, &k_run_map, k_s, &full_k[0], 0, cur);
      for (int t = 0; t < n_tiles && ok; ++t) {
        const TilePages after = pages_of(t + 2);
        if (t + 1 < n_tiles) {
          const int sk = (t + 1) % K_STAGES;
          if (t + 1 >= K_STAGES) ok = mbar_wait(&empty_k[sk], (uint32_t)(((t + 1) / K_STAGES - 1) & 1), a.status, 4, abort_flag);
          if (!ok) break;
          load(&k_map, &k_run_map, k_s + sk * KV_TILE_BYTES, &full_k[sk], t + 1, nxt);
        }
        const int sv = t % V_STAGES;
        if (t >= V_STAGES) ok = mbar_wait(&empty_v[sv], (uint32_t)((t / V_STAGES - 1) & 1), a.status, 7, abort_flag);
        if (!ok) break;
        load(&v_map, &v_run_map, v_s + sv * KV_TILE_BYTES, &full_v[sv], t, cur);
        cur = nxt;
        nxt = after;
      }
    }
  } else if (warp == 4) {
    // ================= product issue, one lane =================
    if ((tid & 31) == 0 && n_tiles > 0) {
      // S(t) = Q . K(t)^T into buffer t & 1: 8 k-steps of 16 columns, 4 per 64-column half
      auto issue_s = [&](int t) {
        constexpr uint32_t idesc = instr_desc(TK);
        const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s + (t % K_STAGES) * KV_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off_q = (ks >> 2) * HALF_Q + (ks & 3) * 32;
          const uint32_t off_k = (ks >> 2) * HALF_K + (ks & 3) * 32;
          umma(tmem + S_COL + (t & 1) * S_BUF, smem_desc(qa + off_q), smem_desc(ka + off_k), idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(&bar_s[t & 1]);
        umma_commit(&empty_k[t % K_STAGES]);
      };
      // O += P(t) . V(t): 4 k-steps of 16 keys; V is MN-major (rows = keys, 128 B of head columns per row)
      auto issue_o = [&](int t) {
        constexpr uint32_t idesc = instr_desc(HD, true);
        const uint32_t va = smem_u32(v_s + (t % V_STAGES) * KV_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk)                  // 16 keys = 8 columns of bfloat16 pairs
          umma_ts(tmem + O_COL, tmem + S_COL + (t & 1) * S_BUF + kk * 8, smem_desc_mn(va + kk * 16 * 128, HALF_K), idesc,
                  (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty_v[t % V_STAGES]);
        umma_commit(bar_pv);
        if (t + 1 == n_tiles) umma_commit(bar_o);
      };
      bool ok = true;
      for (int t = 0; t < 2 && t < n_tiles && ok; ++t) {
        ok = mbar_wait(&full_k[t], 0, a.status, 1, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_s(t);
        }
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        ok = mbar_wait_spin(&bar_p[t & 1], (uint32_t)((t >> 1) & 1), a.status, 6, abort_flag);     // P(t) is in place
        if (!ok) break;
        ok = mbar_wait(&full_v[t % V_STAGES], (uint32_t)((t / V_STAGES) & 1), a.status, 3, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_o(t);
        if (t + 2 < n_tiles) {
          ok = mbar_wait(&full_k[(t + 2) % K_STAGES], (uint32_t)(((t + 2) / K_STAGES) & 1), a.status, 8, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_s(t + 2);                                     // over P(t), behind the product that reads it
        }
      }
    }
  } else {
    // ================= softmax warps: thread = row = tensor-memory lane =================
    float m_ref = -INFINITY, l_run = 0.f;                   // the maximum the exponentials refer to; the sum in its scale
    const float sc = a.scale * LOG2E_F;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const uint32_t s_addr = tmem + lane_addr + S_COL + (t & 1) * S_BUF;
      ok = mbar_wait_spin(&bar_s[t & 1], (uint32_t)((t >> 1) & 1), a.status, 2, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j0 = j_lo + t * TK;
      uint32_t sv[2][32];
      tmem_ld32(s_addr, sv[0]);
      tmem_ld32(s_addr + 32, sv[1]);
      tmem_wait_ld();
      float mx = -INFINITY;
      // tiles wholly before every row of the warp (the common case away from the diagonal) need no mask
      const bool all_visible = __all_sync(0xffffffffu, (j0 + TK - 1 <= pos) && (a.window <= 0 || j0 > pos - a.window));
      if (all_visible) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = __uint_as_float(sv[h][i]) * sc;
            sv[h][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int j = j0 + h * 32 + i;
            const bool vis = (j <= pos) && (a.window <= 0 || j > pos - a.window);
            const float v = vis ? __uint_as_float(sv[h][i]) * sc : -INFINITY;
            sv[h][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
      }
      // the reference maximum follows the true one only in steps (and from nothing to something)
      const bool move = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
      float corr = 1.f;
      if (move) {
        corr = exp2f(m_ref - mx);                             // 0 when there was no reference yet: O and l are 0 then
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rs = 0.f;
      // P (bfloat16 pairs), lane = row, 32 words for the 64 keys
      uint32_t pw[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int i0 = 2 * i;
        const float p0 = exp2f(__uint_as_float(sv[i0 >> 5][i0 & 31]) - m_use);
        const float p1 = exp2f(__uint_as_float(sv[(i0 + 1) >> 5][(i0 + 1) & 31]) - m_use);
        rs += p0 + p1;
        __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        pw[i] = *reinterpret_cast<uint32_t*>(&pk);
      }
      l_run = l_run * corr + rs;
      // rescale O where a reference moved (skipped when no row of the warp needs it): the product of
      // the tile before must be done with O first
      if (t > 0 && __any_sync(0xffffffffu, move)) {
        ok = mbar_wait_spin(bar_pv, (uint32_t)((t - 1) & 1), a.status, 10, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t ov[32];
          tmem_ld32(tmem + lane_addr + O_COL + c, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
          tmem_st32(tmem + lane_addr + O_COL + c, ov);
        }
      }
      tmem_st32(s_addr, pw);                                  // over the first half of S(t), which is in registers
      tmem_wait_st();                                         // P (and a rescaled O) are in tensor memory
      tc_fence_before();
      mbar_arrive(&bar_p[t & 1]);
    }
    // epilogue: O / l -> bfloat16 -> global, one 256-byte row per thread
    if (ok && n_tiles > 0) {
      ok = mbar_wait(bar_o, 0, a.status, 5, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      bf16* dst = a.out + (size_t)(qs + tok) * a.H * HD + (size_t)(kvh * G + g) * HD;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t ov[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem + lane_addr + O_COL + c, ov);       // the whole warp loads; rows without a query store nothing
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * e]) * inv, __uint_as_float(ov[i + 2 * e + 1]) * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// The cache [pages, KVH, page, 128] as a 4-D tensor: boxes of 64 columns x a page's rows x one kv head x
// `run` pages (128-byte swizzle, zeros outside).  Encoded once per (cache, shape).
bool run_map(CUtensorMap* out, const void* cache, int num_pages, int KVH, int page, int run) {
  struct Key {
    const void* p;
    int n, k, g, r;
    bool operator==(const Key& o) const { return p == o.p && n == o.n && k == o.k && g == o.g && r == o.r; }
  };
  static std::vector<std::pair<Key, CUtensorMap>> cache_;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{cache, num_pages, KVH, page, run};
  for (auto& e : cache_)
    if (e.first == key) {
      *out = e.second;
      return true;
    }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)page, (cuuint64_t)KVH, (cuuint64_t)num_pages};
  cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)page * HD * 2, (cuuint64_t)KVH * page * HD * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)page, 1, (cuuint32_t)run};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache_.size() > 1024) cache_.clear();
  cache_.emplace_back(key, *out);
  return true;
}

int* attn_status_word() {
  static int* p = nullptr;
  if (p == nullptr && cudaGetSymbolAddress((void**)&p, g_attn_status) != cudaSuccess) p = nullptr;
  return p;
}

}  // namespace

int* ts_attn_status_word() { return attn_status_word(); }

TS_API int ts_attention_prefill_tc_supported(int H, int KVH, int D, int page, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && D == HD && page >= BOX_ROWS && page % BOX_ROWS == 0;
}

// 0 when no block ever gave up on a wait (synchronises the device).
TS_API int ts_attention_prefill_tc_status() {
  int* p = attn_status_word();
  int v = -1;
  if (p != nullptr) cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

// num_pages: pages in the pool (rows of the cache = num_pages * KVH * page).
TS_API int ts_attention_prefill_tc(void* out, const void* qkv, const void* k_cache, const void* v_cache,
                                   const int* block_tables, const int* q_start, const int* seq_lens, int B,
                                   int table_width, int max_q_len, int H, int KVH, int D, int page, int num_pages,
                                   float scale, int window, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (!ts_attention_prefill_tc_supported(H, KVH, D, page, TS_BF16))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_prefill_tc: H=%d KVH=%d D=%d page=%d is not taken by this kernel", H, KVH, D, page);
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_prefill_tc: %d requests / %d kv heads", B, KVH);
  if ((((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
    TS_REFUSE(TS_ERR_ALIGN, "ts_attention_prefill_tc: buffers must be 16-byte aligned");
  int* status = attn_status_word();
  if (status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_prefill_tc: no status word");
  CUtensorMap k_map, v_map;
  const long long rows = (long long)num_pages * KVH * page;
  if (rows > 0x7fffffffLL) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_prefill_tc: cache of %lld rows", rows);
  const int box = page % 64 == 0 ? 64 : (page % 32 == 0 ? 32 : 16);
  if (!tc::tensor_map(&k_map, k_cache, (int)rows, D, box) || !tc::tensor_map(&v_map, v_cache, (int)rows, D, box))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_prefill_tc: cuTensorMapEncodeTiled failed");
  // pages shorter than a tile: the maps whose one box is a run of pages (a box may be 256 rows at most)
  const int run = (page < TK && box == page) ? TK / page : 0;
  CUtensorMap k_run = k_map, v_run = v_map;
  if (run > 1 && (!run_map(&k_run, k_cache, num_pages, KVH, page, run) || !run_map(&v_run, v_cache, num_pages, KVH, page, run)))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_prefill_tc: cuTensorMapEncodeTiled (runs of pages) failed");
  // Two blocks fit an SM, which is what a launch of several waves wants (8,192 tokens: 261 us against
  // 379 us with one).  A launch of about one wave is as slow as its longest block, and that block
  // runs its chain of tiles faster with an SM to itself (2,048 tokens: 41 us against 48 us): such a
  // launch asks for shared memory it does not use, so that only one block fits.
  constexpr size_t smem_two = Q_BYTES + (K_STAGES + V_STAGES) * KV_TILE_BYTES + (2 * K_STAGES + 2 * V_STAGES + 6) * 8 + 16;
  constexpr size_t smem_one = smem_two + 8192;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_one);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_prefill_tc: shared memory %zu: %s", smem_one, cudaGetErrorString(e));
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sms = 0;
    configured = true;
  }
  AttnArgs a;
  a.out = (bf16*)out;
  a.qkv = (const bf16*)qkv;
  a.block_tables = block_tables;
  a.q_start = q_start;
  a.seq_lens = seq_lens;
  a.table_width = table_width;
  a.H = H;
  a.KVH = KVH;
  a.page = page;
  a.box = box;
  a.run = run > 1 ? run : 0;
  a.scale = scale;
  a.window = window;
  a.status = status;
  const int G = H / KVH;
  dim3 grid(ceil_div(max_q_len * G, TQ), KVH, B);
  const long long blocks = (long long)grid.x * grid.y * grid.z;
  const size_t smem = blocks * 2 <= (long long)sms * 3 ? smem_one : smem_two;
  ts_launch(attention_prefill_tc_kernel, grid, dim3(ATT_THREADS), smem, (cudaStream_t)stream, k_map, v_map, k_run, v_run, a);
  TS_LAUNCH_CHECK();
}
