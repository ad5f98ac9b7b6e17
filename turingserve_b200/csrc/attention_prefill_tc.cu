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
// group shares its key/value tiles).  Warps 0-7 are the softmax: row r = tensor-memory lane r belongs
// to TWO threads, thread r of warps 0-3 with the first 32 keys of every tile and thread r of warps 4-7
// with the last 32 (the chain of a tile, 64 exponentials a row, is what bounds a block, and a pair
// walks it in half the time); the two exchange their maxima through shared memory once a tile.
// Warp 8 (one lane) issues the products, warps 9 and 10 (one lane each) the TMA loads: keys into a
// ring of three stages, values into a ring of two.  S has two buffers in tensor memory, so the score
// product of tile t+1 runs while the softmax warps work on tile t:
//   warp 8   : S(t)[128x64] = Q[128x128] . K(t)[64x128]^T      (issued two tiles ahead of P)
//   warps 0-7: read S(t) from tensor memory, mask, online softmax in 32-bit, write P(t) (bfloat16
//              pairs) over the first half of S(t)'s own columns; arrive on a barrier
//   warp 8   : O[128x128] += P(t)[128x64] . V(t)[64x128]   (P from tensor memory, V MN-major as TMA
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
constexpr int UNIT = 64;           // keys per unit of loading: a tile of keys is one or two of them
// HD, the head size, is 64 or 128: one or two halves of 64 columns (128 bytes, a swizzle line) per row.
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int BOX_ROWS = 16;       // keys per TMA box at least: 64, 32 or 16, the largest that divides the page
// A tile of TK keys (64: two blocks share an SM and hide each other's waits, what a launch of many waves
// wants; 128: one block per SM whose score products are 128 wide, what a launch of about one wave wants,
// which is as slow as its longest block: a tcgen05.mma of 16 columns of K costs the tensor pipe about 95
// cycles whether it is 64 or 128 wide, and the chain of a block is the chain of its products).
template <int TK, int HD>
struct Tile {
  static constexpr int HALVES = HD / 64;
  static constexpr uint32_t Q_BYTES = TQ * HD * 2;        // halves x [128 rows][128 B]
  static constexpr uint32_t KV_TILE_BYTES = TK * HD * 2;  // halves x [TK keys][128 B]
  static constexpr uint32_t HALF_K = TK * 128;            // bytes between the two 64-column halves of a K/V tile
  static constexpr uint32_t S_BUF = TK;                   // columns of one S buffer (and, over its first half, P as bf16 pairs)
  static constexpr uint32_t O_COL = 2 * TK;               // O behind the two S buffers
  static constexpr uint32_t TMEM_COLS = TK == 64 ? 256 : 512;
  static constexpr int KT = TK / 2;                       // keys of a tile per softmax thread
  static constexpr int UNITS = TK / UNIT;
  static constexpr size_t SMEM = Q_BYTES + (K_STAGES + V_STAGES) * KV_TILE_BYTES + (2 * K_STAGES + 2 * V_STAGES + 14) * 8 + 16 + 2 * TQ * 2;
};
constexpr uint32_t HALF_Q = TQ * 128;
constexpr uint32_t S_COL = 0;
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

// 2^x by the special-function unit alone (2 ulp; the results are rounded to bfloat16), 0 for -inf.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// warps 0-7: two threads per query row; warp 8: product issue; warp 9: TMA loads of keys; warp 10: of values
// (one thread each: with pages shorter than a tile in a shuffled pool a tile is up to 16 copies of keys and
// 16 of values at about 100 cycles of issue each, more than one thread gets through in a tile's time)
constexpr int ATT_THREADS = 2 * TQ + 96;
constexpr int MMA_WARP = 2 * TQ / 32, TMA_WARP = MMA_WARP + 1, TMA_V_WARP = MMA_WARP + 2;

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}

template <int TK, int HD>
__global__ void __launch_bounds__(ATT_THREADS, TK == 64 ? 2 : 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            const __grid_constant__ CUtensorMap k_run_map, const __grid_constant__ CUtensorMap v_run_map,
                            const AttnArgs a) {
  using TL = Tile<TK, HD>;
  constexpr uint32_t KV_TILE_BYTES = TL::KV_TILE_BYTES, HALF_K = TL::HALF_K, S_BUF = TL::S_BUF, O_COL = TL::O_COL,
                     TMEM_COLS = TL::TMEM_COLS, Q_BYTES = TL::Q_BYTES;
  constexpr int KT = TL::KT, HALVES = TL::HALVES;
  constexpr int HC = HD / 2;                                // head columns of a row per softmax thread
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
  // the two threads of a row, per pair of warps (w, w + 4): [4] both have left their maximum of the tile
  // in max_x, and [4] both have read the other's (so the next tile's may be written)
  uint64_t* bar_x = bar_o + 1;
  uint64_t* bar_r = bar_x + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_r + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  bf16* max_x = reinterpret_cast<bf16*>(const_cast<int*>(abort_flag) + 2);   // [2 halves][128 rows]

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
    mbar_init(&bar_p[0], 2 * TQ);
    mbar_init(&bar_p[1], 2 * TQ);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bar_x[i], 64);
      mbar_init(&bar_r[i], 64);
    }
    mbar_init(bar_pv, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
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

  // a softmax thread's row and which half of a tile's keys (and of the head's columns) it takes
  const int lane_row = tid & (TQ - 1), hh = (tid >> 7) & 1;
  const int row = row0 + lane_row;
  const bool row_ok = tid < 2 * TQ && row < n_rows;
  const int tok = row_ok ? row / G : 0, g = row_ok ? row % G : 0;
  const int pos = row_ok ? prefix + tok : -1;

  pdl_wait();                                               // q/k/v of this step are written by earlier kernels

  // Q rows -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c of row r at c ^ (r & 7))
  if (tid < 2 * TQ) {                                         // each of a row's two threads half the head's columns
    const bf16* src = a.qkv + (size_t)(qs + tok) * (a.H + 2 * a.KVH) * HD + (size_t)(kvh * G + g) * HD + hh * HC;
    uint4 v[HC / 8];
#pragma unroll
    for (int cc = 0; cc < HC / 8; ++cc) v[cc] = row_ok ? *reinterpret_cast<const uint4*>(src + cc * 8) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int cc = 0; cc < HC / 8; ++cc) {
      const int c = hh * (HC / 8) + cc;                       // 16-byte piece of the row: half c / 8, piece c % 8 of it
      *reinterpret_cast<uint4*>(q_s + (c >> 3) * HALF_Q + lane_row * 128 + (((c & 7) ^ (lane_row & 7)) << 4)) = v[cc];
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == TMA_WARP || warp == TMA_V_WARP) {
    // ================= producers: TMA loads of keys (one warp) and of values (another), one lane each =================
    if ((tid & 31) == 0 && n_tiles > 0) {
      // The page ids of a tile whose pages are shorter than the tile (2 or 4 of them), kept in registers
      // and read two tiles ahead: a table entry fetched where it is used would put a trip to memory
      // into every tile of the one thread that issues the copies.
      struct TilePages { int p[4 * TL::UNITS]; };
      const int run = a.run;
      const int* tab_row = a.block_tables + (size_t)b * a.table_width;
      auto pages_of = [&](int t) {
        TilePages tp;
#pragma unroll
        for (int u = 0; u < TL::UNITS; ++u) {
          const int lp0 = (j_lo + t * TK + u * UNIT) / a.page;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            tp.p[4 * u + i] = (i < run && t < n_tiles && lp0 + i < a.table_width) ? tab_row[lp0 + i] : -1;
        }
        return tp;
      };
      auto load = [&](const CUtensorMap* map, const CUtensorMap* run_map, unsigned char* tile, uint64_t* bar, int t,
                      const TilePages& tp) {
        mbar_expect_tx(bar, KV_TILE_BYTES);
#pragma unroll
        for (int u = 0; u < TL::UNITS; ++u) {
          unsigned char* dst = tile + u * UNIT * 128;          // the unit's rows within each 64-column half
          const int j0 = j_lo + t * TK + u * UNIT;
          if (run > 1) {
            // A TMA copy costs the unit about the same whatever it brings: where the unit's pages follow
            // one another in the pool (page ids p, p + 1, ...), one 4-D box per half head brings them all.
            const int* pg = tp.p + 4 * u;
            bool in_a_row = pg[0] >= 0;
#pragma unroll
            for (int i = 1; i < 4; ++i) in_a_row = in_a_row && (i >= run || pg[i] == pg[0] + i);
            if (in_a_row) {
#pragma unroll
              for (int half = 0; half < HALVES; ++half) tma_load_run(dst + half * HALF_K, run_map, half * 64, kvh, pg[0], bar);
              continue;
            }
            // a box is a page here: one 2-D box per page and half head
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (i >= run) break;
              const int y = (max(pg[i], 0) * a.KVH + kvh) * a.page;
#pragma unroll
              for (int half = 0; half < HALVES; ++half) tma_load_2d(dst + half * HALF_K + i * a.page * 128, map, half * 64, y, bar);
            }
            continue;
          }
          // one TMA box per (`box` keys, 64 columns)
          for (int bx = 0; bx < UNIT / box; ++bx) {
            const int j = j0 + bx * box;
            const int lp = j / a.page;
            const int pg = lp < a.table_width ? tab_row[lp] : 0;
            const int y = (pg * a.KVH + kvh) * a.page + (j - lp * a.page);
#pragma unroll
            for (int half = 0; half < HALVES; ++half) tma_load_2d(dst + half * HALF_K + bx * box * 128, map, half * 64, y, bar);
          }
        }
      };
      // each ring fills as far ahead as its stages allow
      bool ok = true;
      const bool keys = warp == TMA_WARP;
      const CUtensorMap* map = keys ? &k_map : &v_map;
      const CUtensorMap* rmap = keys ? &k_run_map : &v_run_map;
      unsigned char* ring = keys ? k_s : v_s;
      uint64_t* full = keys ? full_k : full_v;
      uint64_t* empty = keys ? empty_k : empty_v;
      const int stages = keys ? K_STAGES : V_STAGES;
      TilePages cur = pages_of(0), nxt = pages_of(1);
      for (int t = 0; t < n_tiles && ok; ++t) {
        const TilePages after = pages_of(t + 2);
        const int st = t % stages;
        if (t >= stages) ok = mbar_wait(&empty[st], (uint32_t)((t / stages - 1) & 1), a.status, keys ? 4 : 7, abort_flag);
        if (!ok) break;
        load(map, rmap, ring + st * KV_TILE_BYTES, &full[st], t, cur);
        cur = nxt;
        nxt = after;
      }
    }
  } else if (warp == MMA_WARP) {
    // ================= product issue, one lane =================
    if ((tid & 31) == 0 && n_tiles > 0) {
      // S(t) = Q . K(t)^T into buffer t & 1: HD / 16 k-steps of 16 columns, 4 per 64-column half
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
    // ================= softmax warps: two threads per row = tensor-memory lane =================
    float m_ref = -INFINITY, l_run = 0.f;                   // the maximum the exponentials refer to; this half's sum in its scale
    const float sc = a.scale * LOG2E_F;
    const int pair = warp & 3;                              // warps `pair` and `pair + 4` share 32 rows
    const uint32_t lane_addr = (uint32_t)(pair * 32) << 16;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const uint32_t s_addr = tmem + lane_addr + S_COL + (t & 1) * S_BUF;
      ok = mbar_wait_spin(&bar_s[t & 1], (uint32_t)((t >> 1) & 1), a.status, 2, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j0 = j_lo + t * TK + hh * KT;               // this thread's first key of the tile
      uint32_t sv[KT / 32][32];
#pragma unroll
      for (int h = 0; h < KT / 32; ++h) tmem_ld32(s_addr + hh * KT + h * 32, sv[h]);
      tmem_wait_ld();
      float mx = -INFINITY;
      // keys wholly before every row of the warp (the common case away from the diagonal) need no mask
      const bool all_visible = __all_sync(0xffffffffu, (j0 + KT - 1 <= pos) && (a.window <= 0 || j0 > pos - a.window));
      if (all_visible) {
#pragma unroll
        for (int h = 0; h < KT / 32; ++h)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = __uint_as_float(sv[h][i]) * sc;
            sv[h][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
      } else {
#pragma unroll
        for (int h = 0; h < KT / 32; ++h)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int j = j0 + h * 32 + i;
            const bool vis = (j <= pos) && (a.window <= 0 || j > pos - a.window);
            const float v = vis ? __uint_as_float(sv[h][i]) * sc : -INFINITY;
            sv[h][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
      }
      // The row's maximum over both halves, as both threads must see the same one: each leaves its own,
      // rounded to bfloat16, and takes the larger of the two rounded values (a maximum that is a little
      // low only lets P run a little above 1, which the 2^8 of headroom below covers).
      if (t > 0) {
        ok = mbar_wait_spin(&bar_r[pair], (uint32_t)((t - 1) & 1), a.status, 11, abort_flag);   // the last one has been read
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const bf16 mine = __float2bfloat16_rn(mx);
      max_x[hh * TQ + lane_row] = mine;
      mbar_arrive(&bar_x[pair]);
      // P (bfloat16 pairs), lane = row, KT / 2 words for this thread's KT keys, and their sum
      uint32_t pw[KT / 2];
      auto exponentials = [&](float m_use) {
        float rs = 0.f;
#pragma unroll
        for (int i = 0; i < KT / 2; ++i) {
          const int i0 = 2 * i;
          const float p0 = ex2(__uint_as_float(sv[i0 >> 5][i0 & 31]) - m_use);
          const float p1 = ex2(__uint_as_float(sv[(i0 + 1) >> 5][(i0 + 1) & 31]) - m_use);
          rs += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          pw[i] = *reinterpret_cast<uint32_t*>(&pk);
        }
        return rs;
      };
      // The reference maximum moves rarely once a row has one: the exponentials are taken against the
      // present reference while the other thread's maximum is on its way, and taken again for the rows
      // whose reference then moves after all.
      const bool ahead = __all_sync(0xffffffffu, m_ref != -INFINITY);
      float rs = 0.f;
      if (ahead) rs = exponentials(m_ref);
      ok = mbar_wait_spin(&bar_x[pair], (uint32_t)(t & 1), a.status, 12, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      mx = fmaxf(__bfloat162float(mine), __bfloat162float(max_x[(hh ^ 1) * TQ + lane_row]));
      mbar_arrive(&bar_r[pair]);
      // the reference maximum follows the true one only in steps (and from nothing to something)
      const bool move = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
      float corr = 1.f;
      if (move) {
        corr = ex2(m_ref - mx);                               // 0 when there was no reference yet: O and l are 0 then
        m_ref = mx;
      }
      if (!ahead || move) rs = exponentials((m_ref == -INFINITY) ? 0.f : m_ref);
      l_run = l_run * corr + rs;
      // rescale O where a reference moved (skipped when no row of the warp needs it), each thread its half
      // of the columns: the product of the tile before must be done with O first
      if (t > 0 && __any_sync(0xffffffffu, move)) {
        ok = mbar_wait_spin(bar_pv, (uint32_t)((t - 1) & 1), a.status, 10, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = hh * HC; c < hh * HC + HC; c += 32) {
          uint32_t ov[32];
          tmem_ld32(tmem + lane_addr + O_COL + c, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
          tmem_st32(tmem + lane_addr + O_COL + c, ov);
        }
      }
      // over the first half of S(t): the second thread's words lie over scores of the FIRST thread of the
      // row, which has them in registers since before it left its maximum
      if constexpr (KT == 32) tmem_st16(s_addr + hh * 16, pw);
      else tmem_st32(s_addr + hh * 32, pw);
      tmem_wait_st();                                         // P (and a rescaled O) are in tensor memory
      tc_fence_before();
      mbar_arrive(&bar_p[t & 1]);
    }
    // epilogue: O / l -> bfloat16 -> global, 128 bytes of the row per thread
    if (ok && n_tiles > 0) {
      ok = mbar_wait(bar_o, 0, a.status, 5, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    // the row's sum is the two halves' sums (same scale): exchanged through the shared memory Q leaves,
    // on the pair's barrier, whose next phase is n_tiles' parity
    if (ok && n_tiles > 0) {
      float* l_x = reinterpret_cast<float*>(q_s);
      l_x[hh * TQ + lane_row] = l_run;
      mbar_arrive(&bar_x[pair]);
      ok = mbar_wait_spin(&bar_x[pair], (uint32_t)(n_tiles & 1), a.status, 13, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) l_run += l_x[(hh ^ 1) * TQ + lane_row];
    }
    if (ok) {
      tc_fence_after();
      bf16* dst = a.out + (size_t)(qs + tok) * a.H * HD + (size_t)(kvh * G + g) * HD;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c = hh * HC; c < hh * HC + HC; c += 32) {
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
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// The cache [pages, KVH, page, 128] as a 4-D tensor: boxes of 64 columns x a page's rows x one kv head x
// `run` pages (128-byte swizzle, zeros outside).  Encoded once per (cache, shape).
bool run_map(CUtensorMap* out, const void* cache, int num_pages, int KVH, int page, int run, int HD) {
  struct Key {
    const void* p;
    int n, k, g, r;
    bool operator==(const Key& o) const { return p == o.p && n == o.n && k == o.k && g == o.g && r == o.r; }
  };
  static std::vector<std::pair<Key, CUtensorMap>> cache_;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{cache, num_pages, KVH, page, run + 1024 * HD};
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

static int g_tile_keys = 0;
// Keys per tile of the prompt attention: 64, 128, or 0 for the launch's own choice (for measurements).
TS_API void ts_set_prefill_tile(int keys) { g_tile_keys = (keys == 64 || keys == 128) ? keys : 0; }

TS_API int ts_attention_prefill_tc_supported(int H, int KVH, int D, int page, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && (D == 64 || D == 128) && page >= BOX_ROWS && page % BOX_ROWS == 0;
}

// 0 when no block ever gave up on a wait (synchronises the device).
TS_API int ts_attention_prefill_tc_status() {
  int* p = attn_status_word();
  int v = -1;
  if (p != nullptr) cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

namespace {
template <int TK, int HD>
cudaError_t launch_tiles(dim3 grid, cudaStream_t stream, const CUtensorMap& k_map, const CUtensorMap& v_map,
                         const CUtensorMap& k_run, const CUtensorMap& v_run, const AttnArgs& a) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<TK, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)Tile<TK, HD>::SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  return ts_launch(attention_prefill_tc_kernel<TK, HD>, grid, dim3(ATT_THREADS), Tile<TK, HD>::SMEM, stream, k_map, v_map, k_run,
                   v_run, a);
}
}  // namespace

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
  const int run = (page < UNIT && box == page) ? UNIT / page : 0;
  CUtensorMap k_run = k_map, v_run = v_map;
  if (run > 1 && (!run_map(&k_run, k_cache, num_pages, KVH, page, run, D) || !run_map(&v_run, v_cache, num_pages, KVH, page, run, D)))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_prefill_tc: cuTensorMapEncodeTiled (runs of pages) failed");
  // Two blocks with tiles of 64 keys fit an SM, which is what a launch of several waves wants (8,192
  // tokens: 261 us against 379 us with one).  A launch of about one wave is as slow as its longest block:
  // it gets tiles of 128 keys, one block per SM.
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sms = 1;
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
  const bool wide = g_tile_keys == 128 || (g_tile_keys == 0 && blocks * 2 <= (long long)sms * 3);
  cudaError_t e;
  if (D == 128)
    e = wide ? launch_tiles<128, 128>(grid, (cudaStream_t)stream, k_map, v_map, k_run, v_run, a)
             : launch_tiles<64, 128>(grid, (cudaStream_t)stream, k_map, v_map, k_run, v_run, a);
  else
    e = wide ? launch_tiles<128, 64>(grid, (cudaStream_t)stream, k_map, v_map, k_run, v_run, a)
             : launch_tiles<64, 64>(grid, (cudaStream_t)stream, k_map, v_map, k_run, v_run, a);
  if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_prefill_tc: %s", cudaGetErrorString(e));
  TS_LAUNCH_CHECK();
}
