// What the two TMA decode-attention kernels share: the layout of a stage of key/value boxes in
// shared memory, the 4-D TMA copy that fills it, and what one warp does with one tile of 64 keys
// (S = Q K^T by mma.sync m16n8k16 with the G heads of the group in the 16 rows, one online-softmax
// update, O += P V).
#pragma once

#include "common.cuh"
#include "mma_utils.cuh"
#include "tc_utils.cuh"

namespace dec {

using namespace tc;

constexpr int TILE = 64;             // keys per tile
constexpr int MIN_BOX = 16;          // keys per TMA box: 64, 32 or 16, the largest that divides the page
constexpr int NT_S = TILE / 8;       // n-tiles of the score product
constexpr float LOG2E_D = 1.4426950408889634f;

// A stage holds 64/box boxes; one box is what ONE TMA copy brings: `box` key rows of K, whole
// (D * 2 bytes each), then the same rows of V, written with the 128-byte swizzle (16-byte chunk q
// of the 128-byte line n sits at chunk q ^ (n & 7); boxes start on multiples of 1024 bytes, so n
// counts from the box).  Byte offset of 16-byte chunk c of key row `key` of K; V is box * D * 2
// bytes further (or the other way round, see v_first).
template <int D>
__device__ __forceinline__ uint32_t tile_off(int key, int c, int box_shift) {
  constexpr int LPR = D / 64;                                    // 128-byte lines per row
  const int grp = key >> box_shift, within = key & ((1 << box_shift) - 1);
  const int line = within * LPR + (c >> 3);
  return (uint32_t)(grp * (2 * D * 2) << box_shift) + (uint32_t)(line * 128 + (((c & 7) ^ (line & 7)) << 4));
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Query fragments of a group: rows 0..G-1, zero above.
template <int D>
__device__ __forceinline__ void load_q_fragments(unsigned (&qf)[D / 16][4], const bf16* qbase, int G, int lane) {
  const int r0 = lane >> 2, r1 = r0 + 8, kc = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int k = ks * 16 + kc;
    qf[ks][0] = r0 < G ? *reinterpret_cast<const unsigned*>(qbase + r0 * D + k) : 0u;
    qf[ks][1] = r1 < G ? *reinterpret_cast<const unsigned*>(qbase + r1 * D + k) : 0u;
    qf[ks][2] = r0 < G ? *reinterpret_cast<const unsigned*>(qbase + r0 * D + k + 8) : 0u;
    qf[ks][3] = r1 < G ? *reinterpret_cast<const unsigned*>(qbase + r1 * D + k + 8) : 0u;
  }
}

// One warp, one tile whose first key is j0; keys outside [k_lo, k_end) are masked.  Returns whether
// the tile was an edge tile (the caller then fences before the stage is refilled: rows of V were
// zeroed with ordinary stores).  two: rows 8..15 hold heads too (G > 8).
template <int D>
__device__ __forceinline__ bool consume_tile(const unsigned char* ks_, unsigned char* vs_, const unsigned (&qf)[D / 16][4],
                                             float (&o)[D / 8][4], float (&m_run)[2], float (&l_run)[2], int j0,
                                             int k_lo, int k_end, float sc, bool two, int bs, int lane) {
  constexpr int KS = D / 16, NT = D / 8;
  const int mat = lane >> 3, r8 = lane & 7;
  const bool edge = j0 < k_lo || j0 + TILE > k_end;           // warp-uniform
  if (edge) {
    // Rows outside the visible range were perhaps never fetched: their probabilities are exactly
    // zero, and zero times whatever shared memory held must stay zero.
    constexpr int CPR = D / 8;                                 // 16-byte chunks per row
    for (int idx = lane; idx < TILE * CPR; idx += 32) {
      const int key = idx / CPR, j = j0 + key;
      if (j >= k_lo && j < k_end) continue;
      *reinterpret_cast<uint4*>(vs_ + tile_off<D>(key, idx % CPR, bs)) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncwarp();
  }
  // scores S[16 x 64] = Q . K^T
  float s_acc[NT_S][4];
#pragma unroll
  for (int nt = 0; nt < NT_S; ++nt) s_acc[nt][0] = s_acc[nt][1] = s_acc[nt][2] = s_acc[nt][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int kg = 0; kg < TILE / 16; ++kg) {
      // matrices: (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
      const int key = kg * 16 + (mat >> 1) * 8 + r8;
      unsigned b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, ks_ + tile_off<D>(key, ks * 2 + (mat & 1), bs));
      mma_bf16(s_acc[kg * 2], qf[ks], b0, b1);
      mma_bf16(s_acc[kg * 2 + 1], qf[ks], b2, b3);
    }
  }
  // mask, online softmax (rows lane/4 and lane/4 + 8; columns (lane%4)*2 + {0,1} of each n-tile)
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float v = s_acc[nt][e] * sc;
      if (edge) {
        const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        v = (j >= k_lo && j < k_end) ? v : -INFINITY;
      }
      s_acc[nt][e] = v;
      mx[e >> 1] = fmaxf(mx[e >> 1], v);
    }
  float corr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m_run[r], mx[r]);                // finite: every tile has a visible key
    corr[r] = exp2f(m_run[r] - m_new);                         // exp2(-inf) = 0 on the first tile
    m_run[r] = m_new;
  }
  float rs[2] = {0.f, 0.f};
#pragma unroll
  for (int nt = 0; nt < NT_S; ++nt) {
    s_acc[nt][0] = exp2f(s_acc[nt][0] - m_run[0]);
    s_acc[nt][1] = exp2f(s_acc[nt][1] - m_run[0]);
    rs[0] += s_acc[nt][0] + s_acc[nt][1];
    if (two) {
      s_acc[nt][2] = exp2f(s_acc[nt][2] - m_run[1]);
      s_acc[nt][3] = exp2f(s_acc[nt][3] - m_run[1]);
      rs[1] += s_acc[nt][2] + s_acc[nt][3];
    } else {
      s_acc[nt][2] = s_acc[nt][3] = 0.f;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
    rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
    l_run[r] = l_run[r] * corr[r] + rs[r];
  }
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    o[t][0] *= corr[0];
    o[t][1] *= corr[0];
    if (two) {
      o[t][2] *= corr[1];
      o[t][3] *= corr[1];
    }
  }
  // O += P . V, P rounded to bfloat16 as the A operand (16 rows x 16 keys per step)
#pragma unroll
  for (int kg = 0; kg < TILE / 16; ++kg) {
    unsigned pf[4];
    pf[0] = pack_bf16(s_acc[kg * 2][0], s_acc[kg * 2][1]);
    pf[1] = pack_bf16(s_acc[kg * 2][2], s_acc[kg * 2][3]);
    pf[2] = pack_bf16(s_acc[kg * 2 + 1][0], s_acc[kg * 2 + 1][1]);
    pf[3] = pack_bf16(s_acc[kg * 2 + 1][2], s_acc[kg * 2 + 1][3]);
#pragma unroll
    for (int t = 0; t < NT; t += 2) {
      // matrices: (keys 0-7, d tile t), (keys 8-15, d tile t), (keys 0-7, d tile t+1), (keys 8-15, d tile t+1)
      const int key = kg * 16 + (mat & 1) * 8 + r8;
      unsigned b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + tile_off<D>(key, t + (mat >> 1), bs));
      mma_bf16(o[t], pf, b0, b1);
      mma_bf16(o[t + 1], pf, b2, b3);
    }
  }
  return edge;
}

}  // namespace dec
