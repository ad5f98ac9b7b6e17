// bfloat16 matrix product for many rows (prompt portions) on PAIRS of SMs:
//   out[M, N] = x[M, K] . w[N, K]^T (+ bias[N])          (turingserve/ops/reference.py:45-47)
// optionally with the gated activation silu(g) * u (turingserve/ops/reference.py:26-28) in its epilogue.
// The reference leaves these products to cuBLAS (turingserve/ops/triton_ops.py:74-76) and runs the
// activation as a kernel of its own (turingserve/ops/triton_silu_mul.py:10-18).
//
// Two blocks on neighbouring SMs form a cluster and compute one 256 x 256 (or 192, or 128) output tile with
// tcgen05.mma.cta_group::2: block r of the pair holds token rows 128 r .. 128 r + 127 of the tile (the A
// operand, and later these rows of the accumulator in its tensor memory) and weight rows 128 r .. of the
// tile (its half of the B operand, which the tensor cores of BOTH blocks read), so every byte that TMA
// brings into shared memory feeds twice the arithmetic of a lone block's 128 x 128 tile.  Blocks are
// persistent (one pair per two SMs, tiles dealt round robin, the tiles that run together share their
// weight tiles in L2) and hold two accumulators of 256 columns: the epilogue of one tile runs under the
// main loop of the next.
//
// Per block: warp 0 issues the TMA loads (one lane), warp 1 owns tensor memory and, in block 0 of the
// pair only, issues the products (one lane); warps 2-9 read the accumulator back and write the result.
// Barriers: full[s] (block 0's; both blocks' loads complete on it), empty[s] and acc_full[b] (each
// block's own, set by a commit that is multicast to the pair), acc_empty[b] (block 0's; one arrival per
// epilogue warp of either block).  Every wait is bounded: a barrier that does not flip in time leaves a
// code in the status word, the block stops, and still meets its peer at the last cluster barrier and frees
// its tensor memory.  No TMA multicast.
#include "common.cuh"
#include "tc_utils.cuh"

namespace {

using namespace tc;

constexpr int PM = 128;                 // token rows per block
constexpr int PAIR_THREADS = 320;       // TMA warp, issue warp, eight epilogue warps
constexpr uint32_t PA_BYTES = PM * BK * 2;
constexpr int ACC_STRIDE = 256;         // tensor-memory columns from one accumulator to the other
constexpr int ACC_COLS = 512;

// A pair tile is 256 tokens x BN outputs; each block brings BN / 2 weight rows.  BN = 256 keeps the tensor
// cores at their full rate; 192 and 128 are for products whose 256-wide tiles would leave SMs idle.
template <int BN> struct PairTile {
  static constexpr int HALF_N = BN / 2;
  static constexpr uint32_t B_BYTES = HALF_N * BK * 2, STAGE_BYTES = PA_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 6 : (BN == 192 ? 7 : 8);
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16;
  // bf16 x bf16 -> f32, M = 256 over the pair, N = BN, both operands K-major
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
};

enum PairEpilogue : int { EPI_PLAIN = 0, EPI_GATED = 1, EPI_QKV = 2 };

struct PairArgs {
  bf16* out;              // PLAIN: [M, N]; GATED: [M, N / 2]
  const bf16* bias;       // [N] or null
  int M, N, K;
  int tiles_m, tiles_n;   // pair tiles along the tokens (256 each) and along the outputs (BN each)
  int* status;
  // QKV: out is q/k/v [M, (H + 2 KVH) D]; q and k heads are rotated (full-width rotate-half, tables
  // [positions][D / 2] float, rounded to bfloat16 at use) and the new keys and values also go to the cache
  // page of the token's slot (slot < 0, or k_cache null: not written).
  const int* positions;
  const float* cos_t;
  const float* sin_t;
  const int* slots;
  bf16* k_cache;
  bf16* v_cache;
  int page, H, KVH, D;
};

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  // the data lands in this block's shared memory, the bytes are counted on block 0's barrier
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the products issued so far have completed, on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Two floats rounded to bfloat16: `lo` in the low half of the word, `hi` in the high half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
}

template <int EPI, int BN>
__global__ void __launch_bounds__(PAIR_THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const PairArgs args) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using TL = PairTile<BN>;
  constexpr int PAIR_STAGES = TL::STAGES, HALF_N = TL::HALF_N, PN = BN;
  constexpr uint32_t PB_BYTES = TL::B_BYTES, PSTAGE_BYTES = TL::STAGE_BYTES;
  unsigned char* a_s = smem;
  unsigned char* b_s = smem + PAIR_STAGES * PA_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(b_s + PAIR_STAGES * PB_BYTES);
  uint64_t* empty = full + PAIR_STAGES;
  uint64_t* acc_full = empty + PAIR_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles = args.tiles_m * args.tiles_n;
  const int n_kb = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);                // eight epilogue warps in each block of the pair
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ACC_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                              // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: those of the first stages are on their
      // way before this block waits for its predecessor; the activations follow after the wait.
      const int early = pair < tiles ? min(n_kb, PAIR_STAGES) : 0;
      {
        const int row_w = (pair / args.tiles_m) * PN + (int)rank * HALF_N;
        for (int kb = 0; kb < early; ++kb) {
          if (rank == 0) mbar_expect_tx(&full[kb], 2 * PSTAGE_BYTES);
          tma_load_2d_pair(b_s + kb * PB_BYTES, &map_w, kb * BK, row_w, peer_shared(&full[kb], 0));
        }
      }
      pdl_wait();
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        const int tm = tile % args.tiles_m, tn = tile / args.tiles_m;
        const int row_x = tm * 2 * PM + (int)rank * PM, row_w = tn * PN + (int)rank * HALF_N;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (it >= PAIR_STAGES && !mbar_wait(&empty[s], ph ^ 1, args.status, 11, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t bar = peer_shared(&full[s], 0);
          if (it >= early) {
            if (rank == 0) mbar_expect_tx(&full[s], 2 * PSTAGE_BYTES);
            tma_load_2d_pair(b_s + s * PB_BYTES, &map_w, kb * BK, row_w, bar);
          }
          tma_load_2d_pair(a_s + s * PA_BYTES, &map_x, kb * BK, row_x, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++t) {
        const int b = t & 1;
        if (t >= 2) {
          ok = mbar_wait(&acc_empty[b], ((t >> 1) - 1) & 1, args.status, 12, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t d = tmem_base + (uint32_t)(b * ACC_STRIDE);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          ok = mbar_wait(&full[s], ph, args.status, 13, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t da = smem_desc(smem_u32(a_s + s * PA_BYTES));
          const uint64_t db = smem_desc(smem_u32(b_s + s * PB_BYTES));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_pair(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), TL::IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s]);             // both blocks may refill the stage once these products have read it
        }
        if (ok) umma_commit_pair(&acc_full[b]);    // the accumulator is complete, in both blocks
      }
    }
  } else {
    const int q = warp & 3;                        // a warp reads TMEM lanes 32 (warp % 4) .. + 31
    const int part = (warp - 2) >> 2;              // the two warps of a lane quarter take every other 32 columns
    const uint32_t done_bar = peer_shared(&acc_empty[0], 0);
    pdl_wait();
    int t = 0;
    bool ok = true;
    for (int tile = pair; tile < tiles && ok; tile += pairs, ++t) {
      const int tm = tile % args.tiles_m, tn = tile / args.tiles_m;
      const int b = t & 1;
      const int row = tm * 2 * PM + (int)rank * PM + q * 32 + lane;
      // QKV: what the rotation needs of this thread's token is fetched while the products run: position, slot,
      // and the 32 cosines and sines of this warp's pairs (the same in every head), rounded to bfloat16 as
      // they are used and packed two to a register.
      int slot = -1;
      uint32_t cs_sn[EPI == EPI_QKV ? 32 : 1];
      if constexpr (EPI == EPI_QKV) {
        const int half = args.D >> 1, p0 = args.D == 128 ? part * 32 : 0;
        const int pos = row < args.M ? args.positions[row] : 0;
        if (row < args.M && args.k_cache != nullptr) slot = args.slots[row];
        const float4* cs = reinterpret_cast<const float4*>(args.cos_t + (size_t)pos * half + p0);
        const float4* sn = reinterpret_cast<const float4*>(args.sin_t + (size_t)pos * half + p0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 c = cs[i], n = sn[i];
          cs_sn[4 * i + 0] = pack_bf16x2(c.x, n.x);
          cs_sn[4 * i + 1] = pack_bf16x2(c.y, n.y);
          cs_sn[4 * i + 2] = pack_bf16x2(c.z, n.z);
          cs_sn[4 * i + 3] = pack_bf16x2(c.w, n.w);
        }
      }
      ok = mbar_wait(&acc_full[b], (t >> 1) & 1, args.status, 14, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * ACC_STRIDE);
      if constexpr (EPI == EPI_GATED) {
        // columns of the pair tile: 64 gates, their 64 ups, the next 64 gates, their 64 ups
        const int half_n = args.N >> 1;
        bf16* dst = args.out + (size_t)row * half_n + tn * (PN / 2);
#pragma unroll 1
        for (int c = part; c < 4; c += 2) {         // 32 outputs each
          const int gcol = (c >> 1) * 128 + (c & 1) * 32;
          uint32_t g[32], u[32];
          tmem_ld32(taddr + gcol, g);
          tmem_ld32(taddr + gcol + 64, u);
          tmem_wait_ld();
          if (row < args.M) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = tn * (PN / 2) + c * 32 + v * 8;
              if (col < half_n) {
                uint4 pack;
                bf16* e = reinterpret_cast<bf16*>(&pack);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  // the roundings of the product and of the activation as kernels of their own leave them
                  const float gg = round_to<bf16>(__uint_as_float(g[v * 8 + i]));
                  const float uu = round_to<bf16>(__uint_as_float(u[v * 8 + i]));
                  e[i] = from_f<bf16>(round_to<bf16>(silu_for<bf16>(gg)) * uu);
                }
                *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = pack;
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_QKV) {
        // Columns p and p + D/2 of a head are a rotation pair (turingserve/ops/reference.py:31-42); the tile
        // holds 256 / D whole heads, a thread one token's row of them, 32 pairs at a time.
        const int D = args.D, half = D >> 1, heads = args.H + 2 * args.KVH;
#pragma unroll 1
        for (int j = part; j < 4; j += 2) {
          const int hl = D == 128 ? (j >> 1) : j, p0 = D == 128 ? (j & 1) * 32 : 0;
          const int head = tn * (PN / D) + hl;
          uint32_t a1[32], a2[32];
          tmem_ld32(taddr + hl * D + p0, a1);
          tmem_ld32(taddr + hl * D + p0 + half, a2);
          tmem_wait_ld();
          if (row >= args.M || head >= heads) continue;
          const bool rotate = head < args.H + args.KVH;
          const size_t col = (size_t)head * D + p0;
          bf16* dst = args.out + (size_t)row * args.N + col;
          bf16* cdst = nullptr;
          if (head >= args.H && slot >= 0) {
            const bool is_k = head < args.H + args.KVH;
            cdst = (is_k ? args.k_cache : args.v_cache) +
                   ((size_t)(slot / args.page) * args.KVH * args.page + (size_t)(slot % args.page)) * D +
                   (size_t)(head - args.H - (is_k ? 0 : args.KVH)) * args.page * D + p0;
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float x1[8], x2[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              x1[i] = __uint_as_float(a1[v * 8 + i]);
              x2[i] = __uint_as_float(a2[v * 8 + i]);
            }
            if (args.bias != nullptr) {
              const uint4 b1 = *reinterpret_cast<const uint4*>(args.bias + col + v * 8);
              const uint4 b2 = *reinterpret_cast<const uint4*>(args.bias + col + half + v * 8);
              const bf16* e1 = reinterpret_cast<const bf16*>(&b1);
              const bf16* e2 = reinterpret_cast<const bf16*>(&b2);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                x1[i] += to_f(e1[i]);
                x2[i] += to_f(e2[i]);
              }
            }
            uint4 o1, o2;
            bf16* w1 = reinterpret_cast<bf16*>(&o1);
            bf16* w2 = reinterpret_cast<bf16*>(&o2);
            if (rotate) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float y1 = round_to<bf16>(x1[i]), y2 = round_to<bf16>(x2[i]);
                const float cc = __uint_as_float(cs_sn[v * 8 + i] << 16), ss = __uint_as_float(cs_sn[v * 8 + i] & 0xffff0000u);
                w1[i] = from_f<bf16>(y1 * cc - y2 * ss);
                w2[i] = from_f<bf16>(y2 * cc + y1 * ss);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                w1[i] = from_f<bf16>(x1[i]);
                w2[i] = from_f<bf16>(x2[i]);
              }
            }
            *reinterpret_cast<uint4*>(dst + v * 8) = o1;
            *reinterpret_cast<uint4*>(dst + half + v * 8) = o2;
            if (cdst != nullptr) {
              *reinterpret_cast<uint4*>(cdst + v * 8) = o1;
              *reinterpret_cast<uint4*>(cdst + half + v * 8) = o2;
            }
          }
        }
      } else {
        bf16* dst = args.out + (size_t)row * args.N + tn * PN;
#pragma unroll 1
        for (int c = part * 32; c < PN; c += 64) {
          uint32_t a[32];
          tmem_ld32(taddr + c, a);
          tmem_wait_ld();
          if (row < args.M) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = tn * PN + c + v * 8;
              if (col < args.N) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(a[v * 8 + i]);
                if (args.bias != nullptr) {
                  const uint4 braw = *reinterpret_cast<const uint4*>(args.bias + col);
                  const bf16* be = reinterpret_cast<const bf16*>(&braw);
#pragma unroll
                  for (int i = 0; i < 8; ++i) f[i] += to_f(be[i]);
                }
                uint4 pack;
                bf16* e = reinterpret_cast<bf16*>(&pack);
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = from_f<bf16>(f[i]);
                *reinterpret_cast<uint4*>(dst + c + v * 8) = pack;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(done_bar + (uint32_t)(b * 8));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                              // neither block's shared memory or tensor memory goes while the other may use it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
  }
}

template <int EPI, int BN>
cudaError_t allow_pair_smem() {
  static bool done = false;
  if (done) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairTile<BN>::SMEM);
  if (e == cudaSuccess) done = true;
  return e;
}

// How many pairs of this kernel's blocks the device holds at once (asked once; 0: none).
template <int EPI, int BN>
int pairs_that_fit() {
  static int known = -1;
  if (known < 0) {
    known = 0;
    if (allow_pair_smem<EPI, BN>() == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2);
      cfg.blockDim = dim3(PAIR_THREADS);
      cfg.dynamicSmemBytes = PairTile<BN>::SMEM;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<EPI, BN>, &cfg) == cudaSuccess && clusters >= 1) known = clusters;
    }
    cudaGetLastError();                              // a refusal above is an answer, not an error
  }
  return known;
}

template <int EPI, int BN>
int launch_pair(const void* x, const void* w, PairArgs args, cudaStream_t s) {
  CUtensorMap mx, mw;
  if (!tensor_map(&mx, x, args.M, args.K, PM) || !tensor_map(&mw, w, args.N, args.K, BN / 2))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair: tensor map for M = %d, N = %d, K = %d", args.M, args.N, args.K);
  const int fit = pairs_that_fit<EPI, BN>();
  if (fit < 1)
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair: no pair of blocks with %zu bytes of shared memory fits this device", PairTile<BN>::SMEM);
  args.tiles_n = (args.N + BN - 1) / BN;
  const int tiles = args.tiles_m * args.tiles_n;
  const int pairs = tiles < fit ? tiles : fit;
  ts_launch_cluster(gemm_pair_kernel<EPI, BN>, dim3(2, 1, 1), dim3(2 * pairs), dim3(PAIR_THREADS), PairTile<BN>::SMEM, s, mx, mw, args);
  TS_LAUNCH_CHECK();
}

// The tile width with the shortest schedule: rounds of tiles over the pairs of SMs times the time of a
// tile, which goes with its width down to 192 columns (narrower tiles cost the tensor cores as much).
int pair_tile_width(int tiles_m, int N, int pairs) {
  int best = 256;
  long best_cost = 0;
  const int widths[3] = {256, 192, 128};
  for (int i = 0; i < 3; ++i) {
    const int bn = widths[i];
    const long tiles = (long)tiles_m * ((N + bn - 1) / bn);
    const long cost = ((tiles + pairs - 1) / pairs) * (bn < 192 ? 192 : bn);
    if (i == 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

int g_pair_width = 0;                    // 0: by pair_tile_width; else forced (for measurements)

template <int EPI>
int launch_pair_any(const void* x, const void* w, const PairArgs& args, cudaStream_t s) {
  const int fit = pairs_that_fit<EPI, 256>();
  int bn = 256;
  if (EPI != EPI_GATED) bn = g_pair_width ? g_pair_width : pair_tile_width(args.tiles_m, args.N, fit > 0 ? fit : 1);
  if (bn == 192) return launch_pair<EPI, 192>(x, w, args, s);
  if (bn == 128) return launch_pair<EPI, 128>(x, w, args, s);
  return launch_pair<EPI, 256>(x, w, args, s);
}

}  // namespace

// epilogue 0: out[M, N] = x . w^T + bias.  1: out[M, N / 2] = silu(g) * u, the rows of w in blocks of 64
// gates followed by their 64 ups (no bias).  K a multiple of 8, N a multiple of 8 (of 128 for the gated
// form), all pointers 16-byte aligned; any M.  The status word is the few-token product's (ts_linear_tc_status):
// 11-14 = a wait of the producer, the issuer (accumulator, stage) or the epilogue ran out.
TS_API int ts_linear_pair(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int epilogue,
                          void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair: K = %d is not a positive multiple of 8", K);
  if ((N % 8) != 0 || (epilogue == EPI_GATED && (N % 128) != 0))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair: N = %d (epilogue %d)", N, epilogue);
  if (epilogue == EPI_GATED && bias != nullptr) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair: the gated epilogue takes no bias");
  if (((uintptr_t)out | (uintptr_t)x | (uintptr_t)w | (uintptr_t)bias) & 15) TS_REFUSE(TS_ERR_ALIGN, "ts_linear_pair: pointers must be 16-byte aligned");
  PairArgs a = {};
  a.out = (bf16*)out;
  a.bias = (const bf16*)bias;
  a.M = M;
  a.N = N;
  a.K = K;
  a.tiles_m = (M + 2 * PM - 1) / (2 * PM);
  a.status = ts_gemm_status_word();
  cudaStream_t s = (cudaStream_t)stream;
  switch (epilogue) {
    case EPI_PLAIN: return launch_pair_any<EPI_PLAIN>(x, w, a, s);
    case EPI_GATED: return launch_pair<EPI_GATED, 256>(x, w, a, s);
    default: TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair: epilogue %d", epilogue);
  }
}

// qkv[M, (H + 2 KVH) D] = x[M, K] . w^T + bias with q and k heads rotated and the new keys and values written
// into the cache pages, all in the product's epilogue: what ts_rope_kv_write does in a kernel of its own, for
// many rows.  Head size 64 or 128; the pointer rules of ts_linear_pair, the caches and tables 16-byte aligned.
TS_API int ts_linear_pair_qkv(void* qkv, const void* x, const void* w, const void* bias, const int* positions,
                              const float* cos_t, const float* sin_t, const int* slots, void* k_cache, void* v_cache,
                              int M, int H, int KVH, int D, int page, int K, void* stream) {
  if (M <= 0) return 0;
  const int N = (H + 2 * KVH) * D;
  if (H <= 0 || KVH <= 0 || (D != 64 && D != 128) || K <= 0 || (K % 8) != 0)
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_pair_qkv: H=%d KVH=%d D=%d K=%d is not taken by this kernel", H, KVH, D, K);
  if (positions == nullptr || cos_t == nullptr || sin_t == nullptr)
    TS_REFUSE(TS_ERR_SHAPE, "ts_linear_pair_qkv: positions and tables are needed");
  if (k_cache != nullptr && (v_cache == nullptr || slots == nullptr || page <= 0))
    TS_REFUSE(TS_ERR_SHAPE, "ts_linear_pair_qkv: the cache write needs both caches, slots and the page size");
  if (((uintptr_t)qkv | (uintptr_t)x | (uintptr_t)w | (uintptr_t)bias | (uintptr_t)cos_t | (uintptr_t)sin_t |
       (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
    TS_REFUSE(TS_ERR_ALIGN, "ts_linear_pair_qkv: pointers must be 16-byte aligned");
  PairArgs a = {};
  a.out = (bf16*)qkv;
  a.bias = (const bf16*)bias;
  a.M = M;
  a.N = N;
  a.K = K;
  a.tiles_m = (M + 2 * PM - 1) / (2 * PM);
  a.status = ts_gemm_status_word();
  a.positions = positions;
  a.cos_t = cos_t;
  a.sin_t = sin_t;
  a.slots = slots;
  a.k_cache = (bf16*)k_cache;
  a.v_cache = (bf16*)v_cache;
  a.page = page;
  a.H = H;
  a.KVH = KVH;
  a.D = D;
  return launch_pair<EPI_QKV, 256>(x, w, a, (cudaStream_t)stream);
}

// 256, 192 or 128: every product takes tiles of this width; 0: the width with the shortest schedule.
TS_API void ts_set_pair_tile_width(int bn) { g_pair_width = (bn == 256 || bn == 192 || bn == 128) ? bn : 0; }
