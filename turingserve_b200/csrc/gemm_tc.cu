// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), operands brought to
// shared memory by TMA, accumulator in tensor memory:
//   out[M, N] = x[M, K] . w[N, K]^T (+ bias[N])          (turingserve/ops/reference.py:45-47)
// The reference leaves its products to cuBLAS (turingserve/ops/triton_ops.py:74-76); this kernel is
// the engine's own.  Two orientations share one kernel:
//   * "tokens on rows"  : the 128 rows of the MMA tile are tokens, its BN columns are outputs;
//   * "weights on rows" : for a handful of tokens (decode) the 128 tile rows are OUTPUTS (weight rows)
//     and the tokens sit in the narrow N dimension (8..128), so the weight matrix streams through
//     full-height tiles once and nothing is wasted on padding tokens.  K can be split over
//     blockIdx.z to put every SM to work; partial sums go to a float scratch and a second kernel
//     reduces them in a fixed order.
//
// One block = one output tile.  Warp 0 issues the TMA loads (one lane), warp 1 issues tcgen05.mma
// (one lane) and owns the tensor-memory allocation, warps 2-5 read the accumulator back with
// tcgen05.ld and write the result.  Stages are handed over through mbarriers; every wait is
// bounded: when a barrier does not flip in time the block records where in `status`, stops, and
// still frees its tensor memory.
#include "common.cuh"
#include "tc_utils.cuh"

namespace {

constexpr int BM = 128;            // tile rows = TMEM lanes
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

using namespace tc;

struct GemmArgs {
  void* out;              // bf16 or float [M, N]; or float scratch [splits, M, N] when splits > 1
  const bf16* bias;       // [N] or null (applied here only when splits == 1)
  int M, N, K;
  int k_blocks_per_split;
  int splits;
  int out_is_float;
  int gated;              // weights-on-rows only: the tile's rows are 64 gates then 64 ups; out is bf16 [M, N / 2]
  int* status;
  // weights-on-rows q/k/v product that finishes itself (rope != 0): a tile is one head of 128 or two of 64; every
  // block leaves its partial sums in rope_part, the block that comes last for a tile (ticket counter)
  // adds them up in split order, adds the bias, rotates q and k heads and writes q/k/v to `out` and the
  // new keys and values into the cache pages: what ts_rope_kv_write_ex does in a kernel of its own.
  int rope;
  float* rope_part;       // [tiles][token blocks][splits][BN][128]
  int* rope_counters;     // [tiles][token blocks], zero on entry and on exit
  const int* positions;
  const float* cos_t;     // [positions][64]
  const float* sin_t;
  const int* slots;       // cache slot of every token, < 0: not written
  bf16* k_cache;
  bf16* v_cache;
  int page, H, KVH;
  int D = 128;            // head size of the product that finishes itself: 64 or 128
  // weights-on-rows, a few tokens, resid != null: the splits of a tile are one thread-block cluster (or a
  // single block); the sum over them in split order, plus bias, is rounded to bfloat16 and added to
  // `resid` [M, N] in place, rounded again: what the product's epilogue and the next norm's residual add do.
  bf16* resid = nullptr;
};

constexpr size_t gemm_smem_bytes(int BN, int STAGES, int KSUB) {
  return 1024 + (size_t)STAGES * KSUB * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 1) * 8 + 24;
}

// BN: tile columns (UMMA N).  SWAP: the tile rows are weight rows (outputs), columns are tokens.
// KSUB: 64-column k-blocks per pipeline stage (their TMA boxes are issued back to back, so a weight
// row is touched KSUB * 128 contiguous bytes at a time).
// Columns p and p + 64 of token m of a head (q heads, then k, then v), given their sums with the
// bias: rounded to bfloat16 as a product's epilogue rounds, rotated (q and k), written to the q/k/v
// tensor and, for k and v, into the cache page of the token's slot.
// (the pair is columns p and p + D/2 of the head)
__device__ __forceinline__ void rope_finish(const GemmArgs& args, int head, int p, int m, float x1, float x2) {
  const int D = args.D, half = D >> 1;
  if (head >= args.H + 2 * args.KVH) return;         // the second half of a last tile that holds one head of 64
  x1 = round_to<bf16>(x1);
  x2 = round_to<bf16>(x2);
  float o1 = x1, o2 = x2;
  if (head < args.H + args.KVH) {
    const int pos = args.positions[m];
    const float cs = round_to<bf16>(args.cos_t[(size_t)pos * half + p]);
    const float sn = round_to<bf16>(args.sin_t[(size_t)pos * half + p]);
    o1 = x1 * cs - x2 * sn;
    o2 = x2 * cs + x1 * sn;
  }
  const bf16 w1 = __float2bfloat16_rn(o1), w2 = __float2bfloat16_rn(o2);
  bf16* qkv = reinterpret_cast<bf16*>(args.out);
  qkv[(size_t)m * args.N + head * D + p] = w1;
  qkv[(size_t)m * args.N + head * D + p + half] = w2;
  if (head >= args.H && args.k_cache != nullptr) {
    const int slot = args.slots[m];
    if (slot >= 0) {
      const size_t cache_base = ((size_t)(slot / args.page) * args.KVH * args.page + (size_t)(slot % args.page)) * D;
      const bool is_k = head < args.H + args.KVH;
      bf16* dst = (is_k ? args.k_cache : args.v_cache) + cache_base +
                  (size_t)(head - args.H - (is_k ? 0 : args.KVH)) * args.page * D;
      dst[p] = w1;
      dst[p + half] = w2;
    }
  }
}

// The same for four neighbouring pairs p..p+3 (p a multiple of 4) with 16- and 8-byte memory operations.
__device__ __forceinline__ void rope_finish4(const GemmArgs& args, int head, int p, int m, const float (&x1)[4],
                                             const float (&x2)[4]) {
  const int D = args.D, half = D >> 1;
  if (head >= args.H + 2 * args.KVH) return;
  float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
  const bool rotate = head < args.H + args.KVH;
  if (rotate) {
    const int pos = args.positions[m];
    const float4 c = *reinterpret_cast<const float4*>(args.cos_t + (size_t)pos * half + p);
    const float4 s4 = *reinterpret_cast<const float4*>(args.sin_t + (size_t)pos * half + p);
    cs[0] = c.x; cs[1] = c.y; cs[2] = c.z; cs[3] = c.w;
    sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
  }
  bf16 w1[4], w2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = round_to<bf16>(x1[i]), b = round_to<bf16>(x2[i]);
    float o1 = a, o2 = b;
    if (rotate) {
      const float c = round_to<bf16>(cs[i]), s1 = round_to<bf16>(sn[i]);
      o1 = a * c - b * s1;
      o2 = b * c + a * s1;
    }
    w1[i] = __float2bfloat16_rn(o1);
    w2[i] = __float2bfloat16_rn(o2);
  }
  const uint2 v1 = *reinterpret_cast<const uint2*>(w1), v2 = *reinterpret_cast<const uint2*>(w2);
  bf16* qkv = reinterpret_cast<bf16*>(args.out);
  *reinterpret_cast<uint2*>(qkv + (size_t)m * args.N + head * D + p) = v1;
  *reinterpret_cast<uint2*>(qkv + (size_t)m * args.N + head * D + p + half) = v2;
  if (head >= args.H && args.k_cache != nullptr) {
    const int slot = args.slots[m];
    if (slot >= 0) {
      const size_t cache_base = ((size_t)(slot / args.page) * args.KVH * args.page + (size_t)(slot % args.page)) * D;
      const bool is_k = head < args.H + args.KVH;
      bf16* dst = (is_k ? args.k_cache : args.v_cache) + cache_base +
                  (size_t)(head - args.H - (is_k ? 0 : args.KVH)) * args.page * D;
      *reinterpret_cast<uint2*>(dst + p) = v1;
      *reinterpret_cast<uint2*>(dst + p + half) = v2;
    }
  }
}

// Thread r (0..127) of the finishing stage owns pair r & 63 of its tile, of tokens r >> 6, r >> 6 + 2, ...:
// the tile's columns c1 and c1 + D/2, which are pair p of head `head`.
struct RopePair {
  int head, p, c1, c2;
};
__device__ __forceinline__ RopePair rope_pair(const GemmArgs& args, int tile, int r) {
  const int half = args.D >> 1, q = r & 63;
  const int in_tile = q / half, p = q - in_tile * half;      // D = 128: head 0 of the tile, p = q
  RopePair rp;
  rp.head = tile * (128 / args.D) + in_tile;
  rp.p = p;
  rp.c1 = in_tile * args.D + p;
  rp.c2 = rp.c1 + half;
  return rp;
}

template <int BN, int STAGES, bool SWAP, int KSUB>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
               const GemmArgs args) {
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* a_s = smem;
  constexpr uint32_t STAGE_A = KSUB * A_BYTES, STAGE_B = KSUB * B_BYTES;
  unsigned char* b_s = smem + STAGES * STAGE_A;
  uint64_t* full = reinterpret_cast<uint64_t*>(b_s + STAGES * STAGE_B);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;
  const bool fuse_resid = SWAP && args.resid != nullptr;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * BM;                 // first tile row (tokens, or weight rows when SWAP)
  const int col0 = blockIdx.y * BN;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb_begin = blockIdx.z * args.k_blocks_per_split;
  const int kb_end = min(total_kb, kb_begin + args.k_blocks_per_split);
  const int n_kb = kb_end - kb_begin;
  const int n_it = (n_kb + KSUB - 1) / KSUB;          // pipeline iterations: KSUB k-blocks each (the last may hold fewer)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: their first stages are on the
      // way before this block waits for its predecessor; the activations follow after the wait.
      const CUtensorMap* w_map = SWAP ? &map_rows : &map_cols;
      const CUtensorMap* x_map = SWAP ? &map_cols : &map_rows;
      unsigned char* w_s = SWAP ? a_s : b_s;
      unsigned char* x_s = SWAP ? b_s : a_s;
      constexpr uint32_t W_BYTES = SWAP ? A_BYTES : B_BYTES, X_BYTES = SWAP ? B_BYTES : A_BYTES;
      constexpr uint32_t W_STAGE = KSUB * W_BYTES, X_STAGE = KSUB * X_BYTES;
      const int w_row = SWAP ? row0 : col0, x_row = SWAP ? col0 : row0;
      const int early = n_it < STAGES ? n_it : STAGES;
      for (int i = 0; i < early; ++i) {
        const int subs = min(KSUB, n_kb - i * KSUB);
        mbar_expect_tx(&full[i], subs * (A_BYTES + B_BYTES));
        for (int u = 0; u < subs; ++u)
          tma_load_2d(w_s + i * W_STAGE + u * W_BYTES, w_map, (kb_begin + i * KSUB + u) * BK, w_row, &full[i]);
      }
      // ... and the rest of this block's weights start towards L2
      for (int kb = kb_begin + early * KSUB; kb < kb_end; ++kb)
        asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(w_map), "r"(kb * BK), "r"(w_row) : "memory");
      pdl_wait();
      for (int i = 0; i < early; ++i) {
        const int subs = min(KSUB, n_kb - i * KSUB);
        for (int u = 0; u < subs; ++u)
          tma_load_2d(x_s + i * X_STAGE + u * X_BYTES, x_map, (kb_begin + i * KSUB + u) * BK, x_row, &full[i]);
      }
      for (int i = early; i < n_it; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, args.status, 1, abort_flag)) break;
        const int subs = min(KSUB, n_kb - i * KSUB);
        mbar_expect_tx(&full[s], subs * (A_BYTES + B_BYTES));
        for (int u = 0; u < subs; ++u) {
          const int k = (kb_begin + i * KSUB + u) * BK;
          tma_load_2d(w_s + s * W_STAGE + u * W_BYTES, w_map, k, w_row, &full[s]);
          tma_load_2d(x_s + s * X_STAGE + u * X_BYTES, x_map, k, x_row, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      bool ok = true;
      for (int i = 0; i < n_it && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        ok = mbar_wait(&full[s], ph, args.status, 2, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int subs = min(KSUB, n_kb - i * KSUB);
        for (int u = 0; u < subs; ++u) {
          const uint64_t da = smem_desc(smem_u32(a_s + s * STAGE_A + u * A_BYTES));
          const uint64_t db = smem_desc(smem_u32(b_s + s * STAGE_B + u * B_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(tmem_base, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc,
                 (i > 0 || u > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);                    // the stage is free once these MMAs have read it
      }
      umma_commit(accum);                          // the accumulator is complete
    }
  } else {
    // epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31
    const int q = warp & 3;
    const int r = q * 32 + lane;                   // tile row of this thread
    pdl_wait();                                    // nothing is written before the predecessor is done
    bool ok = n_kb > 0 && mbar_wait(accum, 0, args.status, 3, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (SWAP && (args.rope == 2 || fuse_resid)) {
      // The splits of this tile are one cluster: the partial sums stay in shared memory (the stage
      // buffers are free by now) for the peers to read; see the end of the kernel.
      constexpr int CW = BN >= 32 ? 32 : 16;
      float* ex = reinterpret_cast<float*>(a_s);                // [BN][128]
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < BN; c += CW) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c;
          if constexpr (CW == 32) {
            tmem_ld32(taddr, v);
          } else {
            uint32_t v16[16];
            tmem_ld16(taddr, v16);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = v16[i];
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < CW; ++i) ex[(c + i) * 128 + r] = __uint_as_float(v[i]);
        }
      }
    } else if (SWAP && args.rope) {
      constexpr int CW = BN >= 32 ? 32 : 16;
      const int slot_id = blockIdx.x * gridDim.y + blockIdx.y;
      float* mine = args.rope_part + ((size_t)slot_id * args.splits + blockIdx.z) * BN * 128;
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < BN; c += CW) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c;
          if constexpr (CW == 32) {
            tmem_ld32(taddr, v);
          } else {
            uint32_t v16[16];
            tmem_ld16(taddr, v16);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = v16[i];
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < CW; ++i)
            if (col0 + c + i < args.M) mine[(size_t)(c + i) * 128 + r] = __uint_as_float(v[i]);
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (r == 0) {
        const int ticket = atomicAdd(&args.rope_counters[slot_id], 1);
        *last_flag = (ticket == args.splits - 1);
        if (ticket == args.splits - 1) args.rope_counters[slot_id] = 0;      // ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag) {
        __threadfence();
        const RopePair rp = rope_pair(args, blockIdx.x, r);    // tiles hold the q heads, then k, then v
        const int head = rp.head, p = rp.p, tg = r >> 6;
        const float* base = args.rope_part + (size_t)slot_id * args.splits * BN * 128;
        const bool real = head < args.H + 2 * args.KVH;
        const float b1 = (args.bias != nullptr && real) ? to_f(args.bias[head * args.D + p]) : 0.f;
        const float b2 = (args.bias != nullptr && real) ? to_f(args.bias[head * args.D + p + (args.D >> 1)]) : 0.f;
        const int tokens = min(BN, args.M - col0);
        for (int tok = tg; tok < tokens; tok += 2) {
          float lo[16], hi[16];
#pragma unroll
          for (int sp = 0; sp < 16; ++sp)
            if (sp < args.splits) {
              lo[sp] = __ldcg(base + ((size_t)sp * BN + tok) * 128 + rp.c1);
              hi[sp] = __ldcg(base + ((size_t)sp * BN + tok) * 128 + rp.c2);
            }
          float x1 = 0.f, x2 = 0.f;
#pragma unroll
          for (int sp = 0; sp < 16; ++sp)
            if (sp < args.splits) {
              x1 += lo[sp];
              x2 += hi[sp];
            }
          rope_finish(args, head, p, col0 + tok, x1 + b1, x2 + b2);
        }
      }
    } else if (SWAP && args.gated) {
      // act[m, 64 * tile + i] = bf16(silu(bf16(gate_i))) * bf16(up_i): the roundings of the unfused
      // path (product rounded to bfloat16, then the activation kernel's).  The up rows (lanes
      // 64..127) go through shared memory to the threads that hold the gate rows; the stage
      // buffers are free by now.  All four warps take the barrier, whether they gave up or not.
      float* ex = reinterpret_cast<float*>(a_s);               // [64][BN]
      constexpr int CW = BN >= 32 ? 32 : 16;
      if (ok) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if constexpr (BN >= 32) {
        // More than 16 tokens: all four warps leave their rows in shared memory, gates and ups, token-major
        // ([2][BN][64 rows]: a warp's 32 rows side by side), and then every thread takes one output column
        // for half of the tokens, so that the activation is spread over 128 threads instead of 64.
        if (ok) {
          float* mine = ex + (size_t)(r >> 6) * BN * 64 + (r & 63);
#pragma unroll 1
          for (int c = 0; c < BN; c += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) mine[(c + i) * 64] = __uint_as_float(v[i]);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok) {
          const int I = args.N / 2;
          const int row = r & 63, c0 = (r >> 6) * (BN / 2);
          const int n = (int)blockIdx.x * 64 + row;              // output column
          bf16* outb = reinterpret_cast<bf16*>(args.out);
          if (n < I) {
#pragma unroll 4
            for (int c = c0; c < c0 + BN / 2; ++c) {
              const int m = col0 + c;                            // token
              if (m >= args.M) break;
              const float g = round_to<bf16>(ex[c * 64 + row]);
              const float u = round_to<bf16>(ex[(BN + c) * 64 + row]);
              const float sl = round_to<bf16>(silu_for<bf16>(g));
              outb[(size_t)m * I + n] = __float2bfloat16_rn(sl * u);
            }
          }
        }
      } else {
      if (ok && q >= 2) {
#pragma unroll 1
        for (int c = 0; c < BN; c += CW) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c;
          if constexpr (CW == 32) {
            tmem_ld32(taddr, v);
          } else {
            uint32_t v16[16];
            tmem_ld16(taddr, v16);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = v16[i];
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < CW; ++i) ex[(r - 64) * BN + c + i] = __uint_as_float(v[i]);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok && q < 2) {
        const int I = args.N / 2;
        const int n = (int)blockIdx.x * 64 + r;                // output column
        bf16* outb = reinterpret_cast<bf16*>(args.out);
#pragma unroll 1
        for (int c = 0; c < BN; c += CW) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c;
          if constexpr (CW == 32) {
            tmem_ld32(taddr, v);
          } else {
            uint32_t v16[16];
            tmem_ld16(taddr, v16);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = v16[i];
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const int m = col0 + c + i;                        // token
            if (n < I && m < args.M) {
              const float g = round_to<bf16>(__uint_as_float(v[i]));
              const float u = round_to<bf16>(ex[r * BN + c + i]);
              const float sl = round_to<bf16>(silu_for<bf16>(g));
              outb[(size_t)m * I + n] = __float2bfloat16_rn(sl * u);
            }
          }
        }
      }
      }
    } else if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int M = args.M, N = args.N;
      float* outf = reinterpret_cast<float*>(args.out);
      bf16* outb = reinterpret_cast<bf16*>(args.out);
      const size_t split_off = (size_t)blockIdx.z * M * N;
      const bool add_bias = args.bias != nullptr && args.splits == 1;
      constexpr int CW = BN >= 32 ? 32 : 16;       // columns per tcgen05.ld
#pragma unroll 1
      for (int c = 0; c < BN; c += CW) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c;
        if constexpr (CW == 32) {
          tmem_ld32(taddr, v);
        } else {
          uint32_t v16[16];
          tmem_ld16(taddr, v16);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = v16[i];
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if constexpr (SWAP) {
          const int n = row0 + r;                  // output feature
          const float bv = (add_bias && n < N) ? to_f(args.bias[n]) : 0.f;
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const int m = col0 + c + i;            // token
            if (n < N && m < M) {
              const float x = __uint_as_float(v[i]) + bv;
              if (args.splits > 1 || args.out_is_float) outf[split_off + (size_t)m * N + n] = x;
              else outb[(size_t)m * N + n] = __float2bfloat16_rn(x);
            }
          }
        } else {
          const int m = row0 + r;                  // token
          if (m < M) {
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
              const int n = col0 + c + i;
              if (n >= N) continue;
              float x0 = __uint_as_float(v[i]), x1 = __uint_as_float(v[i + 1]);
              if (add_bias) {
                x0 += to_f(args.bias[n]);
                if (n + 1 < N) x1 += to_f(args.bias[n + 1]);
              }
              if (args.splits > 1 || args.out_is_float) {
                outf[split_off + (size_t)m * N + n] = x0;
                if (n + 1 < N) outf[split_off + (size_t)m * N + n + 1] = x1;
              } else if (n + 1 < N && ((N & 1) == 0)) {
                *reinterpret_cast<__nv_bfloat162*>(outb + (size_t)m * N + n) = __floats2bfloat162_rn(x0, x1);
              } else {
                outb[(size_t)m * N + n] = __float2bfloat16_rn(x0);
                if (n + 1 < N) outb[(size_t)m * N + n + 1] = __float2bfloat16_rn(x1);
              }
            }
          }
        }
      }
    }
  }
  if (SWAP && args.rope == 2) {
    // Block z of the cluster finishes tokens z, z + splits, ...: each thread sums one pair of columns
    // out of every peer's shared memory, in split order (the sums of the ticket path, bit for bit).
    __syncwarp();
    cluster_sync_all();
    if (BN >= 32 && warp >= 2) {
      // more than 16 tokens: four neighbouring pairs a thread (16 bytes from every peer), eight tokens a pass
      const int r = (warp & 3) * 32 + lane;
      const int q4 = (r & 15) * 4, tsub = r >> 4;
      const int half = args.D >> 1, in_tile = q4 / half, p = q4 - in_tile * half;
      const int head = (int)blockIdx.x * (128 / args.D) + in_tile;
      const int c1 = in_tile * args.D + p, c2 = c1 + half;
      const float* ex = reinterpret_cast<const float*>(a_s);
      float b1[4] = {0.f, 0.f, 0.f, 0.f}, b2[4] = {0.f, 0.f, 0.f, 0.f};
      if (args.bias != nullptr && head < args.H + 2 * args.KVH) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          b1[i] = to_f(args.bias[head * args.D + p + i]);
          b2[i] = to_f(args.bias[head * args.D + p + half + i]);
        }
      }
      const int tokens = min(BN, args.M - col0);
      for (int tok = (int)blockIdx.z + tsub * args.splits; tok < tokens; tok += 8 * args.splits) {
        float4 lo[8], hi[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          if (sp < args.splits) {
            lo[sp] = ld_peer_v4(peer_shared(ex + tok * 128 + c1, sp));
            hi[sp] = ld_peer_v4(peer_shared(ex + tok * 128 + c2, sp));
          }
        float x1[4] = {0.f, 0.f, 0.f, 0.f}, x2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          if (sp < args.splits) {
            x1[0] += lo[sp].x; x1[1] += lo[sp].y; x1[2] += lo[sp].z; x1[3] += lo[sp].w;
            x2[0] += hi[sp].x; x2[1] += hi[sp].y; x2[2] += hi[sp].z; x2[3] += hi[sp].w;
          }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          x1[i] += b1[i];
          x2[i] += b2[i];
        }
        rope_finish4(args, head, p, col0 + tok, x1, x2);
      }
    } else if (warp >= 2) {
      const int r = (warp & 3) * 32 + lane;
      const RopePair rp = rope_pair(args, blockIdx.x, r);
      const int head = rp.head, p = rp.p, tg = r >> 6;
      const float* ex = reinterpret_cast<const float*>(a_s);
      const bool real = head < args.H + 2 * args.KVH;
      const float b1 = (args.bias != nullptr && real) ? to_f(args.bias[head * args.D + p]) : 0.f;
      const float b2 = (args.bias != nullptr && real) ? to_f(args.bias[head * args.D + p + (args.D >> 1)]) : 0.f;
      const int tokens = min(BN, args.M - col0);
      for (int tok = (int)blockIdx.z + tg * args.splits; tok < tokens; tok += 2 * args.splits) {
        float lo[8], hi[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          if (sp < args.splits) {
            lo[sp] = ld_peer_f32(peer_shared(ex + tok * 128 + rp.c1, sp));
            hi[sp] = ld_peer_f32(peer_shared(ex + tok * 128 + rp.c2, sp));
          }
        float x1 = 0.f, x2 = 0.f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          if (sp < args.splits) {
            x1 += lo[sp];
            x2 += hi[sp];
          }
        rope_finish(args, head, p, col0 + tok, x1 + b1, x2 + b2);
      }
    }
    __syncwarp();
    cluster_sync_all();                              // no block leaves while a peer still reads it
  } else if (fuse_resid) {
    // Block z of the cluster finishes tokens z, z + splits, ...: each thread sums one output out of
    // every peer's shared memory in split order, adds the bias, rounds as a product's epilogue does
    // and adds the result to the residual row in place (what ts_reduce_rmsnorm does, bit for bit).
    const bool many = args.splits > 1;
    __syncwarp();
    if (many) cluster_sync_all();
    else __syncthreads();
    if (warp >= 2) {
      const int r = (warp & 3) * 32 + lane;
      const float* ex = reinterpret_cast<const float*>(a_s);
      const int tokens = min(BN, args.M - col0);
      if (BN >= 32 && (args.N & 3) == 0) {
        // more than 16 tokens: four outputs a thread (16 bytes from every peer), four tokens a pass (with 8
        // tokens the one-output-a-thread loop below is the shorter one: 1.398 against 1.408 ms a step)
        const int n = row0 + 4 * (r & 31), tsub = r >> 5;
        float bv[4] = {0.f, 0.f, 0.f, 0.f};
        if (args.bias != nullptr && n < args.N) {
          const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(args.bias + n);
          const float2 b0 = __bfloat1622float2(bp[0]), b1 = __bfloat1622float2(bp[1]);
          bv[0] = b0.x; bv[1] = b0.y; bv[2] = b1.x; bv[3] = b1.y;
        }
        for (int tok = (int)blockIdx.z + tsub * args.splits; tok < tokens; tok += 4 * args.splits) {
          float4 part[8];
          const float* mine = ex + tok * 128 + 4 * (r & 31);
#pragma unroll
          for (int sp = 0; sp < 8; ++sp)
            if (sp < args.splits) part[sp] = many ? ld_peer_v4(peer_shared(mine, sp)) : *reinterpret_cast<const float4*>(mine);
          float x[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int sp = 0; sp < 8; ++sp)
            if (sp < args.splits) {
              x[0] += part[sp].x; x[1] += part[sp].y; x[2] += part[sp].z; x[3] += part[sp].w;
            }
          if (n < args.N) {
            uint2* dst = reinterpret_cast<uint2*>(args.resid + (size_t)(col0 + tok) * args.N + n);
            uint2 old = *dst;
            const float2 r0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&old.x));
            const float2 r1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&old.y));
            __nv_bfloat162 o0 = __floats2bfloat162_rn(round_to<bf16>(x[0] + bv[0]) + r0.x, round_to<bf16>(x[1] + bv[1]) + r0.y);
            __nv_bfloat162 o1 = __floats2bfloat162_rn(round_to<bf16>(x[2] + bv[2]) + r1.x, round_to<bf16>(x[3] + bv[3]) + r1.y);
            old.x = *reinterpret_cast<unsigned*>(&o0);
            old.y = *reinterpret_cast<unsigned*>(&o1);
            *dst = old;
          }
        }
      } else {
        const int n = row0 + r;
        const float bv = (args.bias != nullptr && n < args.N) ? to_f(args.bias[n]) : 0.f;
        for (int tok = (int)blockIdx.z; tok < tokens; tok += args.splits) {
          float part[8];
#pragma unroll
          for (int sp = 0; sp < 8; ++sp)
            if (sp < args.splits) part[sp] = many ? ld_peer_f32(peer_shared(ex + tok * 128 + r, sp)) : ex[tok * 128 + r];
          float x = 0.f;
#pragma unroll
          for (int sp = 0; sp < 8; ++sp)
            if (sp < args.splits) x += part[sp];
          if (n < args.N) {
            bf16* dst = args.resid + (size_t)(col0 + tok) * args.N + n;
            *dst = __float2bfloat16_rn(round_to<bf16>(x + bv) + to_f(*dst));
          }
        }
      }
    }
    __syncwarp();
    if (many) cluster_sync_all();
    else __syncthreads();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// out[m, n] = sum over splits (ascending) of part[s, m, n] + bias[n]
__global__ void splitk_reduce_kernel(void* out, const float* __restrict__ part, const bf16* __restrict__ bias,
                                     int M, int N, int splits, int out_is_float) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)M * N;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += part[(size_t)s * total + idx];
    if (bias != nullptr) acc += to_f(bias[idx % N]);
    if (out_is_float) reinterpret_cast<float*>(out)[idx] = acc;
    else reinterpret_cast<bf16*>(out)[idx] = __float2bfloat16_rn(acc);
  }
}

__device__ int g_gemm_status = 0;       // 0 = fine; otherwise the wait that ran out (see ts_linear_tc_status)

int* status_word() {
  static int* p = nullptr;
  if (p == nullptr && cudaGetSymbolAddress((void**)&p, g_gemm_status) != cudaSuccess) p = nullptr;
  return p;
}

// Raises the kernel's dynamic shared memory limit to `smem` if it is lower (never lowers it).
template <int BN, int STAGES, bool SWAP, int KSUB>
cudaError_t allow_smem(size_t smem) {
  static size_t allowed = 0;                        // (one device's worth: the attribute is per device, the library serves one)
  if (smem <= allowed) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SWAP, KSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) allowed = smem;
  return e;
}

template <int BN, int STAGES, bool SWAP, int KSUB = 1>
int launch(const CUtensorMap& rows_map, const CUtensorMap& cols_map, const GemmArgs& args, dim3 grid, cudaStream_t s,
           dim3 cluster = dim3(1, 1, 1)) {
  constexpr size_t smem = gemm_smem_bytes(BN, STAGES, KSUB);
  {
    cudaError_t e = allow_smem<BN, STAGES, SWAP, KSUB>(smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_linear_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
  }
  ts_launch_cluster(gemm_tc_kernel<BN, STAGES, SWAP, KSUB>, cluster, dim3(grid), dim3(GEMM_THREADS), smem, s, rows_map,
                    cols_map, args);
  TS_LAUNCH_CHECK();
}

// How many clusters of `splits` blocks of this kernel the device holds at once (asked once per count; 0: none).
template <int BN, int STAGES, bool SWAP, int KSUB = 1>
int cluster_fits(int splits) {
  constexpr size_t smem = gemm_smem_bytes(BN, STAGES, KSUB);
  static int known[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (splits < 2 || splits > 8) return 0;
  if (known[splits] < 0) {
    known[splits] = 0;
    auto kernel = gemm_tc_kernel<BN, STAGES, SWAP, KSUB>;
    if (allow_smem<BN, STAGES, SWAP, KSUB>(smem) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1, 1, splits);
      cfg.blockDim = dim3(GEMM_THREADS);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = (unsigned)splits;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1) known[splits] = clusters;
    }
    cudaGetLastError();                              // a refusal above is an answer, not an error
  }
  return known[splits];
}

}  // namespace

int* ts_gemm_status_word() { return status_word(); }

// Shapes this kernel takes: K a multiple of 8 (TMA rows must be 16-byte multiples), pointers 16-byte aligned.
TS_API int ts_linear_tc_supported(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && (K % 8) == 0; }

// Float scratch needed (elements) for a product the kernel would split over K.
TS_API long long ts_linear_tc_scratch_floats(int M, int N, int splits) { return splits > 1 ? (long long)splits * M * N : 0; }

// The block status word: 0 = fine; 1/2/3 = a producer/MMA/epilogue wait ran out.  Reading it
// synchronises the device; meant for tests and post-mortems.
TS_API int ts_linear_tc_status() {
  int* p = status_word();
  int v = -1;
  if (p != nullptr) cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

// out[M, N] (bf16, or float when out_is_float) = x[M, K] . w[N, K]^T + bias.  `splits` > 1 cuts K
// (weights-on-rows orientation only) and needs `scratch` of ts_linear_tc_scratch_floats() floats.
// defer != 0: leave the float partial sums [splits, M, N] in `scratch` (also for one split), add no bias
// and skip the reduction: the caller's next kernel (ts_reduce_rmsnorm) finishes the sum.  The
// number of splits actually used is returned through *splits_used when it is not null.
TS_API int ts_linear_tc_ex(void* out, const void* x, const void* w, const void* bias, void* scratch, int M, int N,
                           int K, int out_is_float, int splits, int defer, int* splits_used, void* stream);

TS_API int ts_linear_tc(void* out, const void* x, const void* w, const void* bias, void* scratch, int M, int N,
                        int K, int out_is_float, int splits, void* stream) {
  return ts_linear_tc_ex(out, x, w, bias, scratch, M, N, K, out_is_float, splits, 0, nullptr, stream);
}

TS_API int ts_linear_tc_ex(void* out, const void* x, const void* w, const void* bias, void* scratch, int M, int N,
                           int K, int out_is_float, int splits, int defer, int* splits_used, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!ts_linear_tc_supported(M, N, K)) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc: K = %d is not a multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w) & 15) TS_REFUSE(TS_ERR_ALIGN, "ts_linear_tc: operands must be 16-byte aligned");
  int* status = status_word();
  if (status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_linear_tc: no status word");
  cudaStream_t s = (cudaStream_t)stream;
  const int total_kb = ceil_div(K, BK);
  GemmArgs a;
  a.out = out;
  a.bias = (const bf16*)bias;
  a.M = M; a.N = N; a.K = K;
  a.out_is_float = out_is_float;
  a.gated = 0;
  a.rope = 0;
  a.status = status;
  const bool swap = M <= 128;
  if (!swap) splits = 1;
  if (splits < 1) splits = 1;
  if (splits > total_kb) splits = total_kb;
  int per = ceil_div(total_kb, splits);
  splits = ceil_div(total_kb, per);                 // every split owns at least one k-block
  a.k_blocks_per_split = per;
  a.splits = splits;
  if (splits_used != nullptr) *splits_used = splits;
  if (splits > 1 || defer) {
    if (scratch == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_linear_tc: %d splits need scratch", splits);
    a.out = scratch;
  }
  if (defer) {
    a.bias = nullptr;
    a.out_is_float = 1;
  }
  CUtensorMap rows_map, cols_map;
  int rc;
  if (swap) {
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    if (!tensor_map(&rows_map, w, N, K, BM) || !tensor_map(&cols_map, x, M, K, bn))
      TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc: cuTensorMapEncodeTiled failed");
    dim3 grid(ceil_div(N, BM), ceil_div(M, bn), splits);
    // Several waves of blocks (the output head): three stages leave room for two blocks on an SM, so
    // one block's pipeline fill and epilogue hide behind the other's main loop.
    const bool waves = (long long)grid.x * grid.y * grid.z >= 592;
    if (bn == 16 && waves) rc = launch<16, 3, true, 2>(rows_map, cols_map, a, grid, s);
    else if (bn == 16) rc = launch<16, 4, true, 2>(rows_map, cols_map, a, grid, s);
    else if (bn == 32) rc = launch<32, 4, true>(rows_map, cols_map, a, grid, s);
    else if (bn == 64) rc = launch<64, 4, true, 2>(rows_map, cols_map, a, grid, s);
    else rc = launch<128, 4, true>(rows_map, cols_map, a, grid, s);
  } else {
    if (!tensor_map(&rows_map, x, M, K, BM) || !tensor_map(&cols_map, w, N, K, 256))
      TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc: cuTensorMapEncodeTiled failed");
    dim3 grid(ceil_div(M, BM), ceil_div(N, 256), 1);
    if (grid.y > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_linear_tc: N = %d too large", N);
    rc = launch<256, 4, false>(rows_map, cols_map, a, grid, s);
  }
  if (rc != 0) return rc;
  if (splits > 1 && !defer) {
    const size_t total = (size_t)M * N;
    const int blocks = (int)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256);
    ts_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, out, (const float*)scratch, (const bf16*)bias, M, N, splits, out_is_float);
    TS_LAUNCH_CHECK();
  }
  return 0;
}

// act[M, N2 / 2] (bf16) = silu(g) * u where [g | u] = x[M, K] . w[N2, K]^T and the rows of w come in
// blocks of 128: the 64 gate rows j*64.. then the 64 up rows j*64...  At most 128 tokens, N2 a
// multiple of 128, no bias: what the fused epilogue takes (TS_ERR_UNSUPPORTED otherwise, and the
// caller does product and activation apart).
TS_API int ts_linear_tc_gated(void* act, const void* x, const void* w, int M, int N2, int K, void* stream) {

  if (M <= 0 || N2 <= 0) return 0;
  if (M > 128 || N2 % 128 != 0 || !ts_linear_tc_supported(M, N2, K))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_gated: M=%d N=%d K=%d is not taken by this kernel", M, N2, K);
  if (((uintptr_t)x | (uintptr_t)w) & 15) TS_REFUSE(TS_ERR_ALIGN, "ts_linear_tc_gated: operands must be 16-byte aligned");
  int* status = status_word();
  if (status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_linear_tc_gated: no status word");
  GemmArgs a;
  a.out = act;
  a.bias = nullptr;
  a.M = M; a.N = N2; a.K = K;
  a.out_is_float = 0;
  a.gated = 1;
  a.rope = 0;
  a.status = status;
  a.k_blocks_per_split = ceil_div(K, BK);
  a.splits = 1;
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap rows_map, cols_map;
  if (!tensor_map(&rows_map, w, N2, K, BM) || !tensor_map(&cols_map, x, M, K, bn))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_gated: cuTensorMapEncodeTiled failed");
  dim3 grid(N2 / BM, ceil_div(M, bn), 1);
  cudaStream_t s = (cudaStream_t)stream;
  if (bn == 16) return launch<16, 4, true, 2>(rows_map, cols_map, a, grid, s);
  if (bn == 32) return launch<32, 4, true>(rows_map, cols_map, a, grid, s);
  if (bn == 64) return launch<64, 4, true>(rows_map, cols_map, a, grid, s);
  return launch<128, 4, true>(rows_map, cols_map, a, grid, s);
}

// Floats of scratch for ts_linear_tc_qkv_rope; `tiles`: 128-row tiles of the product, ceil((H + 2 KVH) * D / 128).
TS_API long long ts_linear_tc_qkv_rope_scratch_floats(int M, int tiles, int splits) {
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  return (long long)tiles * ceil_div(M, bn) * splits * bn * 128;
}

// qkv[M, (H + 2 KVH) * D] = x[M, K] . w^T + bias with q and k heads rotated (full-width rotate-half,
// tables [positions][D / 2] float, rounded to bfloat16 at use) and the new keys and values written into
// the cache pages (slot < 0: not written; k_cache null: no cache write), all in the product's own
// epilogue.  Head size D = 64 or 128, at most 128 tokens (more than 32 only where the splits of a tile can be
// one cluster and all clusters fit the chip: the block that comes last for a tile would otherwise sum token
// after token, which a kernel of its own does faster), up to 16 splits over K.  `scratch` holds
// ts_linear_tc_qkv_rope_scratch_floats() floats, `counters` one zero int per (tile, block of tokens).
TS_API int ts_linear_tc_qkv_rope(void* qkv, const void* x, const void* w, const void* bias, void* scratch, int* counters,
                                 const int* positions, const float* cos_t, const float* sin_t, const int* slots,
                                 void* k_cache, void* v_cache, int M, int H, int KVH, int D, int page, int K, int splits,
                                 void* stream) {
  if (M <= 0) return 0;
  const int heads = H + 2 * KVH, N = heads * D;
  if (M > 128 || H <= 0 || KVH <= 0 || (D != 64 && D != 128) || !ts_linear_tc_supported(M, N, K))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_qkv_rope: M=%d heads=%d D=%d K=%d is not taken by this kernel", M, heads, D, K);
  if (scratch == nullptr || counters == nullptr || positions == nullptr || cos_t == nullptr || sin_t == nullptr)
    TS_REFUSE(TS_ERR_SHAPE, "ts_linear_tc_qkv_rope: scratch, counters, positions and tables are needed");
  if (k_cache != nullptr && (v_cache == nullptr || slots == nullptr || page <= 0))
    TS_REFUSE(TS_ERR_SHAPE, "ts_linear_tc_qkv_rope: the cache write needs both caches, slots and the page size");
  if (((uintptr_t)x | (uintptr_t)w) & 15) TS_REFUSE(TS_ERR_ALIGN, "ts_linear_tc_qkv_rope: operands must be 16-byte aligned");
  int* status = status_word();
  if (status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_linear_tc_qkv_rope: no status word");
  const int total_kb = ceil_div(K, BK);
  if (splits < 1) splits = 1;
  if (splits > 16) splits = 16;
  if (splits > total_kb) splits = total_kb;
  const int per = ceil_div(total_kb, splits);
  splits = ceil_div(total_kb, per);
  GemmArgs a;
  a.out = qkv;
  a.bias = (const bf16*)bias;
  a.M = M; a.N = N; a.K = K;
  a.out_is_float = 0;
  a.gated = 0;
  a.rope = 1;
  a.status = status;
  a.k_blocks_per_split = per;
  a.splits = splits;
  a.rope_part = (float*)scratch;
  a.rope_counters = counters;
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
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap rows_map, cols_map;
  if (!tensor_map(&rows_map, w, N, K, BM) || !tensor_map(&cols_map, x, M, K, bn))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_qkv_rope: cuTensorMapEncodeTiled failed");
  dim3 grid(ceil_div(N, BM), ceil_div(M, bn), splits);
  cudaStream_t s = (cudaStream_t)stream;
  // 2 to 8 splits of a tile as one thread-block cluster: the partial sums cross through shared
  // memory instead of scratch, a fence and a ticket.
  // (a step of 1 or 2 tokens is about 2 % slower with the cluster than with the ticket, one of 4 or 8
  // tokens 1 % faster, one of 16 tokens 10 % faster: the ticket's last block sums token after token)
  const bool want_cluster = ts_clusters_enabled() && splits >= 2 && splits <= 8 && M >= 4;
  const dim3 cl(1, 1, splits);
#define TS_ROPE_LAUNCH(...)                                           \
  do {                                                                \
    if (want_cluster && (int)(grid.x * grid.y) <= cluster_fits<__VA_ARGS__>(splits)) { \
      a.rope = 2;                                                     \
      return launch<__VA_ARGS__>(rows_map, cols_map, a, grid, s, cl); \
    }                                                                 \
    if (M > 32)                                                       \
      TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_qkv_rope: %d tokens only with the splits as clusters", M); \
    return launch<__VA_ARGS__>(rows_map, cols_map, a, grid, s);       \
  } while (0)
  if (bn == 16) TS_ROPE_LAUNCH(16, 4, true, 2);
  if (bn == 32) TS_ROPE_LAUNCH(32, 4, true);
  if (bn == 64) TS_ROPE_LAUNCH(64, 4, true);
  TS_ROPE_LAUNCH(128, 4, true);
#undef TS_ROPE_LAUNCH
}

// resid[M, N] (bf16, in place) = bf16(resid + bf16(x[M, K] . w[N, K]^T + bias)): a few-token product whose
// K splits are one thread-block cluster that sums its partial results through shared memory and adds
// them to the residual stream itself: the product, its reduction and the residual add of the norm that
// follows, in one kernel, with the same roundings.  At most 128 tokens, at most 8 splits.
// TS_ERR_UNSUPPORTED when the clusters are switched off or do not fit the device at once.
TS_API int ts_linear_tc_resid(void* resid, const void* x, const void* w, const void* bias, int M, int N, int K, int splits,
                              void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || !ts_linear_tc_supported(M, N, K))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_resid: M=%d N=%d K=%d is not taken by this kernel", M, N, K);
  if (resid == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_linear_tc_resid: no residual");
  if (((uintptr_t)x | (uintptr_t)w) & 15) TS_REFUSE(TS_ERR_ALIGN, "ts_linear_tc_resid: operands must be 16-byte aligned");
  int* status = status_word();
  if (status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_linear_tc_resid: no status word");
  const int total_kb = ceil_div(K, BK);
  if (splits < 1) splits = 1;
  if (splits > 8) splits = 8;
  if (splits > total_kb) splits = total_kb;
  const int per = ceil_div(total_kb, splits);
  splits = ceil_div(total_kb, per);
  if (splits > 1 && !ts_clusters_enabled()) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_resid: thread-block clusters are switched off");
  GemmArgs a;
  a.out = nullptr;
  a.bias = (const bf16*)bias;
  a.M = M; a.N = N; a.K = K;
  a.out_is_float = 0;
  a.gated = 0;
  a.rope = 0;
  a.status = status;
  a.k_blocks_per_split = per;
  a.splits = splits;
  a.resid = (bf16*)resid;
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap rows_map, cols_map;
  if (!tensor_map(&rows_map, w, N, K, BM) || !tensor_map(&cols_map, x, M, K, bn))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_resid: cuTensorMapEncodeTiled failed");
  dim3 grid(ceil_div(N, BM), ceil_div(M, bn), splits);
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 cl(1, 1, splits);
#define TS_RESID_LAUNCH(...)                                          \
  do {                                                                \
    if (splits > 1 && (int)(grid.x * grid.y) > cluster_fits<__VA_ARGS__>(splits)) \
      TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_linear_tc_resid: %d clusters of %d blocks do not fit the device at once", (int)(grid.x * grid.y), splits); \
    return launch<__VA_ARGS__>(rows_map, cols_map, a, grid, s, cl);   \
  } while (0)
  if (bn == 16) TS_RESID_LAUNCH(16, 4, true, 2);
  if (bn == 32) TS_RESID_LAUNCH(32, 4, true);
  if (bn == 64) TS_RESID_LAUNCH(64, 4, true, 2);
  TS_RESID_LAUNCH(128, 4, true);
#undef TS_RESID_LAUNCH
}
