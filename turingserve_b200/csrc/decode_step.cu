// One whole decode step of a pre-norm decoder (RMSNorm, rotary grouped-query attention over the paged
// cache, gated SiLU feed-forward, output head) for up to 16 single-token requests, as ONE persistent
// kernel: one block per SM, every weight streamed exactly once through a ring of shared-memory stages
// that never drains between the products of a layer or between layers.
//
// The same step out of separate kernels (turingserve/model/qwen2.py:38-61 is the recipe; this
// library's q/k/v, attention, output, gate/up and down kernels are the separate form) pays, per
// kernel, a grid drain, a pipeline fill and a memory round trip during which no weight moves: seven
// links of 3 to 12 microseconds a layer where the layer's weights need 14.  Here the phases of a
// layer are separated by grid-wide barriers (a counter in global memory), and while a block waits at
// one, its producer warp keeps fetching the weights of the phases to come: weights depend on nothing.
//
// Block = 7 warps:
//   warp 0     weight producer: one lane walks the block's whole list of (tile, k-block) units, layer
//              after layer, and issues the TMA loads into the ring as stages free up; further ahead
//              it asks for the weights to be brought into L2 (cp.async.bulk.prefetch).
//   warp 1     issues tcgen05.mma (one lane): tile rows are weight rows (outputs), the 16 columns are
//              the tokens; accumulators in tensor memory, two of them, so one is filled while the
//              other is read back.
//   warp 2     activation loader: for products whose input another phase wrote (attention output,
//              activation), copies the unit's [16 tokens x 64] slices into the stage with cp.async.
//   warps 3-6  everything else: the norm that opens a phase (written straight into the MMA operand
//              layout), reading accumulators back, split-K partial sums to scratch and the finish by
//              the block that comes last for a tile (a ticket, nobody waits): bias + rotary + cache
//              write, residual add, SiLU*mul, logits; the decode attention (mma.sync over cp.async
//              tiles, the four warps on disjoint keys); the grid barriers.
//
// Every wait (mbarrier, shared-memory flag, grid barrier) is bounded: when one runs out the block
// records where in the status word, raises the step's abort flag so that the other blocks stop
// waiting too, and leaves through the common exit, which frees its tensor memory.
//
// Rounding points are those of the separate kernels: a product is rounded to bfloat16 before the
// residual add, the sum again; the norm's x * rstd is rounded before the scale; SiLU and the
// product with `up` round as the activation kernel does; probabilities are rounded to bfloat16 for
// the second attention product; logits leave the accumulator unrounded.
#include <string.h>

#include "common.cuh"
#include "decode_step.h"
#include "mma_utils.cuh"
#include "tc_utils.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;                    // tile rows (weight rows) = TMEM lanes
constexpr int BN = TS_STEP_MAX_TOKENS;     // tile columns = tokens
constexpr int W_BYTES = BM * BK * 2;       // 16 KB of weights per k-block
constexpr int X_BYTES = BN * BK * 2;       // 2 KB of activations per k-block
constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int NUM_WARPS = 7;
constexpr int NUM_THREADS = NUM_WARPS * 32;
constexpr int CW0 = 3;                     // first compute warp
constexpr int CT = 128;                    // compute threads
constexpr int UMMA_K = 16;
constexpr int ATT_TILE = 64;
constexpr int D = 128;                     // head size this kernel is written for
constexpr int PAGES_S = 256;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int EX_BYTES = 5120;               // the gated epilogue's exchange [64][16] floats; the attention's q rows and new key/value
constexpr int FULL_COUNT = 33;             // arrivals a stage needs: the producer's expect_tx + 32 loader lanes

enum Kind : int { K_QKV = 0, K_O = 1, K_GU = 2, K_DOWN = 3, K_HEAD = 4, K_ATTN = 5 };   // 0..4 index TsStepArgs::shape

struct Unit {
  int kind, layer, tile, part, kb0, kb1;
};

// Walks a block's units in the order every role of the block agrees on: layer by layer the q/k/v,
// output, gate/up and down products, then the head.  Unit u of a product is (tile u / S, part u % S);
// block c takes units (c + rot) % blocks, + blocks, ...
struct Walker {
  int layer, slot, u;      // slot: position in the layer's order q/k/v, attention, output, gate/up, down
  __device__ void start() {
    layer = 0;
    slot = 0;
    u = -1;
  }
  __device__ bool next(const TsStepArgs& a, int cta, int nb, Unit& out) {
    while (true) {
      if (layer > a.L) return false;
      const int kind = layer == a.L ? K_HEAD : (slot == 0 ? K_QKV : slot == 1 ? K_ATTN : slot == 2 ? K_O : slot == 3 ? K_GU : K_DOWN);
      if (kind == K_ATTN) {
        // one attention unit a block: its keys and values come through the ring like weights
        slot = 2;
        if (cta < a.T * a.KVH * a.attn_splits) {
          out.kind = K_ATTN;
          out.layer = layer;
          out.tile = out.part = out.kb0 = out.kb1 = 0;
          return true;
        }
        continue;
      }
      const TsStepShape& sh = a.shape[kind];
      if (u < 0) u = (cta + sh.rot) % nb;
      if (u < sh.R * sh.S) {
        out.kind = kind;
        out.layer = layer;
        out.tile = u / sh.S;
        out.part = u % sh.S;
        out.kb0 = out.part * sh.per;
        out.kb1 = min(sh.KB, out.kb0 + sh.per);
        u += nb;
        return true;
      }
      u = -1;
      if (layer == a.L) {
        layer = a.L + 1;
        continue;
      }
      if (++slot == 5) {
        slot = 0;
        ++layer;
      }
    }
  }
};

// Does block `cta` own a unit of product `kind`?
__device__ __forceinline__ bool has_units(const TsStepArgs& a, int kind, int cta, int nb) {
  const TsStepShape& sh = a.shape[kind];
  return (cta + sh.rot) % nb < sh.R * sh.S;
}

__device__ __forceinline__ const CUtensorMap* map_of(const TsStepArgs& a, int kind, int layer) {
  return reinterpret_cast<const CUtensorMap*>(a.maps) + (kind == K_HEAD ? 4 * a.L : 4 * layer + kind);
}

// ---- bounded waits on plain flags ---------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_cta(const volatile int* p) {
  int v;
  asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32((const void*)p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta(volatile int* p, int v) {
  asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"(smem_u32((const void*)p)), "r"(v) : "memory");
}

struct Abort {
  volatile int* flag;      // shared: this block gives up
  int* status;             // global status word
  int* step_abort;         // global: the step gives up (other blocks stop waiting)
  __device__ __forceinline__ bool raised() const { return *flag != 0; }
  __device__ __forceinline__ void raise(int code) const {
    atomicCAS(status, 0, code);
    atomicExch(step_abort, 1);
    *flag = 1;
  }
};

// Waits until the shared counter *p reaches `target`.
__device__ __forceinline__ bool wait_shared_ge(volatile int* p, int target, const Abort& ab, int code) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    if (ld_acquire_cta(p) >= target) return true;
    __nanosleep(40);                                   // a polling warp must not take issue slots from the working ones
    if ((i & 63u) == 63u) {
      if (ab.raised()) return false;
      if (clock64() - t0 > 2 * WAIT_LIMIT_CYCLES) break;
    }
  }
  ab.raise(code);
  return false;
}
// The same for a whole warp: one lane polls.
__device__ __forceinline__ bool warp_wait_shared_ge(volatile int* p, int target, const Abort& ab, int code, int lane) {
  bool ok = true;
  if (lane == 0) ok = wait_shared_ge(p, target, ab, code);
  return __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
}

[[maybe_unused]] __device__ __forceinline__ bool mwait(uint64_t* bar, uint32_t parity, const Abort& ab, int code) {
  if (mbar_wait(bar, parity, ab.status, code, ab.flag)) return true;
  atomicExch(ab.step_abort, 1);
  return false;
}
// The same without the hardware's suspend between polls: for the hand-overs a phase's length hangs on
// (norm -> products -> accumulator read-back), where the waiter's reaction time counts.
__device__ __forceinline__ bool mwait_now(uint64_t* bar, uint32_t parity, const Abort& ab, int code) {
  if (mbar_wait_spin(bar, parity, ab.status, code, ab.flag)) return true;
  atomicExch(ab.step_abort, 1);
  return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, int n) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// True when `ok` holds in all 128 compute threads (a barrier among them as well).
__device__ __forceinline__ bool compute_all(bool ok) {
  int r;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n bar.red.and.pred q, 1, 128, p;\n selp.u32 %0, 1, 0, q;\n}\n"
      : "=r"(r) : "r"((int)ok) : "memory");
  return r != 0;
}

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// Shared memory of a block: one base address, the rest by offset (a pointer per field would keep two
// dozen registers busy through every phase).
struct Smem {
  unsigned char* base;       // 1024-byte aligned
  int nst;                   // ring stages
  int work_bytes;
  __device__ __forceinline__ unsigned char* ring_() const { return base; }                       // [stages][STAGE_BYTES]
  // the norm's output (MMA operand, [k-blocks][16][64] swizzled) or the attention's stages
  __device__ __forceinline__ unsigned char* work_() const { return base + (size_t)nst * STAGE_BYTES; }
  __device__ __forceinline__ float* ex_() const { return reinterpret_cast<float*>(work_() + work_bytes); }   // [64][16] exchange of the gated epilogue
  __device__ __forceinline__ uint64_t* full_() const { return reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(ex_()) + EX_BYTES); }  // [stages]
  __device__ __forceinline__ uint64_t* empty_() const { return full_() + nst; }                    // [stages]
  __device__ __forceinline__ uint64_t* acc_full_() const { return empty_() + nst; }                // [2]
  __device__ __forceinline__ uint64_t* acc_empty_() const { return acc_full_() + 2; }              // [2]
  __device__ __forceinline__ uint64_t* x_ready_() const { return acc_empty_() + 2; }               // [1]
  __device__ __forceinline__ uint32_t* tmem_slot_() const { return reinterpret_cast<uint32_t*>(x_ready_() + 1); }
  // (the barriers end 8 bytes past a multiple of 16: two words further the integers start 16-byte aligned,
  // which the cp.async copies into the scale slots behind them need)
  __device__ __forceinline__ volatile int* ints_() const { return reinterpret_cast<volatile int*>(tmem_slot_() + 2); }
  __device__ __forceinline__ volatile int* abort_flag_() const { return ints_(); }
  __device__ __forceinline__ volatile int* w_issued_() const { return ints_() + 1; }   // k-blocks whose weights the producer has asked for
  __device__ __forceinline__ volatile int* phase_open_() const { return ints_() + 2; } // grid barriers this block has passed
  __device__ __forceinline__ volatile int* flag_() const { return ints_() + 3; }       // compute warps' broadcast word (ticket results)
  __device__ __forceinline__ int* pos_() const { return const_cast<int*>(ints_()) + 4; }           // [16] the step's positions
  __device__ __forceinline__ int* seq_() const { return pos_() + BN; }                             // [16] context lengths
  __device__ __forceinline__ int* slot_() const { return seq_() + BN; }                            // [groups][16] cache slots of the new tokens
  // [groups][PAGES_S] pages of this block's share of the keys (the same in every layer of a group)
  __device__ __forceinline__ int* pages_() const { return slot_() + TS_STEP_MAX_GROUPS * BN; }
  // [2][hidden] scale of the norm in use and of the next one (brought in while the phases between them run)
  __device__ __forceinline__ unsigned char* scale_(int slot, int bytes) const {
    return reinterpret_cast<unsigned char*>(pages_() + TS_STEP_MAX_GROUPS * PAGES_S) + 2 * sizeof(TsStepLayer) + (size_t)slot * bytes;
  }
  // [2] the table entries of the layer in work and of the next one
  __device__ __forceinline__ TsStepLayer* layer_(int slot) const {
    return reinterpret_cast<TsStepLayer*>(pages_() + TS_STEP_MAX_GROUPS * PAGES_S) + slot;
  }
};

// This block's share of the keys of its attention unit, for a group whose layers see `window` keys.
struct KeyRange {
  int b, kvh, split, k_begin, k_end, page_first, n_pages;
};
__device__ __forceinline__ KeyRange key_range(const TsStepArgs& a, int unit, int seq_len, int window) {
  KeyRange k;
  const int NS = a.attn_splits;
  k.b = unit / (a.KVH * NS);
  k.kvh = (unit / NS) % a.KVH;
  k.split = unit % NS;
  const int lo = window > 0 ? max(0, seq_len - window) : 0;
  const int span = max(seq_len - lo, 0);
  int chunk = (span + NS - 1) / NS;
  chunk = (chunk + ATT_TILE - 1) / ATT_TILE * ATT_TILE;
  k.k_begin = lo + k.split * chunk;
  k.k_end = min(seq_len, k.k_begin + chunk);
  k.page_first = k.k_begin / a.page;
  k.n_pages = k.k_end > k.k_begin ? (k.k_end - 1) / a.page - k.page_first + 1 : 0;
  return k;
}

// A time stamp for the timeline: slot k (2..7) of the interval that ends at barrier `seq`.
__device__ __forceinline__ void mark(const TsStepArgs& a, int seq, int k, int ct) {
  if (a.trace != nullptr && ct == 0) a.trace[((size_t)blockIdx.x * (5 * a.L + 2) + (seq - 1)) * 8 + k] = clock64();
}

// ---- the grid barrier ---------------------------------------------------------------------------
// All compute threads of all blocks.  `seq` counts the barriers of the step from 1; the counter in
// global memory starts the step at 0 (cleared by the host in stream order).
__device__ __forceinline__ bool grid_barrier(const TsStepArgs& a, const Smem& sm, int seq, int nb, int ct, const Abort& ab) {
  compute_sync();
  if (ct == 0) {
    bool ok = !ab.raised();
    if (ok) {
      if (a.trace != nullptr) a.trace[((size_t)blockIdx.x * (5 * a.L + 2) + (seq - 1)) * 8] = clock64();
      __threadfence();
      atomicAdd(a.ctrl, 1);
      const int target = seq * nb;
      const long long t0 = clock64();
      for (uint32_t i = 0;; ++i) {
        if (ld_acquire_gpu(a.ctrl) >= target) break;
        if ((i & 15u) == 15u) {
          if (ab.raised() || ld_acquire_gpu(a.ctrl + 1) != 0) {
            ok = false;
            break;
          }
          if (clock64() - t0 > 4 * WAIT_LIMIT_CYCLES) {
            ab.raise(40);
            ok = false;
            break;
          }
        }
      }
    }
    if (ok && a.trace != nullptr) a.trace[((size_t)blockIdx.x * (5 * a.L + 2) + (seq - 1)) * 8 + 1] = clock64();
    if (!ok) *ab.flag = 1;
    st_release_cta(sm.phase_open_(), ok ? seq : (1 << 30));          // a block that gives up lets its loader through
  }
  compute_sync();
  return !ab.raised();
}

// ---- the norm that opens a phase ------------------------------------------------------------------
// x[t, :] = w * bf16(r * rsqrt(mean(r^2) + eps)) for the step's tokens, r = resid[t, :] (32-bit
// statistics, turingserve/ops/reference.py:13-23), written as the B operand of the products that
// follow: k-block kb is a [16 tokens][64] tile of 128-byte rows with the 128-byte swizzle.
// Half a warp per token (eight tokens a pass).  The residual stream is 32-bit (the products that feed
// it add their parts into it with atomic adds); a row of up to 1,536 values stays in registers between
// the two passes (12 chunks of 8 values a lane; the host sends wider models down the other path).  The
// scale `ws` is in shared memory, 32-bit (the host converts the norms' scales once).  This code exists
// once in the kernel and is kept short: the phases of a layer run so seldom that what they execute
// comes from the instruction cache only if all of it fits there.
__device__ void norm_to_operand(const TsStepArgs& a, unsigned char* work, uint64_t* x_ready, const float* ws, int ct, long long* tr) {
  const int half = ct >> 4, hl = ct & 15;
  const int chunks = a.hidden / 8;                     // chunks of 8 values a row
  constexpr int KEEP = TS_STEP_MAX_HIDDEN / 8 / 16;
#pragma unroll 1
  for (int t0 = 0; t0 < a.T; t0 += 8) {
    const int t = t0 + half;
    const bool live = t < a.T;
    const float* row = a.resid + (size_t)t * a.hidden;
    float4 kept[KEEP][2];
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int c = hl + 16 * j;
      const bool in = live && c < chunks;
      kept[j][0] = in ? ldcg4(row + c * 8) : make_float4(0.f, 0.f, 0.f, 0.f);
      kept[j][1] = in ? ldcg4(row + c * 8 + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (t0 == 0)                                       // rows of tokens that do not exist are zero (while the loads travel)
#pragma unroll 1
      for (int tz = a.T + half; tz < BN; tz += 8)
#pragma unroll 1
        for (int c = hl; c < chunks; c += 16)
          *reinterpret_cast<uint4*>(work + (c >> 3) * X_BYTES + tz * 128 + (((c & 7) ^ (tz & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const float4 f = kept[j][q];
        ss += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
      }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);      // over the 16 lanes of the token
    const float rstd = rsqrtf(ss / (float)a.hidden + a.eps);
    if (tr != nullptr && ct == 0) tr[6] = clock64();
    if (live) {
#pragma unroll
      for (int j = 0; j < KEEP; ++j) {
        const int c = hl + 16 * j;
        if (c < chunks) {
          const float4 w0 = *reinterpret_cast<const float4*>(ws + c * 8), w1 = *reinterpret_cast<const float4*>(ws + c * 8 + 4);
          const float4 f0 = kept[j][0], f1 = kept[j][1];
          uint4 o;
          __nv_bfloat162* oe = reinterpret_cast<__nv_bfloat162*>(&o);
          oe[0] = __floats2bfloat162_rn(w0.x * round_to<bf16>(f0.x * rstd), w0.y * round_to<bf16>(f0.y * rstd));
          oe[1] = __floats2bfloat162_rn(w0.z * round_to<bf16>(f0.z * rstd), w0.w * round_to<bf16>(f0.w * rstd));
          oe[2] = __floats2bfloat162_rn(w1.x * round_to<bf16>(f1.x * rstd), w1.y * round_to<bf16>(f1.y * rstd));
          oe[3] = __floats2bfloat162_rn(w1.z * round_to<bf16>(f1.z * rstd), w1.w * round_to<bf16>(f1.w * rstd));
          *reinterpret_cast<uint4*>(work + (c >> 3) * X_BYTES + t * 128 + (((c & 7) ^ (t & 7)) << 4)) = o;
        }
      }
    }
  }
  if (tr != nullptr && ct == 0) tr[7] = clock64();
  fence_async_smem();                                  // ordinary stores, read by the tensor core
  mbar_arrive(x_ready);
}

// ---- accumulator read-back ----------------------------------------------------------------------
// Row r = quadrant * 32 + lane of accumulator `acc`: the 16 token columns.
__device__ __forceinline__ bool read_accumulator(const Smem& sm, uint32_t tmem_base, int v, int quad, float (&x)[BN],
                                                 const Abort& ab) {
  const int acc = v & 1;
  bool ok = mwait_now(&sm.acc_full_()[acc], (uint32_t)(v >> 1) & 1u, ab, 31);
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) return false;
  tc_fence_after();
  uint32_t raw[16];
  tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN), raw);
  tmem_wait_ld();
  tc_fence_before();
  mbar_arrive(&sm.acc_empty_()[acc]);
#pragma unroll
  for (int i = 0; i < BN; ++i) x[i] = __uint_as_float(raw[i]);
  return true;
}

// ---- decode attention for one (request, kv head, key split) -----------------------------------------
// The four compute warps on disjoint 16-key slices of every 64-key tile (as ts_attention_decode).
// Tiles of 64 keys of this block's attention unit (windows are not taken by this kernel: the host
// sends windowed models down the other path).
__device__ __forceinline__ int attention_tiles(const TsStepArgs& a, const Smem& sm, int unit, KeyRange& kr) {
  kr = key_range(a, unit, sm.seq_()[unit / (a.KVH * a.attn_splits)], 0);
  return kr.k_end > kr.k_begin ? (kr.k_end - kr.k_begin + ATT_TILE - 1) / ATT_TILE : 0;
}

// Keys and values arrive through the ring like weights (the producer warp copies them page by page, a
// stage of keys and a stage of values per tile of 64, rows of 256 bytes one after the other): tile t of
// the unit is in stages q0 + 2 t and q0 + 2 t + 1 of the block's sequence.  Returns false when a wait ran out.
__device__ bool attention_unit(const TsStepArgs& a, const TsStepLayer& ly, const Smem& sm, int unit, int ct, int seq1, int q0,
                               const Abort& ab) {
  constexpr int KS = D / 16, NT = D / 8;
  const int NS = a.attn_splits, NST = sm.nst;
  const int H = a.H, KVH = a.KVH, G = H / KVH, page = a.page;
  const int lane = ct & 31, warp = ct >> 5;
  KeyRange kr;
  const int n_tiles = attention_tiles(a, sm, unit, kr);
  const int b = kr.b, kvh = kr.kvh, split = kr.split, k_begin = kr.k_begin, k_end = kr.k_end;
  unsigned char* work = sm.work_();
  volatile int* flag = sm.flag_();
  // The q/k/v product left 32-bit sums (all its parts added up) in a.qkv: bias, rounding to bfloat16
  // and rotation happen here, where they are used.  The group's G query heads go to shared memory as
  // the A operand's rows; the block whose share ends at the new token also makes that token's key and
  // value, writes them into the cache and into its place in the last tile.
  const int N = (H + 2 * KVH) * D;
  const int seq_len = sm.seq_()[b];
  const bool has_new = n_tiles > 0 && k_end == seq_len;
  const int new_tile = has_new ? (seq_len - 1 - k_begin) / ATT_TILE : -1;
  const int new_key = has_new ? (seq_len - 1 - k_begin) % ATT_TILE : 0;
  bf16* q_s = reinterpret_cast<bf16*>(sm.ex_());                       // [16][D]: rows >= G zero
  bf16* kv_new = q_s + 16 * D;                                         // [2][D]
  {
    const float* acc = a.qkv + (size_t)b * N;
    const bf16* bias = reinterpret_cast<const bf16*>(ly.qkv_bias);
    const int pos = sm.pos_()[b];
    const int items = (G + (has_new ? 2 : 0)) * 64;                   // pairs (p, p + 64) of the group's q heads, then k, then v
    const bool rope = ly.cos_t != nullptr;
#pragma unroll 1
    for (int base = 0; base < items; base += 4 * CT) {                // four pairs a thread, all their loads in flight together
      float x1[4], x2[4], cs[4], sn[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = base + i * CT + ct;
        const bool live = idx < items;
        const int hh = idx >> 6, p = idx & 63;
        const int head = hh < G ? kvh * G + hh : (hh == G ? H + kvh : H + KVH + kvh);
        x1[i] = live ? __ldcg(acc + head * D + p) : 0.f;
        x2[i] = live ? __ldcg(acc + head * D + p + 64) : 0.f;
        if (live && bias != nullptr) {
          x1[i] += to_f(bias[head * D + p]);
          x2[i] += to_f(bias[head * D + p + 64]);
        }
        const bool rot = live && rope && hh <= G;
        cs[i] = rot ? ly.cos_t[(size_t)pos * 64 + p] : 1.f;
        sn[i] = rot ? ly.sin_t[(size_t)pos * 64 + p] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = base + i * CT + ct;
        if (idx >= items) continue;
        const int hh = idx >> 6, p = idx & 63;
        const float v1 = round_to<bf16>(x1[i]), v2 = round_to<bf16>(x2[i]);
        float o1 = v1, o2 = v2;
        if (rope && hh <= G) {
          const float c1 = round_to<bf16>(cs[i]), s1 = round_to<bf16>(sn[i]);
          o1 = v1 * c1 - v2 * s1;
          o2 = v2 * c1 + v1 * s1;
        }
        bf16* dst = hh < G ? q_s + hh * D : kv_new + (hh - G) * D;
        dst[p] = __float2bfloat16_rn(o1);
        dst[p + 64] = __float2bfloat16_rn(o2);
      }
    }
    for (int idx = ct; idx < (16 - G) * (D / 8); idx += CT)            // rows of heads that do not exist
      reinterpret_cast<uint4*>(q_s + G * D)[idx] = make_uint4(0u, 0u, 0u, 0u);
  }
  compute_sync();
  if (has_new) {                                                        // the new key and value into the cache
    const int slot = sm.slot_()[ly.group * BN + b];
    if (slot >= 0 && ct < 2 * (D / 8)) {
      const int which = ct / (D / 8), c = ct % (D / 8);
      bf16* dst = reinterpret_cast<bf16*>(which == 0 ? ly.k_cache : ly.v_cache) +
                  (((size_t)(slot / page) * KVH + kvh) * page + (size_t)(slot % page)) * D;
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(kv_new + which * D)[c];
    }
  }
  mark(a, seq1, 2, ct);
  unsigned qf[KS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, kc = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int k = ks * 16 + kc;
      qf[ks][0] = *reinterpret_cast<const unsigned*>(q_s + r0 * D + k);
      qf[ks][1] = *reinterpret_cast<const unsigned*>(q_s + r1 * D + k);
      qf[ks][2] = *reinterpret_cast<const unsigned*>(q_s + r0 * D + k + 8);
      qf[ks][3] = *reinterpret_cast<const unsigned*>(q_s + r1 * D + k + 8);
    }
  }
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sc = a.scale * LOG2E;

  bool ok = true;
#pragma unroll 1
  for (int t = 0; t < n_tiles; ++t) {
    const int qk = q0 + 2 * t, qv = qk + 1;
    const int sk = qk % NST, sv = qv % NST;
    ok = mwait_now(&sm.full_()[sk], (uint32_t)(qk / NST) & 1u, ab, 61) && mwait_now(&sm.full_()[sv], (uint32_t)(qv / NST) & 1u, ab, 62);
    ok = compute_all(ok);
    if (!ok) return false;
    unsigned char* ks_ = sm.ring_() + (size_t)sk * STAGE_BYTES;
    unsigned char* vs_ = sm.ring_() + (size_t)sv * STAGE_BYTES;
    if (t == new_tile) {                               // the new token's key and value take their place in the tile
      if (ct < 2 * (D / 8)) {
        const int which = ct / (D / 8), c = ct % (D / 8);
        *reinterpret_cast<uint4*>((which == 0 ? ks_ : vs_) + new_key * (D * 2) + c * 16) = reinterpret_cast<const uint4*>(kv_new + which * D)[c];
      }
      compute_sync();
    }
    const int rows_here = min(ATT_TILE, k_end - (k_begin + t * ATT_TILE));
    if (rows_here < ATT_TILE) {
      // Value rows past the unit's last key were not copied: their probabilities are exactly zero, and
      // zero times whatever the stage held before must stay zero.
      for (int idx = ct; idx < (ATT_TILE - rows_here) * (D / 8); idx += CT)
        *reinterpret_cast<uint4*>(vs_ + (size_t)rows_here * (D * 2) + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
      compute_sync();
    }
    const int key0 = warp * 16;
    const int j_base = k_begin + t * ATT_TILE + key0;
    if (j_base < k_end) {
      float s_acc[2][4] = {};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int mat = lane >> 3, r = lane & 7;
        const int key = key0 + (mat >> 1) * 8 + r;
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks_ + key * (D * 2) + (ks * 2 + (mat & 1)) * 16);
        mma_bf16(s_acc[0], qf[ks], b0, b1);
        mma_bf16(s_acc[1], qf[ks], b2, b3);
      }
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
        const float m_new = fmaxf(m_run[r], mx[r]);
        corr[r] = exp2f(m_run[r] - m_new);
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
      unsigned pf[4];
      pf[0] = pack_bf16(p[0][0], p[0][1]);
      pf[1] = pack_bf16(p[0][2], p[0][3]);
      pf[2] = pack_bf16(p[1][0], p[1][1]);
      pf[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
      for (int i = 0; i < NT; i += 2) {
        const int mat = lane >> 3, r = lane & 7;
        const int key = key0 + (mat & 1) * 8 + r;
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + key * (D * 2) + (i + (mat >> 1)) * 16);
        mma_bf16(o[i], pf, b0, b1);
        mma_bf16(o[i + 1], pf, b2, b3);
      }
    }
    if (rows_here < ATT_TILE || t == new_tile) fence_async_smem();      // ordinary stores above, before the stage is refilled by a copy
    compute_sync();                                    // every warp is done with the two stages
    if (ct == 0) {
      mbar_arrive(&sm.empty_()[sk]);
      mbar_arrive(&sm.empty_()[sv]);
    }
  }
  compute_sync();
  mark(a, seq1, 3, ct);

  // merge the four warps' states (the stage buffers are free now)
  float* m_s = reinterpret_cast<float*>(work);
  float* l_s = m_s + 4 * 16;
  float* o_s = l_s + 4 * 16;                                       // [4][16][D]
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
      float* x = o_s + ((size_t)warp * 16 + r0) * D + d;
      float* y = o_s + ((size_t)warp * 16 + r1) * D + d;
      x[0] = o[i][0];
      x[1] = o[i][1];
      y[0] = o[i][2];
      y[1] = o[i][3];
    }
  }
  compute_sync();
  float* f_s = o_s + 4 * 16 * D;                                   // [4][16]
  float* M_s = f_s + 4 * 16;
  float* L_s = M_s + 16;
  if (ct < 4 * G) {
    const int v = ct / G, g = ct % G;
    float M = -INFINITY;
#pragma unroll
    for (int u = 0; u < 4; ++u) M = fmaxf(M, m_s[u * 16 + g]);
    const float mv = m_s[v * 16 + g];
    f_s[v * 16 + g] = (mv == -INFINITY) ? 0.f : exp2f(mv - M);
    if (v == 0) {
      float L = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float mu = m_s[u * 16 + g];
        if (mu != -INFINITY) L += l_s[u * 16 + g] * exp2f(mu - M);
      }
      M_s[g] = M;
      L_s[g] = L;
    }
  }
  compute_sync();
  float* part_acc = a.attn_part;
  float* part_ml = a.attn_part + (size_t)a.T * H * NS * D;
  for (int idx = ct; idx < G * (D / 4); idx += CT) {
    const int g = idx / (D / 4), d = (idx % (D / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const float f = f_s[v * 16 + g];
      const float4 x = *reinterpret_cast<const float4*>(o_s + ((size_t)v * 16 + g) * D + d);
      acc.x += x.x * f; acc.y += x.y * f; acc.z += x.z * f; acc.w += x.w * f;
    }
    const int h = kvh * G + g;
    if (NS == 1) {
      const float L = L_s[g], inv = L > 0.f ? 1.f / L : 0.f;
      bf16* op = reinterpret_cast<bf16*>(a.attn) + (size_t)b * H * D + (size_t)h * D + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    } else {
      const size_t pi = ((size_t)b * H + h) * NS + split;
      *reinterpret_cast<float4*>(part_acc + pi * D + d) = acc;
      if (d == 0) *reinterpret_cast<float2*>(part_ml + pi * 2) = make_float2(M_s[g], L_s[g]);
    }
  }
  if (NS == 1) {
    compute_sync();
    return true;
  }
  compute_sync();                                      // every thread's stores precede thread 0's fence
  if (ct == 0) {
    __threadfence();
    int* counter = a.tickets + TS_STEP_TICKETS_ATTN + b * KVH + kvh;
    const int ticket = atomicAdd(counter, 1);
    const int last = ticket == NS - 1;
    if (last) {
      *counter = 0;
      __threadfence();                                 // the other splits' states are visible from here on
    }
    *flag = last;
  }
  compute_sync();
  mark(a, seq1, 4, ct);
  if (*flag == 0) {
    compute_sync();
    return true;
  }
  float* w_s = reinterpret_cast<float*>(work);                  // [G][NS]
  float* m_all = w_s + G * NS;
  float* l_all = m_all + G * NS;
  const int pieces = G * (D / 4);                                  // 16-byte pieces of the output
#pragma unroll 1
  for (int idx = ct; idx < G * NS; idx += CT) {
    const int g = idx / NS, s2 = idx % NS;
    const size_t pi = ((size_t)b * H + kvh * G + g) * NS + s2;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + pi * 2));
    m_all[idx] = ml.x;
    l_all[idx] = ml.y;
  }
  compute_sync();
#pragma unroll 1
  for (int idx = ct; idx < G * NS; idx += CT) {
    const int g = idx / NS;
    float M = -INFINITY, L = 0.f;
#pragma unroll 1
    for (int s2 = 0; s2 < NS; ++s2) M = fmaxf(M, m_all[g * NS + s2]);
    if (M > -INFINITY)
#pragma unroll 1
      for (int s2 = 0; s2 < NS; ++s2) {
        const float ms = m_all[g * NS + s2];
        if (ms != -INFINITY) L += l_all[g * NS + s2] * exp2f(ms - M);
      }
    const float mi = m_all[idx];
    w_s[idx] = (L > 0.f && mi != -INFINITY) ? exp2f(mi - M) / L : 0.f;
  }
  compute_sync();
#pragma unroll 1
  for (int idx = ct; idx < pieces; idx += CT) {
    const int g = idx / (D / 4), d = (idx % (D / 4)) * 4;
    const int h = kvh * G + g;
    const float* src = part_acc + (((size_t)b * H + h) * NS) * D + d;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int s0 = 0; s0 < NS; s0 += 16) {                           // sixteen splits' pieces in flight together
      float4 v[16];
#pragma unroll
      for (int s2 = 0; s2 < 16; ++s2) v[s2] = s0 + s2 < NS ? ldcg4(src + (size_t)(s0 + s2) * D) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s2 = 0; s2 < 16; ++s2) {
        const float w = s0 + s2 < NS ? w_s[g * NS + s0 + s2] : 0.f;
        acc.x += v[s2].x * w; acc.y += v[s2].y * w; acc.z += v[s2].z * w; acc.w += v[s2].w * w;
      }
    }
    bf16* op = reinterpret_cast<bf16*>(a.attn) + (size_t)b * H * D + (size_t)h * D + d;
    *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x, acc.y);
    *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z, acc.w);
  }
  compute_sync();
  mark(a, seq1, 5, ct);
  return true;
}

// ---- the kernel -----------------------------------------------------------------------------------
__global__ void __launch_bounds__(NUM_THREADS, 1) decode_step_kernel(const __grid_constant__ TsStepArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int NST = a.stages;
  const Smem sm{base, a.stages, a.work_bytes};

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, nb = gridDim.x;
  const Abort ab{sm.abort_flag_(), a.status, a.ctrl + 1};

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&sm.full_()[s], FULL_COUNT);
      mbar_init(&sm.empty_()[s], 1);
    }
    mbar_init(&sm.acc_full_()[0], 1);
    mbar_init(&sm.acc_full_()[1], 1);
    mbar_init(&sm.acc_empty_()[0], CT);
    mbar_init(&sm.acc_empty_()[1], CT);
    mbar_init(sm.x_ready_(), CT);
    *sm.abort_flag_() = 0;
    *sm.w_issued_() = 0;
    *sm.phase_open_() = 0;
    *sm.flag_() = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the activation part of every stage starts as zeros: rows of tokens that do not exist are never written
  for (int i = threadIdx.x; i < NST * (X_BYTES / 16); i += NUM_THREADS)
    *reinterpret_cast<uint4*>(sm.ring_() + (size_t)(i / (X_BYTES / 16)) * STAGE_BYTES + W_BYTES + (i % (X_BYTES / 16)) * 16) =
        make_uint4(0u, 0u, 0u, 0u);
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sm.tmem_slot_())), "r"(32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_slot_();

  if (warp == 0) {
    // ---- weight producer ------------------------------------------------------------------------
    if (lane == 0) {
      Walker w, ahead;
      w.start();
      ahead.start();
      Unit u, ua;
      int q = 0;
      int a_kb = 0;                                   // the look-ahead cursor: k-block within `ua`
      bool a_more = ahead.next(a, cta, nb, ua);
      if (a_more) a_kb = ua.kb0;
      int a_q = 0;                                    // k-blocks the look-ahead has asked L2 for
      bool ok = true;
      bool staged = false;
      while (ok && w.next(a, cta, nb, u)) {
        if (u.kind == K_ATTN) {
          // This block's share of the keys and values of layer u.layer, a stage of 64 key rows and a
          // stage of 64 value rows per tile, copied page by page (rows of one page and kv head lie one
          // after the other in the cache).  Rows past the unit's last key are not copied.
          if (!staged) {                               // the step's lengths and pages are in shared memory after the first barrier
            ok = wait_shared_ge(sm.phase_open_(), 1, ab, 12);
            staged = true;
            if (!ok) break;
          }
          KeyRange kr;
          const int n_tiles = attention_tiles(a, sm, cta, kr);
          const TsStepLayer* ly = a.layers + u.layer;
          const unsigned char* caches[2] = {reinterpret_cast<const unsigned char*>(ly->k_cache), reinterpret_cast<const unsigned char*>(ly->v_cache)};
          const int group = ly->group;
          const int page = a.page, SL = page < ATT_TILE ? page : ATT_TILE;     // key rows one copy brings
          const bool in_smem = kr.n_pages <= PAGES_S;
          const int* table = a.block_tables[group] + (size_t)kr.b * a.table_width[group];
          for (int t = 0; t < n_tiles && ok; ++t)
            for (int kv = 0; kv < 2 && ok; ++kv, ++q) {
              const int s = q % NST;
              if (q >= NST) ok = mwait_now(&sm.empty_()[s], (uint32_t)((q / NST) - 1) & 1u, ab, 13);
              if (!ok) break;
              const int j0 = kr.k_begin + t * ATT_TILE;
              const int rows = min(ATT_TILE, kr.k_end - j0);
              mbar_expect_tx(&sm.full_()[s], (uint32_t)rows * D * 2);
              unsigned char* dst = sm.ring_() + (size_t)s * STAGE_BYTES;
              for (int r0 = 0; r0 < rows; r0 += SL) {
                const int j = j0 + r0, lp = j / page;
                const int pg = in_smem ? sm.pages_()[group * PAGES_S + lp - kr.page_first] : table[lp];
                const int n = min(SL, rows - r0);
                if (pg < 0 || pg >= a.num_pages || n < 1 || n > ATT_TILE || lp < kr.page_first || (in_smem && lp - kr.page_first >= PAGES_S) ||
                    r0 + n > ATT_TILE || j - lp * page + n > page) {          // a copy that would leave the cache or the stage: refuse, say so
                  ab.raise(70);
                  ok = false;
                  break;
                }
                bulk_load(dst + (size_t)r0 * D * 2, caches[kv] + (((size_t)pg * a.KVH + kr.kvh) * page + (size_t)(j - lp * page)) * D * 2,
                          (uint32_t)n * D * 2, &sm.full_()[s]);
              }
              mbar_arrive_n(&sm.full_()[s], 32);
            }
          continue;
        }
        const CUtensorMap* map = map_of(a, u.kind, u.layer);
        const bool streamed = u.kind == K_O || u.kind == K_DOWN;
        for (int kb = u.kb0; kb < u.kb1 && ok; ++kb, ++q) {
          // keep L2 `lookahead` k-blocks ahead of the ring
          while (a_more && a_q < q + NST + a.lookahead) {
            if (a_q >= q + NST)
              asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map_of(a, ua.kind, ua.layer)),
                           "r"(a_kb * BK), "r"(ua.tile * BM) : "memory");
            ++a_q;
            if (++a_kb >= ua.kb1) {
              do a_more = ahead.next(a, cta, nb, ua);
              while (a_more && ua.kind == K_ATTN);
              if (a_more) a_kb = ua.kb0;
            }
          }
          const int s = q % NST;
          if (q >= NST) ok = mwait_now(&sm.empty_()[s], (uint32_t)((q / NST) - 1) & 1u, ab, 11);
          if (!ok) break;
          mbar_expect_tx(&sm.full_()[s], W_BYTES);
          tma_load_2d(sm.ring_() + (size_t)s * STAGE_BYTES, map, kb * BK, u.tile * BM, &sm.full_()[s]);
          if (streamed) st_release_cta(sm.w_issued_(), q + 1);        // the loader adds this k-block's activations
          else mbar_arrive_n(&sm.full_()[s], 32);                     // the norm's output is the operand: nothing to add
        }
      }
      if (!ok) {
        st_release_cta(sm.w_issued_(), 1 << 30);         // the loader must not wait for weights that will not come
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) {}            // copies already asked for land in shared memory before the block leaves
      }
    }
  } else if (warp == 1) {
    // ---- tensor-core issue ----------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      Walker w;
      w.start();
      Unit u;
      int q = 0, v = 0, xr = 0, cur_phase = -1;
      bool ok = true;
      while (ok && w.next(a, cta, nb, u)) {
        if (u.kind == K_ATTN) {
          // The compute warps use these stages.  This thread still waits for each of them to fill: a
          // parity wait tells a phase only from its neighbours, so a waiter must never fall two uses
          // of a stage behind (with as many key/value stages as the ring is long, the next weights
          // land in the very stage the first keys are still on their way to).
          ok = wait_shared_ge(sm.phase_open_(), 1, ab, 24);
          KeyRange kr;
          const int n = ok ? 2 * attention_tiles(a, sm, cta, kr) : 0;
          for (int i = 0; i < n && ok; ++i, ++q) ok = mwait(&sm.full_()[q % NST], (uint32_t)(q / NST) & 1u, ab, 25);
          continue;
        }
        const bool from_norm = u.kind == K_QKV || u.kind == K_GU || u.kind == K_HEAD;
        const int phase = u.layer * 4 + u.kind;
        if (from_norm && phase != cur_phase) {          // this phase's norm output must be in place
          ok = mwait_now(sm.x_ready_(), (uint32_t)xr & 1u, ab, 21);
          ++xr;
          if (!ok) break;
        }
        cur_phase = phase;
        const int acc = v & 1;
        if (v >= 2) ok = mwait_now(&sm.acc_empty_()[acc], (uint32_t)((v >> 1) - 1) & 1u, ab, 22);
        if (!ok) break;
        tc_fence_after();
        for (int kb = u.kb0; kb < u.kb1; ++kb, ++q) {
          const int s = q % NST;
          ok = mwait_now(&sm.full_()[s], (uint32_t)(q / NST) & 1u, ab, 23);
          if (!ok) break;
          tc_fence_after();
          if (!from_norm) fence_async_smem();           // activations arrived by cp.async, an ordinary-proxy write
          const uint64_t da = smem_desc(smem_u32(sm.ring_() + (size_t)s * STAGE_BYTES));
          const uint64_t db = smem_desc(smem_u32(from_norm ? sm.work_() + (size_t)kb * X_BYTES
                                                            : sm.ring_() + (size_t)s * STAGE_BYTES + W_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(tmem_base + (uint32_t)(acc * BN), da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16),
                 idesc, (kb > u.kb0 || k > 0) ? 1u : 0u);
          umma_commit(&sm.empty_()[s]);
        }
        if (!ok) break;
        umma_commit(&sm.acc_full_()[acc]);
        ++v;
      }
    }
  } else if (warp == 2) {
    // ---- activation loader ----------------------------------------------------------------------
    Walker w;
    w.start();
    Unit u;
    int q = 0, l2_layer = -1;
    bool ok = true;
    while (ok && w.next(a, cta, nb, u)) {
      if (a.l2_ahead && u.layer != l2_layer && u.layer < a.L) {
        // A layer begins (barrier 5 l + 1 is passed): its q/k/v, attention and output phases move little
        // memory, so this block's gate/up and down weights set out for L2 now and are read from there
        // when their turn comes.
        l2_layer = u.layer;
        ok = warp_wait_shared_ge(sm.phase_open_(), 5 * u.layer + 1, ab, 53, lane) && !ab.raised();
        if (!ok) break;
        for (int kind = K_GU; kind <= K_DOWN; ++kind) {
          const TsStepShape& sh = a.shape[kind];
          const CUtensorMap* map = map_of(a, kind, u.layer);
          for (int un = (cta + sh.rot) % nb; un < sh.R * sh.S; un += nb) {
            const int tile = un / sh.S, kb0 = (un % sh.S) * sh.per, kb1 = min(sh.KB, kb0 + sh.per);
            for (int kb = kb0 + lane; kb < kb1; kb += 32)
              asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(kb * BK), "r"(tile * BM) : "memory");
          }
        }
      }
      if (u.kind == K_ATTN) {
        ok = warp_wait_shared_ge(sm.phase_open_(), 1, ab, 54, lane) && !ab.raised();
        KeyRange kr;
        if (ok) q += 2 * attention_tiles(a, sm, cta, kr);
        continue;
      }
      const bool stream = u.kind == K_O || u.kind == K_DOWN;
      if (!stream) {                                   // the producer arrives for this warp's lanes
        q += u.kb1 - u.kb0;
        continue;
      }
      const bf16* src = reinterpret_cast<const bf16*>(u.kind == K_O ? a.attn : a.act);
      const int K = u.kind == K_O ? a.H * D : a.inter;
      // the output projection of layer l opens after barrier 5 l + 3, the down projection after 5 l + 5
      ok = warp_wait_shared_ge(sm.phase_open_(), 5 * u.layer + (u.kind == K_O ? 3 : 5), ab, 51, lane) && !ab.raised();
      if (!ok) break;
      for (int kb = u.kb0; kb < u.kb1; ++kb, ++q) {
        const int s = q % NST;
        ok = warp_wait_shared_ge(sm.w_issued_(), q + 1, ab, 52, lane) && !ab.raised();
        if (!ok) break;
        unsigned char* xs = sm.ring_() + (size_t)s * STAGE_BYTES + W_BYTES;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = lane + 32 * j, t = i >> 3, c = i & 7;
          if (t < a.T) cp_async_16(xs + t * 128 + ((c ^ (t & 7)) << 4), src + (size_t)t * K + kb * BK + c * 8, true);
        }
        cp_async_arrive_noinc(&sm.full_()[s]);
      }
    }
    cp_async_wait_all();
  } else {
    // ---- compute warps ----------------------------------------------------------------------------
    const int ct = threadIdx.x - CW0 * 32;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    int v = 0, seq = 0, q = 0;                         // q: stages of the ring this block's units have taken so far
    bool ok = true;
    if (ct < (int)sizeof(TsStepLayer) / 16)            // the first layer's table entry
      cp_async_16(reinterpret_cast<unsigned char*>(sm.layer_(0)) + 16 * ct, reinterpret_cast<const unsigned char*>(a.layers) + 16 * ct, true);
    {                                                  // the first norm's scale: a weight, it need not wait for anything
      const int sb = a.hidden * 4;
      unsigned char* dst = sm.scale_(0, sb);
      for (int i = ct * 16; i < sb; i += CT * 16) cp_async_16(dst + i, reinterpret_cast<const unsigned char*>(a.layers[0].ln1_w) + i, true);
    }
    pdl_wait();                                        // the step's ids, positions and tables are in place
    // What the step's index arrays say about this block's work goes to shared memory once: positions,
    // context lengths, cache slots, and the pages of this block's share of the keys (the same in every
    // layer of a cache group).
    if (ct < BN) {
      sm.pos_()[ct] = ct < a.T ? a.positions[ct] : 0;
      sm.seq_()[ct] = ct < a.T ? a.seq_lens[ct] : 0;
      for (int g = 0; g < a.num_groups; ++g) sm.slot_()[g * BN + ct] = ct < a.T ? a.slot_mapping[g][ct] : -1;
    }
    compute_sync();
    if (cta < a.T * a.KVH * a.attn_splits)
      for (int g = 0; g < a.num_groups; ++g) {
        const KeyRange kr = key_range(a, cta, sm.seq_()[cta / (a.KVH * a.attn_splits)], a.group_window[g]);
        if (kr.n_pages <= PAGES_S) {
          const int* table = a.block_tables[g] + (size_t)kr.b * a.table_width[g];
          for (int i = ct; i < kr.n_pages; i += CT) sm.pages_()[g * PAGES_S + i] = table[kr.page_first + i];
        }
      }
    // embedding rows into the residual stream (32-bit from here on); the q/k/v accumulator starts at zero
    if (cta < a.T) {
      const int id = a.ids[cta];
      const bf16* src = reinterpret_cast<const bf16*>(a.embedding) + (size_t)id * a.hidden;
      float* dst = a.resid + (size_t)cta * a.hidden;
      for (int i = ct; i < a.hidden; i += CT) dst[i] = to_f(src[i]);
    }
    {
      const int total = a.T * (a.H + 2 * a.KVH) * D;
      for (int i = cta * CT + ct; i < total; i += nb * CT) a.qkv[i] = 0.f;
    }
    ok = grid_barrier(a, sm, ++seq, nb, ct, ab);

    // The phases of the step, one loop so that every piece of code exists once: phase p of layer p / 5
    // is 0 q/k/v, 1 attention, 2 output projection, 3 gate/up, 4 down; after the last layer, the head.
    const int scale_bytes = a.hidden * 4;
    const int n_phases = 5 * a.L + 1;
#pragma unroll 1
    for (int p = 0; p < n_phases && ok; ++p) {
      const int layer = p / 5, k = p % 5;
      const bool head = p == 5 * a.L;
      const int kind = head ? K_HEAD : (k == 0 ? K_QKV : k == 2 ? K_O : k == 3 ? K_GU : k == 4 ? K_DOWN : -1);
      // the table entries of this layer and of the next one sit in shared memory (slots layer & 1)
      const TsStepLayer& ly = *sm.layer_(layer & 1);
      const TsStepLayer& next_ly = *sm.layer_((layer + 1) & 1);
      if (k == 0 && layer + 1 < a.L && ct < (int)sizeof(TsStepLayer) / 16)      // the next entry sets out (the slot's old one, layer - 1, is done)
        cp_async_16(reinterpret_cast<unsigned char*>(sm.layer_((layer + 1) & 1)) + 16 * ct,
                    reinterpret_cast<const unsigned char*>(a.layers + layer + 1) + 16 * ct, true);
      if (kind == K_QKV || kind == K_GU || kind == K_HEAD) {
        // Norm n of the step (0, 1: layer 0's two; ...; 2 L: the final one) finds its scale in shared
        // memory slot n & 1, brought there with cp.async while the phases before it ran.
        const int n = head ? 2 * a.L : 2 * layer + (kind == K_GU ? 1 : 0);
        cp_async_wait_all();
        compute_sync();                                // scale n is in its slot; everyone is done with slot (n + 1) & 1
        if (has_units(a, kind, cta, nb)) {
          long long* tr = a.trace == nullptr ? nullptr : a.trace + ((size_t)blockIdx.x * (5 * a.L + 2) + seq) * 8;
          norm_to_operand(a, sm.work_(), sm.x_ready_(), reinterpret_cast<const float*>(sm.scale_(n & 1, scale_bytes)), ct, tr);
          mark(a, seq + 1, 2, ct);
        }
        if (n + 1 <= 2 * a.L) {                        // the next norm's scale sets out now
          const int m = n + 1;
          const void* w = m == 2 * a.L ? a.final_norm_w : (m & 1 ? ly.ln2_w : next_ly.ln1_w);
          unsigned char* dst = sm.scale_(m & 1, scale_bytes);
          for (int i = ct * 16; i < scale_bytes; i += CT * 16) cp_async_16(dst + i, reinterpret_cast<const unsigned char*>(w) + i, true);
        }
      }
      if (kind == K_O) {
        // the q/k/v accumulator has been read (attention is over): zero again for the next layer
        const int total = a.T * (a.H + 2 * a.KVH) * D;
        for (int i = cta * CT + ct; i < total; i += nb * CT) a.qkv[i] = 0.f;
      }
      if (kind < 0) {
        if (cta < a.T * a.KVH * a.attn_splits) {
          KeyRange kr;
          const int n_tiles = attention_tiles(a, sm, cta, kr);
          ok = attention_unit(a, ly, sm, cta, ct, seq + 1, q, ab);
          q += 2 * n_tiles;
        }
      } else {
        const TsStepShape& sh = a.shape[kind];
        #pragma unroll 1
        for (int un = (cta + sh.rot) % nb; ok && un < sh.R * sh.S; un += nb) {
          const Unit u{kind, layer, un / sh.S, un % sh.S, 0, 0};
          q += min(sh.KB, (u.part + 1) * sh.per) - u.part * sh.per;
          float x[BN];
          ok = compute_all(read_accumulator(sm, tmem_base, v, quad, x, ab));
          ++v;
          mark(a, seq + 1, 3, ct);
          if (!ok) break;
          if (kind == K_GU) {
            // SiLU * mul: rows 0..63 of a tile are gates, 64..127 their ups
            if (quad >= 2) {
#pragma unroll
              for (int c = 0; c < BN; ++c) sm.ex_()[(r - 64) * BN + c] = x[c];
            }
            compute_sync();
            if (quad < 2) {
              const int n = u.tile * 64 + r;
              if (n < a.inter)
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                  if (c >= a.T) break;
                  const float g = round_to<bf16>(x[c]);
                  const float up = round_to<bf16>(sm.ex_()[r * BN + c]);
                  const float sl = round_to<bf16>(silu_for<bf16>(g));
                  reinterpret_cast<bf16*>(a.act)[(size_t)c * a.inter + n] = __float2bfloat16_rn(sl * up);
                }
            }
            compute_sync();
          } else if (kind == K_HEAD) {
            const int n = u.tile * BM + r;
            if (n < a.V)
#pragma unroll
              for (int c = 0; c < BN; ++c)
                if (c < a.T) a.logits[(size_t)c * a.V + n] = x[c];
          } else {
            // A part of a product that is split over K: its sums are added into the 32-bit q/k/v
            // accumulator or straight into the residual stream (red.global.add: nobody waits for the
            // result, no ticket, no second pass; the order of the additions is not fixed).
            const int n = u.tile * BM + r;
            float* dst = kind == K_QKV ? a.qkv + n : a.resid + n;
            const int width = kind == K_QKV ? (a.H + 2 * a.KVH) * D : a.hidden;
            if (n < width)
#pragma unroll
              for (int c = 0; c < BN; ++c)
                if (c < a.T) atomicAdd(dst + (size_t)c * width, x[c]);
          }
          mark(a, seq + 1, 5, ct);
        }
      }
      if (!head) ok = grid_barrier(a, sm, ++seq, nb, ct, ab) && ok;
    }
  }
  if (*sm.abort_flag_() != 0) {
    // A block that gives up may still have copies on their way into its shared memory, and products
    // in flight: it stays for a millisecond (far longer than either takes) before it leaves.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32) : "memory");
  }
}

__device__ int g_step_status = 0;

int* step_status_word() {
  static int* p = nullptr;
  if (p == nullptr && cudaGetSymbolAddress((void**)&p, g_step_status) != cudaSuccess) p = nullptr;
  return p;
}

}  // namespace

int* ts_step_status_word() { return step_status_word(); }

TS_API int ts_decode_step_status() {
  int* p = step_status_word();
  int v = -1;
  if (p != nullptr) cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

// Encodes the tensor map of one weight matrix [rows, K] (bfloat16, row-major) as the kernel reads it:
// boxes of 128 rows x 64 columns, 128-byte swizzle, zeros outside.  `out` is 128 bytes of HOST memory
// (the caller copies the maps of all matrices to the device in one piece).
TS_API int ts_decode_step_encode_map(void* out, const void* weights, int rows, int K) {
  if (((uintptr_t)weights & 15) || K % 8) TS_REFUSE(TS_ERR_ALIGN, "ts_decode_step_encode_map: weights must be 16-byte aligned, K a multiple of 8");
  CUtensorMap m;
  if (!tc::tensor_map(&m, weights, rows, K, BM)) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_decode_step_encode_map: cuTensorMapEncodeTiled failed");
  memcpy(out, &m, sizeof(m));
  return 0;
}

TS_API int ts_decode_step_sizes(int* args_bytes, int* layer_bytes, int* map_bytes) {
  *args_bytes = (int)sizeof(TsStepArgs);
  *layer_bytes = (int)sizeof(TsStepLayer);
  *map_bytes = (int)sizeof(CUtensorMap);
  return 0;
}

// Shared memory the kernel needs for `stages` ring stages and a work area of `work_bytes`.
static size_t step_smem(int stages, int work_bytes, int hidden) {
  return 1024 + (size_t)stages * STAGE_BYTES + (size_t)work_bytes + EX_BYTES + (size_t)(2 * stages + 5) * 8 + 32 +
         (size_t)(2 * BN + TS_STEP_MAX_GROUPS * (BN + PAGES_S)) * 4 + 2 * sizeof(TsStepLayer) + 2 * (size_t)hidden * 4;
}

// The work area: the norm's output for `hidden` columns, or the attention's merge space.
TS_API int ts_decode_step_work_bytes(int hidden) {
  const int x = (hidden / BK) * X_BYTES;
  const int merge = 4 * (3 * 4 * 16 + 32 + 5 * 16 * D);
  int m = x > merge ? x : merge;
  return (m + 1023) / 1024 * 1024;
}

// The most ring stages that fit beside the work area (0: the shape does not fit at all).
TS_API int ts_decode_step_max_stages(int hidden) {
  int dev = 0, limit = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
  const int work = ts_decode_step_work_bytes(hidden);
  int st = 0;
  while (st < 16 && step_smem(st + 1, work, hidden) <= (size_t)limit) ++st;
  return st >= 3 ? st : 0;
}

// Blocks of the kernel that run at once on the current device (one per SM when the shape fits).
TS_API int ts_decode_step_blocks(int stages, int hidden) {
  int dev = 0, sms = 0, per = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  const size_t smem = step_smem(stages, ts_decode_step_work_bytes(hidden), hidden);
  if (cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, decode_step_kernel, NUM_THREADS, smem) != cudaSuccess || per < 1) {
    cudaGetLastError();
    return 0;
  }
  return sms;
}

// Runs one decode step.  `args` is a TsStepArgs in HOST memory, filled by the caller (see
// decode_step.h); its `status` is set here.  The control words (barrier counter, abort flag) are
// cleared in stream order before the launch.  The launch is cooperative where the driver allows it
// (all blocks are then guaranteed to be resident together, which the grid barriers need); where it
// does not (inside some stream captures), an ordinary launch of one block per SM is the same thing as
// long as nothing else occupies the device, and the barriers are bounded either way.
TS_API int ts_decode_step(const void* args_host, int blocks, int cooperative, void* stream) {
  TsStepArgs a;
  memcpy(&a, args_host, sizeof(a));
  if (a.T < 1 || a.T > BN) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_decode_step: %d tokens (1..%d)", a.T, BN);
  if (a.hidden > TS_STEP_MAX_HIDDEN || !a.norm_w_is_f32)
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_decode_step: hidden %d (at most %d), norm scales must be 32-bit", a.hidden, TS_STEP_MAX_HIDDEN);
  if (a.page < 1 || (ATT_TILE % a.page != 0 && a.page % ATT_TILE != 0))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_decode_step: pages of %d tokens (a divisor or a multiple of %d)", a.page, ATT_TILE);
  for (int g = 0; g < a.num_groups; ++g)
    if (a.group_window[g] > 0) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_decode_step: windowed attention is not taken by this kernel");
  if (a.hidden % BK || a.inter % BK || a.H % a.KVH || a.H / a.KVH > 16 || a.L < 1)
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_decode_step: hidden %d, inner %d, heads %d/%d are not taken by this kernel", a.hidden, a.inter, a.H, a.KVH);
  if (a.stages < 3 || a.work_bytes < ts_decode_step_work_bytes(a.hidden)) TS_REFUSE(TS_ERR_SHAPE, "ts_decode_step: stages %d, work area %d", a.stages, a.work_bytes);
  if (a.T * a.KVH * a.attn_splits > blocks || a.attn_splits < 1) TS_REFUSE(TS_ERR_SHAPE, "ts_decode_step: %d attention units on %d blocks", a.T * a.KVH * a.attn_splits, blocks);
  for (int k = 0; k < 5; ++k) {
    const TsStepShape& sh = a.shape[k];
    if (sh.R < 1 || sh.KB < 1 || sh.S < 1 || sh.per < 1 || sh.S * sh.per < sh.KB || (sh.S - 1) * sh.per >= sh.KB)
      TS_REFUSE(TS_ERR_SHAPE, "ts_decode_step: product %d is cut badly (R %d, KB %d, S %d, per %d)", k, sh.R, sh.KB, sh.S, sh.per);
    if ((k == K_GU || k == K_HEAD) && sh.S != 1) TS_REFUSE(TS_ERR_SHAPE, "ts_decode_step: product %d cannot be split over K", k);
    if (k != K_GU && k != K_HEAD && sh.R * sh.S > TS_STEP_MAX_UNITS) TS_REFUSE(TS_ERR_LIMIT, "ts_decode_step: product %d has too many units", k);
    if (k != K_GU && k != K_HEAD && sh.R > TS_STEP_TICKETS_EACH) TS_REFUSE(TS_ERR_LIMIT, "ts_decode_step: product %d has too many tiles", k);
  }
  if (a.T * a.KVH > TS_STEP_TICKETS_EACH) TS_REFUSE(TS_ERR_LIMIT, "ts_decode_step: too many (request, kv head) pairs");
  a.status = step_status_word();
  if (a.status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_decode_step: no status word");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = step_smem(a.stages, a.work_bytes, a.hidden);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_decode_step: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  cudaError_t e = cudaMemsetAsync(a.ctrl, 0, 2 * sizeof(int), s);
  if (e != cudaSuccess) TS_REFUSE((int)e, "ts_decode_step: clearing the control words: %s", cudaGetErrorString(e));
  // 0: cooperative, 1: ordinary; remembered once one of them has worked
  static int mode = 0;
  if (!cooperative && mode == 0) mode = 1;
  for (; mode < 2; ++mode) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (mode == 0) {
      attr[n].id = cudaLaunchAttributeCooperative;
      attr[n].val.cooperative = 1;
      ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    e = cudaLaunchKernelEx(&cfg, decode_step_kernel, a);
    if (e == cudaSuccess) return 0;
    cudaGetLastError();
  }
  mode = 0;
  ts_set_error("ts_decode_step: launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}
