// Paged grouped-query DECODE attention in bfloat16 (one new token per request) with key/value
// tiles brought in by TMA: the kernel the engine uses when pages are multiples of 16 tokens.
//
// Counterpart of the reference's split-K flash-decoding kernels
// (turingserve/ops/triton_decode_attention.py:101-163: partial (m, l, acc) per partition, then a
// reduce kernel; :60-95: the G query heads of a kv head share every key/value tile).  Semantics as
// turingserve/ops/reference.py:60-77,94-111 for q_len = 1.
//
// Work split: one block per (key split, kv head, request).  The request's keys are seen as tiles
// of 64 at absolute positions (tile i holds keys 64i .. 64i+63); the tiles that hold visible keys
// are dealt out evenly over the splits that get at least one, and the remaining splits leave at
// once.  Inside a block one producer warp issues TMA copies, ONE per box: a box is the keys AND the
// values of one page (or of 64 keys where pages are larger), all head columns, through a 4-D tensor
// map over both caches with the 128-byte swizzle; a copy costs the TMA unit about 100 cycles
// whatever its size, so fewer and larger ones matter.  The boxes go into a ring of stages
// (2..8; three by default, which lets two blocks share an SM) and min(4, stages) consumer warps each
// take WHOLE tiles (the tiles of stage s go to warp s % warps, so that a stage's barriers are waited
// on by one warp, phase after phase): a warp waits for its tile's mbarrier, computes S = Q K^T for 16 x 64 with
// mma.sync m16n8k16 (the G heads in the 16 rows), one online-softmax update per 64 keys, then
// O += P V, and hands the stage back.  No block-wide barrier and no per-thread address
// arithmetic in the loop.  The warps' states merge through shared memory; with several splits the
// block writes an unnormalised partial and the block that finishes last for a (request, kv head)
// merges them (a ticket counter: no second launch, nobody waits).  With 2 to 8 splits the blocks of
// a (request, kv head) are one thread-block cluster instead: the partial stays in shared memory and
// block r sums the 16-byte pieces r, r + n, ... of the output out of its peers' (two cluster
// barriers, which blocks that leave early take too).
//
// Before the wait for the preceding kernel the producer already fetches every box of its first
// stages except the one holding the new token's row: the step's index arrays come from the host
// and earlier rows of the cache from earlier steps, so no kernel of this step writes them.
#include "decode_tile.cuh"

namespace {

using namespace dec;

constexpr int CWARPS = 4;            // consumer warps at most: min(4, stages) of them, then the producer warp
constexpr int MAX_THREADS = (CWARPS + 1) * 32;
constexpr int MAX_STAGES = 8;
// The ticket's merge: up to MERGE_FLAT splits by one block; more in groups of MERGE_GROUP, then the groups.
constexpr int MERGE_FLAT = 32, MERGE_GROUP = 8, MERGE_GROUPS_MAX = 16;

__device__ int g_dec_status = 0;     // 0 = fine; otherwise the wait that ran out

struct DecArgs {
  bf16* out;
  float* part_acc;
  float* part_ml;
  const bf16* qkv;
  const int* block_tables;
  const int* q_start;
  const int* seq_lens;
  int table_width, H, KVH, page;
  float scale;
  int window, nsplit, stages, box_shift, v_first;
  int cluster;            // the splits of a (request, kv head) are one thread-block cluster (2..8 of them)
  int* counters;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(MAX_THREADS, 1)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const DecArgs a) {
  pdl_launch_dependents();
  if (threadIdx.x == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");
  constexpr int KS = D / 16;                      // k-steps of the score product
  constexpr int NT = D / 8;                       // n-tiles of the output
  constexpr uint32_t STAGE_BYTES = 2 * TILE * D * 2;          // K and V rows of one tile
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t full[MAX_STAGES], empty[MAX_STAGES];
  __shared__ int abort_word;
  __shared__ int is_last;
  volatile int* abort_flag = &abort_word;

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.H / a.KVH;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stages = a.stages;
  const int cw = min(CWARPS, stages);             // consumer warps; warp `cw` is the producer
  const int THREADS = (cw + 1) * 32;
  const int seq_len = a.seq_lens[b];
  const int row_q = a.q_start[b];                 // the request's single query token
  const int lo = (a.window > 0) ? max(0, seq_len - a.window) : 0;

  // A block of a cluster that leaves early still takes the cluster's two barriers (every branch that
  // leaves is uniform over the block), so that its peers' barriers complete.
  auto leave = [&]() {
    if (a.cluster) {
      cluster_sync_all();
      cluster_sync_all();
    }
  };
  if (seq_len <= 0) {                             // nothing to attend to: zeros, from split 0
    pdl_wait();
    if (split == 0)
      for (int idx = threadIdx.x; idx < G * D; idx += THREADS)
        a.out[(size_t)row_q * a.H * D + (size_t)kvh * G * D + idx] = __float2bfloat16_rn(0.f);
    __syncthreads();
    leave();
    return;
  }
  // tiles with visible keys, dealt out evenly over `eff` splits
  const int tile_first = lo / TILE, tile_last = (seq_len - 1) / TILE;
  const int total = tile_last - tile_first + 1;
  const int per = (total + a.nsplit - 1) / a.nsplit;
  const int eff = (total + per - 1) / per;
  if (split >= eff) {
    leave();
    return;
  }
  const int base = total / eff, rem = total % eff;
  const int my_first = tile_first + split * base + min(split, rem);
  const int n_tiles = base + (split < rem ? 1 : 0);              // >= 1
  const int k_lo = max(lo, my_first * TILE);                     // visible keys of this block
  const int k_end = min(seq_len, (my_first + n_tiles) * TILE);

  if ((smem_u32(smem) & 1023u) != 0) {                           // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(a.status, 0, 9);
    __syncthreads();
    leave();
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  if (warp == cw) {
    // ===================== producer: lanes 0..3 each own one box of every tile =====================
    const int new_pos = seq_len - 1;                             // the row this step writes
    const int BOX = 1 << a.box_shift, BOXES = TILE >> a.box_shift;
    auto box_y = [&](int j) {                                    // cache row of key j (j a multiple of BOX)
      const int lp = j / a.page;
      const int pg = lp < a.table_width ? a.block_tables[(size_t)b * a.table_width + lp] : 0;
      return (pg * a.KVH + kvh) * a.page + (j - lp * a.page);
    };
    auto issue_box = [&](int stage, int bx, int j) {
      const int y = box_y(j);
      // one copy: [2 (K, V)][BOX rows][D / 64 lines][64 columns]
      tma_load_4d(smem + (size_t)stage * STAGE_BYTES + (size_t)bx * (2 * BOX * D * 2), &kv_map, 0, 0, y, 0, &full[stage]);
    };
    // boxes of tile i that hold visible keys of this block
    auto issue_tile = [&](int i, bool skip_new) {
      const int stage = i % stages;
      const int j0 = (my_first + i) * TILE;
      int n_valid = 0;
      for (int bx = 0; bx < BOXES; ++bx) n_valid += (j0 + bx * BOX + BOX > k_lo && j0 + bx * BOX < k_end) ? 1 : 0;
      if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)n_valid * BOX * D * 2 * 2);
      __syncwarp();
      if (lane < BOXES) {
        const int j = j0 + lane * BOX;
        const bool valid = j + BOX > k_lo && j < k_end;
        const bool holds_new = new_pos >= j && new_pos < j + BOX;
        if (valid && !(skip_new && holds_new)) issue_box(stage, lane, j);
      }
    };
    const int ahead = min(n_tiles, stages);
    for (int i = 0; i < ahead; ++i) issue_tile(i, true);
    pdl_wait();
    {
      const int i_new = new_pos / TILE - my_first;               // tile of the new row, if it is one of the above
      if (i_new >= 0 && i_new < ahead && lane == 0) issue_box(i_new % stages, (new_pos % TILE) / BOX, new_pos & ~(BOX - 1));
    }
    bool ok = true;
    for (int i = ahead; i < n_tiles && ok; ++i) {
      ok = mbar_wait(&empty[i % stages], (uint32_t)((i / stages - 1) & 1), a.status, 2, abort_flag);
      if (ok) issue_tile(i, false);
    }
  } else {
    // ===================== consumers: whole tiles; stage s belongs to warp s % cw =====================
    // A stage's barriers are thus waited on by one warp, phase after phase: a parity wait tells
    // apart only neighbouring phases, so no waiter may ever be two phases behind.
    pdl_wait();
    unsigned qf[KS][4];
    load_q_fragments<D>(qf, a.qkv + (size_t)row_q * (a.H + 2 * a.KVH) * D + (size_t)kvh * G * D, G, lane);
    const bool two = G > 8;                                      // rows 8..15 hold heads too
    const float sc = a.scale * LOG2E_D;
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int stage = i % stages;
      if (stage % cw != warp) continue;
      ok = mbar_wait_spin(&full[stage], (uint32_t)((i / stages) & 1), a.status, 1, abort_flag);
      if (!ok) break;
      const uint32_t box_bytes = (uint32_t)(D * 2) << a.box_shift;  // the K rows (or the V rows) of one box
      unsigned char* ks_ = smem + (size_t)stage * STAGE_BYTES + (a.v_first ? box_bytes : 0u);
      unsigned char* vs_ = smem + (size_t)stage * STAGE_BYTES + (a.v_first ? 0u : box_bytes);
      const int bs = a.box_shift;
      const int j0 = (my_first + i) * TILE;
      const bool edge = consume_tile<D>(ks_, vs_, qf, o, m_run, l_run, j0, k_lo, k_end, sc, two, bs, lane);
      if (edge) fence_async_smem();                                // the zeros above, before a TMA refill
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);                   // the stage may be refilled
    }
  }
  __syncthreads();
  if (*abort_flag) {
    leave();
    return;
  }

  // merge the four warps' states through shared memory (every fetched tile has been consumed)
  float* m_s = reinterpret_cast<float*>(smem);                     // [CWARPS][16]
  float* l_s = m_s + CWARPS * 16;                                  // [CWARPS][16]
  float* o_s = l_s + CWARPS * 16;                                  // [CWARPS][16][D]
  if (warp < cw) {
    const int r0 = lane >> 2, r1 = r0 + 8;
    if ((lane & 3) == 0) {
      m_s[warp * 16 + r0] = m_run[0];
      m_s[warp * 16 + r1] = m_run[1];
      l_s[warp * 16 + r0] = l_run[0];
      l_s[warp * 16 + r1] = l_run[1];
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int d = t * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(o_s + ((size_t)warp * 16 + r0) * D + d) = make_float2(o[t][0], o[t][1]);
      if (r1 < G) *reinterpret_cast<float2*>(o_s + ((size_t)warp * 16 + r1) * D + d) = make_float2(o[t][2], o[t][3]);
    }
  }
  __syncthreads();
  // each warp's weight 2^(m_w - M) and the block's (M, L), once per head; then 16 bytes a thread
  float* f_s = o_s + CWARPS * 16 * D;                              // [CWARPS][16]
  float* M_s = f_s + CWARPS * 16;                                  // [16]
  float* L_s = M_s + 16;                                           // [16]
  float* c_acc = L_s + 16;                                         // [G][D], read by the cluster's blocks
  if ((int)threadIdx.x < cw * G) {
    const int v = threadIdx.x / G, g = threadIdx.x % G;
    float M = -INFINITY;
    for (int u = 0; u < cw; ++u) M = fmaxf(M, m_s[u * 16 + g]);
    const float mv = m_s[v * 16 + g];
    f_s[v * 16 + g] = (mv == -INFINITY) ? 0.f : exp2f(mv - M);     // a warp without a tile weighs nothing
    if (v == 0) {
      float L = 0.f;
      for (int u = 0; u < cw; ++u) {
        const float mu = m_s[u * 16 + g];
        if (mu != -INFINITY) L += l_s[u * 16 + g] * exp2f(mu - M);
      }
      M_s[g] = M;
      L_s[g] = L;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * (D / 4); idx += THREADS) {
    const int g = idx / (D / 4), d = (idx % (D / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int v = 0; v < cw; ++v) {
      const float f = f_s[v * 16 + g];
      const float4 x = *reinterpret_cast<const float4*>(o_s + ((size_t)v * 16 + g) * D + d);
      acc.x += x.x * f; acc.y += x.y * f; acc.z += x.z * f; acc.w += x.w * f;
    }
    const int h = kvh * G + g;
    if (eff == 1) {
      const float L = L_s[g], inv = L > 0.f ? 1.f / L : 0.f;
      bf16* op = a.out + (size_t)row_q * a.H * D + (size_t)h * D + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    } else if (a.cluster) {
      *reinterpret_cast<float4*>(c_acc + g * D + d) = acc;
    } else {
      const size_t pi = ((size_t)b * a.H + h) * a.nsplit + split;
      *reinterpret_cast<float4*>(a.part_acc + pi * D + d) = acc;
      if (d == 0) *reinterpret_cast<float2*>(a.part_ml + pi * 2) = make_float2(M_s[g], L_s[g]);
    }
  }
  if (eff == 1) {
    __syncthreads();
    leave();
    return;
  }

  if (a.cluster) {
    // Block `split` finishes the 16-byte pieces split, split + eff, ... of the output out of the
    // shared memory of the eff blocks that got tiles, in split order:
    //   out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
    __syncthreads();
    cluster_sync_all();
    for (int piece = split + eff * (int)threadIdx.x; piece < G * (D / 4); piece += eff * THREADS) {
      const int g = piece / (D / 4), d = (piece % (D / 4)) * 4;
      float m[8], l[8];
      float4 x[8];
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2)
        if (s2 < eff) {
          m[s2] = ld_peer_f32(peer_shared(M_s + g, s2));
          l[s2] = ld_peer_f32(peer_shared(L_s + g, s2));
          x[s2] = ld_peer_v4(peer_shared(c_acc + g * D + d, s2));
        }
      float M = -INFINITY;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2)
        if (s2 < eff) M = fmaxf(M, m[s2]);
      float L = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2)
        if (s2 < eff) {
          const float f = (m[s2] == -INFINITY) ? 0.f : exp2f(m[s2] - M);
          L += l[s2] * f;
          acc.x += x[s2].x * f; acc.y += x[s2].y * f; acc.z += x[s2].z * f; acc.w += x[s2].w * f;
        }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      bf16* op = a.out + (size_t)row_q * a.H * D + (size_t)(kvh * G + g) * D + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
    __syncthreads();
    cluster_sync_all();                                            // no block leaves while a peer still reads it
    return;
  }

  // The block that finishes last for this (request, kv head) merges all splits, in split order:
  //   out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
  // More than 32 splits (one or two requests with a very long context) merge in two levels, or the one
  // block that merges would fetch hundreds of kilobytes alone (128 splits: 22 us of a 53 us launch): the
  // last block of every 8 neighbouring splits folds them into the first one's place (same form: sums
  // against the group's maximum), the last of those blocks merges the groups.
  float* w_s = reinterpret_cast<float*>(smem);                     // [G][count]
  auto merge = [&](int first, int stride, int count, bool final) {
    float* m_all = w_s + G * count;                                // [G][count]
    float* l_all = m_all + G * count;                              // [G][count]
    float* ML = l_all + G * count;                                 // [G][2]: what a fold leaves as (m, l)
    for (int idx = threadIdx.x; idx < G * count; idx += THREADS) {
      const int g = idx / count, s2 = idx % count;
      const size_t pi = ((size_t)b * a.H + kvh * G + g) * a.nsplit + first + s2 * stride;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + pi * 2));
      m_all[idx] = ml.x;
      l_all[idx] = ml.y;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * count; idx += THREADS) {
      const int g = idx / count;
      float M = -INFINITY, L = 0.f;
      for (int s2 = 0; s2 < count; ++s2) M = fmaxf(M, m_all[g * count + s2]);
      if (M > -INFINITY)
        for (int s2 = 0; s2 < count; ++s2) L += l_all[g * count + s2] * exp2f(m_all[g * count + s2] - M);
      if (final) {
        w_s[idx] = (L > 0.f) ? exp2f(m_all[idx] - M) / L : 0.f;
      } else {
        w_s[idx] = (M > -INFINITY) ? exp2f(m_all[idx] - M) : 0.f;
        if (idx % count == 0) {
          ML[2 * g] = M;
          ML[2 * g + 1] = L;
        }
      }
    }
    __syncthreads();
    // sum_s w[g, s] * acc[g, s, d..d+3]: independent 16-byte loads, split order
    for (int idx = threadIdx.x; idx < G * (D / 4); idx += THREADS) {
      const int g = idx / (D / 4), d = (idx % (D / 4)) * 4;
      const int h = kvh * G + g;
      float* src = a.part_acc + (((size_t)b * a.H + h) * a.nsplit + first) * D + d;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
      for (int s2 = 0; s2 < count; ++s2) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)s2 * stride * D));
        const float w = w_s[g * count + s2];
        acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
      }
      if (final) {
        bf16* op = a.out + (size_t)row_q * a.H * D + (size_t)h * D + d;
        *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x, acc.y);
        *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z, acc.w);
      } else {
        *reinterpret_cast<float4*>(src) = acc;                     // (this thread alone reads and writes this piece)
        if (d == 0) {
          const size_t pi = ((size_t)b * a.H + h) * a.nsplit + first;
          *reinterpret_cast<float2*>(a.part_ml + pi * 2) = make_float2(ML[2 * g], ML[2 * g + 1]);
        }
      }
    }
  };
  // true for the block that arrives last of `of` at `counter`, which it leaves at zero for the next launch
  auto last_of = [&](int* counter, int of) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int ticket = atomicAdd(counter, 1);
      is_last = (ticket == of - 1);
      if (is_last) *counter = 0;
    }
    __syncthreads();
    const bool last = is_last;
    __syncthreads();                                               // (is_last is written again at the second level)
    if (last) __threadfence();
    return last;
  };
  const int pair = b * a.KVH + kvh;
  if (eff <= MERGE_FLAT) {
    if (!last_of(&a.counters[pair], eff)) return;
    merge(0, 1, eff, true);
    return;
  }
  const int group = split / MERGE_GROUP, first = group * MERGE_GROUP;
  const int groups = (eff + MERGE_GROUP - 1) / MERGE_GROUP;
  if (!last_of(&a.counters[(int)gridDim.z * a.KVH + pair * MERGE_GROUPS_MAX + group], min(MERGE_GROUP, eff - first))) return;
  merge(first, 1, min(MERGE_GROUP, eff - first), false);
  if (!last_of(&a.counters[pair], groups)) return;
  merge(0, MERGE_GROUP, groups, true);
}

// K and V caches ([rows, D] bfloat16 each, `gap` bytes apart) as one tensor of
// [2][rows][D / 64][64] copied in boxes of [2][box_rows][D / 64][64] with the 128-byte swizzle.
bool kv_tensor_map(CUtensorMap* out, const void* lo_ptr, unsigned long long gap, int rows, int D, int box_rows) {
  struct Key {
    const void* ptr;
    unsigned long long gap;
    int rows, D, box;
    bool operator==(const Key& o) const { return ptr == o.ptr && gap == o.gap && rows == o.rows && D == o.D && box == o.box; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.ptr) ^ std::hash<unsigned long long>()(k.gap * 31 + (unsigned)k.rows) ^ ((size_t)k.D << 50) ^ ((size_t)k.box << 40);
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{lo_ptr, gap, rows, D, box_rows};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  tc::EncodeTiledFn fn = tc::encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {64, (cuuint64_t)(D / 64), (cuuint64_t)rows, 2};
  cuuint64_t strides[3] = {128, (cuuint64_t)D * 2, (cuuint64_t)gap};
  cuuint32_t box[4] = {64, (cuuint32_t)(D / 64), (cuuint32_t)box_rows, 2};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(lo_ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

int* dec_status_word() {
  static int* p = nullptr;
  if (p == nullptr && cudaGetSymbolAddress((void**)&p, g_dec_status) != cudaSuccess) p = nullptr;
  return p;
}

int g_cluster_max = 8;

template <int D>
int launch_tma(const CUtensorMap& kv_map, const DecArgs& a, int B, cudaStream_t s) {
  const size_t smem = (size_t)a.stages * 2 * TILE * D * 2;
  static size_t configured = 0;
  if (smem != configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_decode_tma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  const int threads = ((a.stages < CWARPS ? a.stages : CWARPS) + 1) * 32;
  // Up to 8 splits can be one thread-block cluster per (request, kv head), but only while all clusters
  // fit the chip at once: clusters that come in two waves lose more than the merge gains (batch 24 x
  // 2 kv heads: clusters of 6 25 us, 6 splits with the ticket 21 us, clusters of 4 17 us).  So: the
  // largest count from the wanted one down to 0.6 of it whose clusters all fit (from 0.8 of it down where
  // more than 8 are wanted); none: the ticket.
  DecArgs b = a;
  b.cluster = 0;
  if (ts_clusters_enabled() && a.nsplit >= 2) {
    static int known[MAX_STAGES + 1][9];                           // 0: not asked, -1: no cluster, else how many fit at once
    const int pairs = B * a.KVH;
    for (int n = a.nsplit < g_cluster_max ? a.nsplit : g_cluster_max; n >= 2 && 10 * n >= 6 * a.nsplit; --n) {
      // (9 or 10 wanted and clusters of 8 instead lose inside a step: 32 (request, kv head) pairs, 9 wanted:
      // 1.711 against 1.511 ms a decode step with the ticket; while 12 wanted, clusters of 8: 1.436 against
      // 1.480 ms, and 6 wanted, clusters of 5: 1.686 against 1.806 ms)
      if (a.nsplit > 8 && 10 * n > 8 * a.nsplit) continue;
      int& k = known[a.stages][n];
      if (k == 0) {
        k = -1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n, 1, 1);
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)n;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, attention_decode_tma_kernel<D>, &cfg) == cudaSuccess && clusters >= 1) k = clusters;
        cudaGetLastError();                                        // a refusal is an answer, not an error
      }
      if (k >= pairs) {
        b.cluster = 1;
        b.nsplit = n;
        break;
      }
    }
  }
  ts_launch_cluster(attention_decode_tma_kernel<D>, dim3(b.cluster ? b.nsplit : 1, 1, 1), dim3(b.nsplit, a.KVH, B),
                    dim3(threads), smem, s, kv_map, b);
  TS_LAUNCH_CHECK();
}

}  // namespace

// The largest cluster the splits of a (request, kv head) may form (2..8; for measurements).
TS_API void ts_set_decode_tma_cluster_max(int n) { g_cluster_max = n < 1 ? 1 : (n > 8 ? 8 : n); }

// Whether this kernel takes the shape (else the caller uses ts_attention_decode or the generic kernel).
int* ts_dec_status_word() { return dec_status_word(); }

TS_API int ts_attention_decode_tma_supported(int H, int KVH, int D, int page, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && H / KVH <= 16 && (D == 64 || D == 128) && page >= MIN_BOX &&
         page % MIN_BOX == 0;
}

// 0 when no block ever gave up on a wait (synchronises the device).
TS_API int ts_attention_decode_tma_status() {
  int* p = dec_status_word();
  int v = -1;
  if (p != nullptr) cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

// Blocks of this kernel that fit one SM at `stages` stages: what the caller sizes nsplit with.
TS_API int ts_attention_decode_tma_blocks_per_sm(int D, int stages) {
  if ((D != 64 && D != 128) || stages < 2 || stages > MAX_STAGES) return 0;
  const size_t smem = (size_t)stages * 2 * TILE * D * 2;
  const int threads = ((stages < CWARPS ? stages : CWARPS) + 1) * 32;
  int n = 0;
  cudaError_t e;
  if (D == 64) {
    cudaFuncSetAttribute(attention_decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_tma_kernel<64>, threads, smem);
  } else {
    cudaFuncSetAttribute(attention_decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_tma_kernel<128>, threads, smem);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// One query token per request (rows q_start[b]).  `scratch` holds
// ts_attention_decode_scratch_floats(B, H, D, nsplit) floats when nsplit > 1, and `counters`
// B * KVH ints, 17 times as many when nsplit > 16 (one per group of 8 splits besides), that are zero on
// entry (the kernel leaves them zero).  num_pages: pages in the pool
// (rows of the cache = num_pages * KVH * page).  window <= 0: none.  stages: 2..8 tiles of
// 64 keys in flight per block.
TS_API int ts_attention_decode_tma(void* out, void* scratch, int* counters, const void* qkv, const void* k_cache,
                                   const void* v_cache, const int* block_tables, const int* q_start,
                                   const int* seq_lens, int B, int table_width, int H, int KVH, int D, int page,
                                   int num_pages, float scale, int window, int nsplit, int stages, void* stream) {
  if (B <= 0) return 0;
  if (!ts_attention_decode_tma_supported(H, KVH, D, page, TS_BF16))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_decode_tma: H=%d KVH=%d D=%d page=%d is not taken by this kernel", H, KVH, D, page);
  if (nsplit < 1 || nsplit > 128 || B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_tma: nsplit=%d B=%d", nsplit, B);
  if (stages < 2 || stages > MAX_STAGES || (size_t)stages * 2 * TILE * D * 2 > 220 * 1024)
    TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_tma: %d stages at head_dim %d", stages, D);
  if (nsplit > 1 && (scratch == nullptr || counters == nullptr))
    TS_REFUSE(TS_ERR_SHAPE, "ts_attention_decode_tma: %d splits need scratch and counters", nsplit);
  if ((((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
    TS_REFUSE(TS_ERR_ALIGN, "ts_attention_decode_tma: buffers must be 16-byte aligned");
  // the merges reuse the stage buffers: 3 * G * nsplit floats and (2 + D) * 64 floats must fit
  const int G = H / KVH;
  const size_t smem = (size_t)stages * 2 * TILE * D * 2;
  if (sizeof(float) * 3 * G * nsplit > smem || sizeof(float) * ((3 + D) * CWARPS * 16 + 32 + 16 * D) > smem)
    TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_tma: %d stages are too few for the merge buffers", stages);
  int* status = dec_status_word();
  if (status == nullptr) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_tma: no status word");
  const long long rows = (long long)num_pages * KVH * page;
  if (rows <= 0 || rows > 0x7fffffffLL) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_decode_tma: cache of %lld rows", rows);
  const int box_shift = page % 64 == 0 ? 6 : (page % 32 == 0 ? 5 : 4);
  // K and V as one tensor [2][rows][D / 64][64]: the lower address first
  const bool v_first = (uintptr_t)v_cache < (uintptr_t)k_cache;
  const void* lo_ptr = v_first ? v_cache : k_cache;
  const unsigned long long gap = v_first ? (uintptr_t)k_cache - (uintptr_t)v_cache : (uintptr_t)v_cache - (uintptr_t)k_cache;
  if (gap < (unsigned long long)rows * D * 2 || gap >= (1ull << 40))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_decode_tma: key and value caches %llu bytes apart", gap);
  CUtensorMap kv_map;
  if (!kv_tensor_map(&kv_map, lo_ptr, gap, (int)rows, D, 1 << box_shift))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_decode_tma: cuTensorMapEncodeTiled failed");
  DecArgs a;
  a.out = (bf16*)out;
  a.part_acc = (float*)scratch;
  a.part_ml = a.part_acc ? a.part_acc + (size_t)B * H * nsplit * D : nullptr;
  a.qkv = (const bf16*)qkv;
  a.block_tables = block_tables;
  a.q_start = q_start;
  a.seq_lens = seq_lens;
  a.table_width = table_width;
  a.H = H;
  a.KVH = KVH;
  a.page = page;
  a.scale = scale;
  a.window = window;
  a.nsplit = nsplit;
  a.stages = stages;
  a.box_shift = box_shift;
  a.v_first = v_first ? 1 : 0;
  a.counters = counters;
  a.status = status;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 64) return launch_tma<64>(kv_map, a, B, s);
  return launch_tma<128>(kv_map, a, B, s);
}
