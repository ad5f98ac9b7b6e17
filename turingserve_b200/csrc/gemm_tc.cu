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
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int BM = 128;            // tile rows = TMEM lanes
constexpr int BK = 64;             // 64 bf16 = 128 bytes = one swizzle line
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false (and `status` set) when the phase does not complete in time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  atomicCAS(status, 0, code);
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor: K-major tile of [rows][64] bf16 written by TMA with the 128-byte
// swizzle; 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address, 16-byte units
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                            // 128-byte swizzle
  return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}

struct GemmArgs {
  void* out;              // bf16 or float [M, N]; or float scratch [splits, M, N] when splits > 1
  const bf16* bias;       // [N] or null (applied here only when splits == 1)
  int M, N, K;
  int k_blocks_per_split;
  int splits;
  int out_is_float;
  int* status;
};

// BN: tile columns (UMMA N).  SWAP: the tile rows are weight rows (outputs), columns are tokens.
template <int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
               const GemmArgs args) {
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* a_s = smem;
  unsigned char* b_s = smem + STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(b_s + STAGES * B_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * BM;                 // first tile row (tokens, or weight rows when SWAP)
  const int col0 = blockIdx.y * BN;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb_begin = blockIdx.z * args.k_blocks_per_split;
  const int kb_end = min(total_kb, kb_begin + args.k_blocks_per_split);
  const int n_kb = kb_end - kb_begin;

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
      const int w_row = SWAP ? row0 : col0, x_row = SWAP ? col0 : row0;
      const int early = n_kb < STAGES ? n_kb : STAGES;
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&full[i], A_BYTES + B_BYTES);
        tma_load_2d(w_s + i * W_BYTES, w_map, (kb_begin + i) * BK, w_row, &full[i]);
      }
      pdl_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(x_s + i * X_BYTES, x_map, (kb_begin + i) * BK, x_row, &full[i]);
      for (int i = early; i < n_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, args.status, 1, abort_flag)) break;
        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
        const int k = (kb_begin + i) * BK;
        tma_load_2d(w_s + s * W_BYTES, w_map, k, w_row, &full[s]);
        tma_load_2d(x_s + s * X_BYTES, x_map, k, x_row, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        ok = mbar_wait(&full[s], ph, args.status, 2, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc(smem_u32(a_s + s * A_BYTES));
        const uint64_t db = smem_desc(smem_u32(b_s + s * B_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma(tmem_base, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc,
               (i > 0 || k > 0) ? 1u : 0u);
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
    if (ok) {
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

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, K, box_rows;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K << 20) ^ ((size_t)k.box_rows << 44);
  }
};

// A [rows, K] bf16 row-major matrix seen as boxes of [box_rows][64] with the 128-byte swizzle;
// reads outside the matrix give zeros.
bool tensor_map(CUtensorMap* out, const void* ptr, int rows, int K, int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{ptr, rows, K, box_rows};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

__device__ int g_gemm_status = 0;       // 0 = fine; otherwise the wait that ran out (see ts_linear_tc_status)

int* status_word() {
  static int* p = nullptr;
  if (p == nullptr && cudaGetSymbolAddress((void**)&p, g_gemm_status) != cudaSuccess) p = nullptr;
  return p;
}

template <int BN, int STAGES, bool SWAP>
int launch(const CUtensorMap& rows_map, const CUtensorMap& cols_map, const GemmArgs& args, dim3 grid, cudaStream_t s) {
  constexpr size_t smem = 1024 + (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_linear_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  ts_launch(gemm_tc_kernel<BN, STAGES, SWAP>, dim3(grid), dim3(GEMM_THREADS), smem, s, rows_map, cols_map, args);
  TS_LAUNCH_CHECK();
}

}  // namespace

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
    if (bn == 16) rc = launch<16, 4, true>(rows_map, cols_map, a, grid, s);
    else if (bn == 32) rc = launch<32, 4, true>(rows_map, cols_map, a, grid, s);
    else if (bn == 64) rc = launch<64, 4, true>(rows_map, cols_map, a, grid, s);
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
