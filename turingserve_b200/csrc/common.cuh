// Shared helpers for the sm_100a kernels: storage types, conversions, reductions, the C ABI.
//
// Every entry point is `extern "C" int ts_<name>(..., void* stream)`.  It returns 0 on success,
// a positive cudaError_t when the launch failed, or a negative code when the arguments were
// refused (ts_last_error() then holds the reason).  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TS_API extern "C" __attribute__((visibility("default")))

enum TsDtype : int { TS_F32 = 0, TS_BF16 = 1 };

// Argument refusals (negative return codes).
enum TsError : int {
  TS_ERR_DTYPE = -1,
  TS_ERR_SHAPE = -2,
  TS_ERR_ALIGN = -3,
  TS_ERR_UNSUPPORTED = -4,
  TS_ERR_LIMIT = -5,
};

void ts_set_error(const char* fmt, ...);

#define TS_REFUSE(code, ...)   \
  do {                         \
    ts_set_error(__VA_ARGS__); \
    return (code);             \
  } while (0)

#define TS_LAUNCH_CHECK()                                          \
  do {                                                             \
    cudaError_t e__ = cudaGetLastError();                          \
    if (e__ != cudaSuccess) {                                      \
      ts_set_error("%s: %s", __func__, cudaGetErrorString(e__));   \
      return (int)e__;                                             \
    }                                                              \
    return 0;                                                      \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }
// silu(g) = g / (1 + e^-g) on its way to a rounding to T.  For bfloat16 the hardware's approximate
// exponential and reciprocal serve: their error (about 2^-21 relative) is far inside half a
// bfloat16 step (2^-9), and the exact ones cost as much issue time as the activation kernel's
// memory traffic takes.  The 32-bit path keeps the exact ones.
template <typename T> __device__ __forceinline__ float silu_for(float g) { return g / (1.f + expf(-g)); }
template <> __device__ __forceinline__ float silu_for<__nv_bfloat16>(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// Round a 32-bit value to the storage type and back (the model-dtype rounding points).
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f(from_f<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds at least 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch: a kernel launched with ts_launch may start while its predecessor
// in the stream is still running.  Every kernel calls pdl_launch_dependents() first (its successor
// may be scheduled) and pdl_wait() before it reads or writes anything a predecessor may touch;
// because every kernel in a chain waits, completion stays ordered along the whole chain.  Both are
// no-ops for a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Thread-block clusters: every thread of every block of the cluster takes the barrier; a block's
// shared memory may be read by its peers between two of them.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of block `rank`'s copy of this block's `own`.
__device__ __forceinline__ unsigned peer_shared(const void* own, unsigned rank) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(own);
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_peer_f32(unsigned addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_v4(unsigned addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// Status words of the kernels whose waits are bounded (0 = fine; otherwise which wait ran out):
// the tcgen05 product, the tcgen05 prompt attention, the TMA decode attention, the fused decode step.  Device addresses,
// null when a word could not be found.  ts_sample / ts_sample_greedy copy them out beside the tokens.
constexpr int TS_STATUS_WORDS = 4;
struct TsStatusPtrs {
  const int* p[TS_STATUS_WORDS];
};
int* ts_gemm_status_word();
int* ts_attn_status_word();
int* ts_dec_status_word();
int* ts_step_status_word();
TsStatusPtrs ts_status_ptrs();

bool ts_pdl_enabled();
bool ts_clusters_enabled();

// cluster: the shape of the thread-block clusters the grid is cut into (each grid dimension must be
// a multiple of the cluster's); (1, 1, 1): none.
template <typename... KArgs, typename... Args>
inline cudaError_t ts_launch_cluster(void (*kernel)(KArgs...), dim3 cluster, dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (ts_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t ts_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  return ts_launch_cluster(kernel, dim3(1, 1, 1), grid, block, smem, stream, static_cast<Args&&>(args)...);
}
