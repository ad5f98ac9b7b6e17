// Last-error text of the C ABI (one buffer per host thread).
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void ts_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

TS_API const char* ts_last_error() { return g_error; }

// Compiled-for architecture and ABI version, so the Python side can refuse a stale library.
TS_API int ts_abi_version() { return 8; }

// Programmatic dependent launch for this library's kernels (on by default).
static bool g_pdl = true;
bool ts_pdl_enabled() { return g_pdl; }
TS_API void ts_set_pdl(int on) { g_pdl = on != 0; }

// Thread-block clusters where the splits of a kernel merge through distributed shared memory (the
// decode attention, the q/k/v product that rotates): on by default; off: scratch and a ticket
// counter at every split count.
static bool g_clusters = true;
bool ts_clusters_enabled() { return g_clusters; }
TS_API void ts_set_clusters(int on) { g_clusters = on != 0; }

// The status words of the kernels with bounded waits, in the order the sampler reports them.
TsStatusPtrs ts_status_ptrs() {
  TsStatusPtrs s;
  s.p[0] = ts_gemm_status_word();
  s.p[1] = ts_attn_status_word();
  s.p[2] = ts_dec_status_word();
  s.p[3] = ts_step_status_word();
  return s;
}

// Sets every status word back to 0, in stream order (after a fault was reported and dealt with).
TS_API int ts_clear_status(void* stream) {
  const TsStatusPtrs s = ts_status_ptrs();
  for (int i = 0; i < TS_STATUS_WORDS; ++i)
    if (s.p[i] != nullptr) {
      cudaError_t e = cudaMemsetAsync(const_cast<int*>(s.p[i]), 0, sizeof(int), (cudaStream_t)stream);
      if (e != cudaSuccess) TS_REFUSE((int)e, "ts_clear_status: %s", cudaGetErrorString(e));
    }
  return 0;
}

// Test hook: writes `value` into status word `which` in stream order, as a kernel that gave up would.
TS_API int ts_poke_status(int which, int value, void* stream) {
  const TsStatusPtrs s = ts_status_ptrs();
  if (which < 0 || which >= TS_STATUS_WORDS || s.p[which] == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_poke_status: no word %d", which);
  cudaError_t e = cudaMemcpyAsync(const_cast<int*>(s.p[which]), &value, sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) TS_REFUSE((int)e, "ts_poke_status: %s", cudaGetErrorString(e));
  return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? 0 : 1;
}
