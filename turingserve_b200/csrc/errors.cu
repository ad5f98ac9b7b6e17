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
TS_API int ts_abi_version() { return 3; }

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
