// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference (its kernels get their scratch from torch's
// allocator, turingserve/ops/triton_decode_attention.py:187-200); it exists for users of this
// library who call it from places where cudaMalloc is off limits: a host thread that runs while a
// CUDA graph is being captured on its stream, a process whose memory pool was sized once at start-up
// and is policed, a real-time loop that may not take the allocator's lock.
//
// ts_attention_decode_static is ts_attention_decode (paged decode attention with the keys split
// over several blocks) with its scratch memory -- the per-split partial results and the ticket
// counters -- taken from one fixed array that is part of the library image instead of from the
// caller.  The array holds TS_STATIC_SCRATCH_FLOATS floats (4 MiB) and TS_STATIC_COUNTERS
// counters; every GPU that loads the library carries it until the process exits.
//
//   * It allocates nothing: no cudaMalloc, no cudaFree, no library routine that allocates.
//   * Shapes whose scratch would not fit (B * H * nsplit * (D + 2) floats, B * KVH counters) are
//     refused with TS_ERR_LIMIT and a message in ts_last_error(); nothing is launched.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current), under a lock, so two host threads may make it together.  Make
//     that first call outside any stream capture.
//   * All calls share the one array and it keeps what the last call left there.  The counters are
//     cleared on the stream before every launch.  Two calls that may overlap on the GPU (different
//     streams, no ordering between them) race on the array; order them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define TS_STATIC_SCRATCH_FLOATS (1 << 20)
#define TS_STATIC_COUNTERS 4096

// Same arguments and return codes as ts_attention_decode, without `scratch` and `counters`.
int ts_attention_decode_static(void* out, const void* qkv, const void* k_cache, const void* v_cache,
                               const int* block_tables, const int* q_start, const int* seq_lens, int B,
                               int table_width, int H, int KVH, int D, int page, float scale, int window,
                               int nsplit, void* stream);

#ifdef __cplusplus
}
#endif
