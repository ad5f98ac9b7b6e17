// Arguments of the fused decode step (decode_step.cu).  Plain C structs: the Python side mirrors them
// with ctypes and hands ts_decode_step a host copy.
#pragma once

#include <stdint.h>

#define TS_STEP_MAX_TOKENS 16        // requests (one token each) a step may hold
#define TS_STEP_MAX_HIDDEN 1536     // widest residual stream the in-kernel norm keeps in registers
#define TS_STEP_MAX_GROUPS 4         // cache groups (block table + slot mapping each)
#define TS_STEP_MAX_UNITS 1024       // (tile, part) units of a product that is split over K: slots of partial sums
#define TS_STEP_TICKETS_EACH 512     // ticket counters per kind
#define TS_STEP_TICKETS_QKV 0
#define TS_STEP_TICKETS_O (1 * TS_STEP_TICKETS_EACH)
#define TS_STEP_TICKETS_DOWN (2 * TS_STEP_TICKETS_EACH)
#define TS_STEP_TICKETS_ATTN (3 * TS_STEP_TICKETS_EACH)
#define TS_STEP_TICKETS (4 * TS_STEP_TICKETS_EACH)

// How one product (q/k/v, output, gate/up, down, head: indices 0..4) is cut into units.
typedef struct {
  int R;        // tiles of 128 weight rows
  int KB;       // k-blocks of 64 columns
  int S;        // parts K is cut into (1: a unit is a whole tile)
  int per;      // k-blocks a part
  int rot;      // block c takes units (c + rot) % blocks, + blocks, ...
  int pad[3];
} TsStepShape;

// One layer.  Device pointers.
typedef struct {
  const void* ln1_w;          // norm before the mixer [hidden], 32-bit
  const void* ln2_w;          // norm before the feed-forward [hidden], 32-bit
  const void* qkv_bias;       // bfloat16 [(H + 2 KVH) * 128] or null
  void* k_cache;              // [pages, KVH, page, 128] bfloat16
  void* v_cache;
  const float* cos_t;         // [positions, 64] or null (no rotation)
  const float* sin_t;
  int group;                  // which block table / slot mapping
  int window;                 // keys a query sees; <= 0: all
} TsStepLayer;

typedef struct {
  const TsStepLayer* layers;  // device, [L]
  const void* maps;           // device, CUtensorMap [4 L + 1]: per layer q/k/v, output, gate/up, down; then the head
  int L, T, H, KVH, hidden, inter, V, page;
  int norm_w_is_f32, stages, work_bytes, lookahead, attn_splits;
  float eps, scale;
  TsStepShape shape[5];
  // the step's inputs (device)
  const int* ids;             // [T]
  const int* positions;       // [T]
  const int* seq_lens;        // [T] context length including the new token; 0: a padding row
  const int* block_tables[TS_STEP_MAX_GROUPS];
  const int* slot_mapping[TS_STEP_MAX_GROUPS];
  int table_width[TS_STEP_MAX_GROUPS];
  int group_window[TS_STEP_MAX_GROUPS];   // the window of the layers of each group (<= 0: none)
  int num_groups;
  int num_pages;              // pages of a cache pool (what a block table may name)
  int l2_ahead;               // != 0: a layer's gate/up and down weights are asked into L2 when the layer begins
  const void* embedding;      // bfloat16 [vocabulary, hidden]
  const void* final_norm_w;
  // work buffers (device)
  float* resid;               // [16, hidden]: the residual stream, 32-bit (products add their parts into it)
  float* qkv;                 // [16, (H + 2 KVH) * 128]: sums of the q/k/v product's parts, before bias and rotation
  void* attn;                 // bfloat16 [16, H * 128]
  void* act;                  // bfloat16 [16, inter]
  float* logits;              // [T, V]
  float* attn_part;           // [T * H * attn_splits * (128 + 2)]
  int* ctrl;                  // [0] barrier counter, [1] abort flag: cleared by ts_decode_step
  int* tickets;               // [TS_STEP_TICKETS], zero (the attention's key splits take tickets)
  int* status;                // set by ts_decode_step
  long long* trace;           // null, or [blocks][5 L + 2][8] clock64: arrival at and exit from every grid barrier, marks within the phase before it
} TsStepArgs;
