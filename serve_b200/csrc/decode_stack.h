// The description of one layer that sb_decode_stack (decode_stack.cu) runs: an array of these lies in device memory.
// All pointers are device pointers; weights are bfloat16, row-major [out, in]. Filled by the host once per model
// (serve_b200/kernels/cuda.py builds the same layout with numpy: keep the two in step).
#pragma once
#include <stdint.h>

#define SB_STACK_MAX_GROUPS 4      // cache groups (block tables) a run of layers may name

#ifdef __cplusplus
extern "C" {
#endif

typedef struct SbStackLayer {
  const void* wqkv;        // [(H + 2 Hkv) D, hidden]: q rows, k rows, v rows; rotary pairs adjacent
  const void* wo;          // [hidden, H D]
  const void* wgu;         // [2 inter, hidden]: gate rows, then up rows
  const void* wdown;       // [hidden, inter]
  const void* norm1;       // [hidden] float or bfloat16 (norm_f32 bit 0)
  const void* norm2;       // [hidden] (norm_f32 bit 1)
  const float* inv_freq;   // [rot / 2]
  void* kc;                // [num_pages, Hkv, page_size, D] bfloat16
  void* vc;
  float eps1;
  float eps2;
  float scale_log2;        // softmax scale times log2(e)
  int32_t rot;             // rotated elements of a head (even, <= D)
  int32_t window;          // 0: all keys
  int32_t norm_f32;
  int32_t group;           // which block table
  int32_t num_pages;
  int32_t write_cache;     // 0: this execution reads a cache another one wrote
  int32_t pad;
} SbStackLayer;

#ifdef __cplusplus
}
#endif
