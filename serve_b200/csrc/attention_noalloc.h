// Decoding attention over the paged cache for callers that must not allocate device memory.
//
// This entry point has no counterpart in limei1221/serve; it exists for users of this library whose
// process cannot ask for device memory at the moment they need attention: programs that carve up the
// whole device at start-up and serve from that fixed budget (a later cudaMalloc would fail or would
// break their accounting), and code that runs inside another runtime's plug-in or callback, where
// calling an allocator is forbidden. The regular entry point (sb_attention_mma) expects the caller to
// bring scratch memory for the partial results of split key ranges; this one brings its own.
//
// The scratch is one file-scope array in device memory, linked into the library: every GPU on which
// the library is loaded sets aside SB_NOALLOC_MAX_TILES * 16 * (head_dim + 2) floats (2.2 MB at
// head_dim 64, 8.5 MB at 256) plus SB_NOALLOC_MAX_TILES ints, from load until the process exits.
// All calls share that array. It keeps whatever the last call left in it; the only part that has to
// start at zero (the arrival counters of the split merge) is cleared by every call before its kernels
// run. Two calls whose kernels overlap on the GPU (different streams, no ordering between them) race
// on the array and give wrong results: order such calls.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress) and keeps it;
// make that first call outside any stream capture. No call allocates or frees memory.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Most (request, kv head, key split) triples one call may have: n_rows * Hkv * num_splits.
#define SB_NOALLOC_MAX_TILES 512

// Returns SB_NOALLOC_MAX_TILES (so that a caller can size num_splits without reading this header).
int sb_attention_decode_noalloc_max_tiles(void);

// Attention for a step in which every request brings at most 16 / (H / Hkv) tokens (decoding).
// Arguments as for sb_attention_mma: qkv [tokens, q_stride] bfloat16 with queries in the first H * head_dim
// columns; kc, vc [num_pages, Hkv, ps, head_dim] bfloat16; block_table [n_rows, bt_width]; cu_q [n_rows + 1];
// kv_len [n_rows]; out [tokens, H * head_dim] bfloat16. max_q is the largest number of tokens any request
// brings. num_splits (1..32) cuts each request's keys into that many ranges.
// Returns 0, or -2 for a shape it does not take (more than 16 rows for some request, H not a multiple of
// Hkv, num_splits out of range), -3 for misaligned pointers, -4 when n_rows * Hkv * num_splits exceeds
// SB_NOALLOC_MAX_TILES, or a positive cudaError_t.
int sb_attention_decode_noalloc(const void* qkv, int q_stride, const void* kc, const void* vc, const int* block_table,
                                int bt_width, const int* cu_q, const int* kv_len, int H, int Hkv, int ps, int num_pages,
                                float scale, int window, void* out, int n_rows, int max_q, int num_splits,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
