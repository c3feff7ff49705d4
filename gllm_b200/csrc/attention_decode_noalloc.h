// gllm_attention_decode_bf16_noalloc: split-KV decode attention for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in TheEpicDolphin/gllm; it exists for
// users of this library.
//
// Who needs it: code that runs where cudaMalloc is not an option.  Examples are
// a host callback or a plugin inside someone else's runtime that owns all
// device memory and forbids further allocations, code that runs after a
// device-wide memory budget was fixed, and a latency-critical loop in which an
// allocation (which may synchronise the whole device) is not acceptable.  The ordinary entry
// point, gllm_attention_decode_bf16, asks its caller for two scratch buffers
// for the per-chunk partial results; such callers have nowhere to get them from.
//
// What it does: exactly what gllm_attention_decode_bf16 does (same kernels,
// same arguments, same results bit for bit), but the partial results live in
// an array that is compiled into the library's device image, so the caller
// passes only inputs and outputs.  The function calls no cudaMalloc, no
// cudaFree and no library routine that allocates.
//
// Limits and rules:
//  * The array holds GLLM_DECODE_NOALLOC_MAX_FLOATS floats (16 MiB).  Every GPU
//    that loads this library holds that much until the process exits.
//    A call needs  num_queries * hq * num_chunks * (d + 2)  floats;
//    a call that needs more returns cudaErrorInvalidValue (1) and launches nothing.
//  * The device that ``stream`` belongs to must be the current device of the
//    calling thread: the array's address is looked up, and remembered, for the
//    current device.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress).  Make that first call before any stream capture
//    begins.
//  * All calls share the one array and it keeps the previous call's contents.
//    Nothing in it has to start at zero: every entry a call reads was written by
//    that call first.  Two calls whose kernels overlap on the GPU (different
//    streams, or two host threads) race on the array: run them one after the
//    other on one stream.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GLLM_DECODE_NOALLOC_MAX_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as gllm_attention_decode_bf16 without part_o / part_ml:
// query token i is row i of q / out / positions / token_row; cache layer layout
// [page][k|v][kv_head][block_size][d]; num_chunks >= ceil(longest sequence /
// gllm_attention_decode_chunk(d)).  Returns 0 or a cudaError_t.
int gllm_attention_decode_bf16_noalloc(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                       int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                       int bt_stride, const int* positions, const int* token_row, int num_queries,
                                       int hq, int hkv, int d, int block_size, int num_pages, int num_chunks,
                                       float scale, int window, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
