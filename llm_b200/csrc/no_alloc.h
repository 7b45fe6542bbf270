// Entry points for callers that must not allocate device memory.
//
// This has no counterpart in the reference project.  It exists for hosts that embed
// these kernels but own all device memory themselves: a runtime that sized one arena
// for weights and cache at start-up and left nothing for anybody else (a later
// cudaMalloc may simply fail there), or a serving loop that cannot afford the
// device-wide synchronisation an allocation may imply.  Such a caller cannot provide
// the split-key scratch buffers that llmk_paged_attention_decode asks for, nor let a
// library routine allocate them.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Most scratch the static variant can use, in floats (4 MiB).  A call needs
// 4096 + n_entries * n_heads * splits * (head_dim + 2) floats.
#define LLMK_DECODE_STATIC_SCRATCH_FLOATS (1 << 20)

// Same computation and arguments as llmk_paged_attention_decode, without its scratch
// pointer: the partial results of the key ranges live in a fixed array inside the library
// (every GPU that loads the library holds those 4 MiB until the process exits).
//
// * Allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
// * The first call on a device looks up the array's device address (once per device, with
//   that device current).  Make that first call before any stream capture.
// * Sizes whose scratch would exceed LLMK_DECODE_STATIC_SCRATCH_FLOATS are refused with a
//   negative return code and a message for llmk_last_error(); nothing is launched.
// * All calls share the one array and it keeps the last call's contents.  Only its first 4096
//   words (arrival counters of the key ranges) have to be zero when a call starts: the array
//   is zero when the library is loaded and every call sets the counters it used back to zero
//   before it ends; the partial results behind them are written before they are read.  Two
//   calls that overlap on the GPU (different streams, no ordering between them) race on the
//   array; order them on one stream or with events.
// Returns 0, a cudaError_t (> 0), or a negative code for refused arguments.
int llmk_paged_attention_decode_static(void* out, long long out_stride, const void* q, long long q_stride,
                                       const void* k_pages, const void* v_pages, const int* block_table,
                                       int table_width, const int* kv_lens, int n_entries, int n_heads, int n_kv,
                                       int head_dim, int page_size, int window, float scale, int splits, int dtype,
                                       cudaStream_t stream);

#ifdef __cplusplus
}
#endif
