// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the upstream project: upstream allocates
// every buffer once at start-up with cudaMalloc and its attention kernels need no
// scratch at all.  It exists for hosts of this library that cannot call cudaMalloc
// at the moment they need attention: code running inside a memory pool it does not
// own, a plug-in whose host application has handed the whole device to its own
// allocator, a real-time loop where an allocation's implicit synchronisation is
// not acceptable.  Such a caller still brings its inputs and its output; only the
// scratch that the split kernel needs between its two launches comes from here.
//
// The scratch is one file-scope `static __device__` array inside attention.so,
// KVB_DECODE_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which the
// library is loaded carries that array until the process ends, whether or not
// this function is ever called.
//
// Rules of use
//   * Sizes: the call needs R * nq * NB * (d + 2) floats of scratch, NB being the
//     number of key blocks.  If that exceeds the array the call does nothing and
//     returns KVB_ERR_SCRATCH_TOO_SMALL (-4); kvb_decode_attention_noalloc_error
//     turns a return code into text.  All other size rules are those of
//     kvb_decode_attention (head size 32, 64 or 128; group size 1..8; KB a multiple
//     of 128).
//   * First call on a device: the address of the array on the current device is
//     looked up then (cudaGetSymbolAddress) and remembered for that device.  Make
//     this first call on each device before any stream capture begins, with that
//     device current.
//   * Every call on a device shares the one array.  Two calls whose kernels can
//     overlap on the GPU (different streams, no ordering between them) race on it;
//     calls on one stream, or ordered by events, are safe.
//   * The array keeps whatever the last call left in it.  Nothing in it has to start
//     at zero: a call writes every partial result it later reads.
//   * No cudaMalloc, cudaFree or other allocating routine is called, here or in the
//     kernels it launches.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVB_DECODE_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)
#define KVB_ERR_SCRATCH_TOO_SMALL (-4)
#define KVB_ERR_SCRATCH_SETUP (-5)

// Same meaning of every argument as kvb_decode_attention, without part_o / part_ml.
// One query token per request r: its row in q is q_start[r], its position ctx_len[r]-1.
// Returns 0, a negative KVB_ERR_* code, or a positive cudaError_t.
int kvb_decode_attention_noalloc(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                 const int* block_table, int max_pages, int page_size, int num_pages,
                                 const int* q_start, const int* ctx_len, void* out, int R, int nq, int nkv,
                                 int d, float scale, int window, int KB, int NB, int dtype, int* status,
                                 cudaStream_t stream);

// Floats of scratch a call with these sizes needs.
unsigned long long kvb_decode_attention_noalloc_scratch_needed(int R, int nq, int NB, int d);

// A sentence for a return code of kvb_decode_attention_noalloc.
const char* kvb_decode_attention_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
