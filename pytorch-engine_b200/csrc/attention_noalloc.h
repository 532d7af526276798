// pe_attention_decode_noalloc: decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in binief/pytorch-engine.  It exists for users of this library
// whose code runs where cudaMalloc is off limits: a plug-in inside a host application that owns all
// device memory and hands out fixed buffers, a real-time loop that must not touch the allocator, or
// any caller that wants one C function it can call with its own input and output buffers and nothing
// else.  The ordinary decode entry point (pe_attention_generic with decode = 1) needs a scratch
// buffer for the partial results of the key ranges; here that scratch lives inside the library, in a
// fixed array in device memory, so the caller passes inputs and outputs only.
//
// Limits and rules
//   * The array holds PE_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  It is part of the library image:
//     every GPU on which the library is used keeps those 8 MiB until the process exits.
//   * A call needs n_seqs * n_heads * max_splits * (head_dim + 1) floats.  A call that needs more
//     is refused with PE_ERR_SCRATCH_TOO_LARGE and launches nothing.
//   * Every sequence must fit its ranges: seq_past[b] + 1 <= split_keys * max_splits.  The lengths live on
//     the device, so the host cannot check this before the launch; the kernel does.  For a longer sequence
//     it sets the status word (code 3: sequence index, last position, the limit), reads nothing outside the
//     array and writes the attention over the first split_keys * max_splits keys only.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per
//     device, with that device current).  Make that first call outside any stream capture.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing has to be
//     cleared between calls: every element that the merge step reads is written earlier in the same
//     call.  Two calls that overlap on the GPU (different streams, or different host threads with
//     streams of their own) would write the same array and race; run them one after the other.
//
// Arguments and result are those of pe_attention_generic in its decode form, without `scratch`:
// one query token per sequence (row seq_qstart[b] of q), keys and values from the paged cache,
// seq_past[b] tokens already cached before this one, ranges of `split_keys` keys (a multiple of 32),
// `max_splits` ranges at most per sequence.  Returns 0, a negative PE_ERR_* code, or a positive CUDA
// runtime error number.
#pragma once
#include <cuda_runtime.h>

#define PE_NOALLOC_SCRATCH_FLOATS (1 << 21)
#define PE_ERR_SCRATCH_TOO_LARGE (-6)

#ifdef __cplusplus
extern "C" {
#endif

int pe_attention_decode_noalloc(int dtype, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs,
                                int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                const int* seq_qstart, const int* seq_past, const int* seq_slot, const int* page_table,
                                int table_stride, int num_pages, const void* k_pages, const void* v_pages,
                                int split_keys, int max_splits, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
