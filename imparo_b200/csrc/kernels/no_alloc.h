// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in zeraix/imparo: the reference always works out of buffers its
// own backend allocated.  It exists here for hosts that embed the attention kernel and
// cannot hand it scratch memory or let it ask for some:
//   * code running while a stream is being captured into a CUDA graph, where cudaMalloc is
//     not permitted;
//   * serving loops with a latency budget, where an allocation may serialise the whole
//     device behind it;
//   * hosts whose device memory is fully partitioned up front by an allocator of their own,
//     so that a library asking the driver for more would fail or break their accounting.
//
// imparo_paged_attention_split_static does what imparo_paged_attention_split does (split-key
// attention for single query tokens over the paged cache, then an ordered combine) but keeps
// its scratch (the per-split partial results) in a fixed array that is part of the library
// image, instead of taking two scratch pointers.  It calls no cudaMalloc, cudaFree or any
// routine that allocates.
//
// Limits and rules
//   * The array holds IMPARO_STATIC_SCRATCH_FLOATS floats (8 MiB).  A call needs
//     n_tok * nh * n_splits * (hd + 2) floats; a call that needs more is refused with
//     IMPARO_ERR_STATIC_SCRATCH_TOO_SMALL and launches nothing.  Every GPU that loads the
//     library carries the 8 MiB until the process exits.
//   * The first call on a device resolves the array's device address (cudaGetSymbolAddress,
//     with that device current).  Make that first call outside any stream capture.
//   * All calls on a device share the one array, and it keeps what the last call left.
//     Nothing in it has to be zero: every slot a call reads it has written itself first
//     (unused splits are marked, not skipped).  Two calls that overlap on the GPU — different
//     streams, or graph branches that may run concurrently — would overwrite each other's
//     partials: run them one after the other.
//   * Inputs and outputs are the caller's, exactly as for imparo_paged_attention_split.
//   * chunk * n_splits must be at least max_blocks * page_size (every position the block table
//     can hold lies in some chunk; fewer splits would drop keys), and n_splits at most 2048 (the
//     combine kernel keeps one pair per split in shared memory).  Both are checked, with the
//     head size, the head counts and n_tok <= 65535, before the scratch need is computed and
//     before anything is launched; a call that breaks one returns -2 (-3, -5 for the heads).
#pragma once
#include <cuda_runtime.h>

#define IMPARO_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define IMPARO_ERR_STATIC_SCRATCH_TOO_SMALL (-30)
#define IMPARO_ERR_STATIC_SCRATCH_ADDRESS (-31)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, a negative refusal code (see above; -3 head size, -5 head counts, -8 group size
// above 8, -2 grid limits), or a positive cudaError_t.
int imparo_paged_attention_split_static(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                        const int* positions, const int* item_of_token,
                                        const int* table, int max_blocks, int page_size, int n_pages,
                                        int window, float scale, void* out,
                                        int n_tok, int nh, int nkv, int hd, int chunk, int n_splits,
                                        int* status, cudaStream_t stream);

// How many floats of the fixed array a call with these sizes needs.
long long imparo_paged_attention_split_static_need(int n_tok, int nh, int hd, int n_splits);

#ifdef __cplusplus
}
#endif
