// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library
// whose code runs where cudaMalloc is off limits: a plug-in that is handed its tensors by a
// host runtime and owns no allocator, or a service loop that may not stall on the
// device-wide synchronisation an allocation can cause.  Such callers still pass the inputs
// and the output; what they cannot provide is the kernel's scratch space (the split-K partial
// results), so that space lives inside the library, in a fixed array in device memory that
// every GPU loading the library holds until the process exits
// (HB_NOALLOC_SCRATCH_FLOATS floats = 8 MiB).
//
// Rules of use:
//  * The arguments mean what they mean for hb_attention_decode (api.h), minus `scratch`.
//  * A call whose batch x heads x splits x (head size + 2) exceeds HB_NOALLOC_SCRATCH_FLOATS is
//    refused with an error; nothing runs.
//  * The first call on each device looks up the array's device address (with that device
//    current) before launching.  Make that first call outside any stream capture.
//  * All calls share the one array.  Nothing in it needs to be zero: every call overwrites
//    what it later reads.  Two calls that may run on the GPU at the same time (different
//    streams, no dependency between them) would overwrite each other's partial results:
//    order them.
//  * The function calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once

#define HB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int hb_attention_decode_noalloc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                const int* page_table, int pt_width, const int* positions, void* out,
                                long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
                                float scale, int window, int splits, int max_pages, int n_pages, void* stream);

#ifdef __cplusplus
}
#endif
