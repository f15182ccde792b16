// Decode attention for callers that must not allocate.
//
// This entry point has no counterpart in mirmir-tech/libmir; it exists for embedders of this library.
//
// Who needs it: code that runs where device memory cannot be requested at call time.  Examples are a
// host application that gave the whole GPU to its own arena at start-up and forbids cudaMalloc afterwards
// (a later allocation could fail, or would fragment what the arena owner planned), a callback running
// inside someone else's stream-ordered pipeline where an allocation would synchronise the device, and a
// plug-in loaded into a process whose allocator this library must not bypass.  Such callers can pass
// inputs and outputs they already own, but they have nowhere to take split-attention's scratch from.
//
// What it does: the same split-over-the-keys decode attention as mir_decode_attention_bf16 (one token per
// request over the paged cache, bf16, head_dim 64 or 128), with the partial results of the partitions kept
// in a fixed array that is part of the library's device image instead of in caller-provided scratch.
//
// Limits and rules:
//   * The array holds MIR_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU on which the library is loaded
//     carries these 8 MiB from load until the process exits.  A call needs
//         rows * heads * num_partitions * (head_dim + 2)   floats   (none when num_partitions == 1)
//     and is refused with MIR_BAD_ARGUMENT and a message naming both numbers when that exceeds the array.
//   * The entry point calls no cudaMalloc, cudaFree or allocating library routine.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress with that
//     device current) and keeps it.  Make that first call outside any stream capture.
//   * All calls share the one array and it keeps whatever the previous call left.  Nothing in it has to
//     start at zero: every value the merge step reads was written by the same call's partitions.  Because it
//     is shared, two calls whose kernels can overlap on the GPU (different streams, or the same device from
//     two threads without ordering) race on it; order such calls yourself.
#pragma once
#include <cuda_runtime.h>

#define MIR_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as mir_decode_attention_bf16 without the scratch pair.  Returns 0, or a MirStatus code with
// the text available from mir_last_error().
int mir_decode_attention_bf16_static(const void* q, long long q_stride, void* out, const void* k_pages,
                                     const void* v_pages, const int* block_table, int table_width,
                                     const int* positions, int rows, int page_size, int heads, int kv_heads,
                                     int head_dim, float scale, int window, int partition, int num_partitions,
                                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif
