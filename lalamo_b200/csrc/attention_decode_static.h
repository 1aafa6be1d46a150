// lb_attention_decode_static: split-key paged attention for callers that must not allocate.
// This entry point has no counterpart in the reference.
//
// Who needs it.  lb_attention_decode wants a scratch buffer from its caller.  A caller may be unable
// to provide one: it runs where a call into an allocator is forbidden or unsafe (inside another
// program's capture of a stream, on a thread that must not block on allocator or driver locks, in a
// plug-in without a memory budget of its own).  Here the scratch is a fixed 16 MiB array inside the
// library's device image instead; the caller passes only inputs and outputs.  The entry point calls
// no cudaMalloc, cudaFree or other allocating routine.
//
// Limits and rules.
//  * tokens * num_heads * splits * (head_dim + 2) must not exceed 4,194,304 floats; beyond that the
//    call returns -4 and, if a buffer is given, writes a message saying so.  Other sizes are those
//    of lb_attention_decode (head_dim a multiple of 16 up to 128, page_size a multiple of 16): -2.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and, like the first call of lb_attention_decode on a device, raises the
//    kernel's shared-memory limit there (cudaFuncSetAttribute).  Both happen once per device, under a
//    lock.  Make that first call before any stream capture starts.
//  * All calls on a device share the one array.  Calls that overlap on the GPU (different streams, or
//    graphs replayed side by side) race on it; order them on one stream or with events.  The array
//    keeps the last call's partial results; nothing in it has to be cleared between calls.
//  * Every GPU that loads the library holds the 16 MiB until the process exits.
//
// Arguments are those of lb_attention_decode without `scratch`, plus an optional buffer for an error
// message.  Returns 0, -2, -4, or a CUDA error code.
#pragma once

#include <cuda_runtime.h>

extern "C" int lb_attention_decode_static(const void* q, const void* k_pages, const void* v_pages, void* out, const int* positions,
                                          const int* token_segment, const int* block_table, const int* token_list, int tokens,
                                          int num_heads, int num_groups, int head_dim, int page_size, int num_pages, int max_blocks,
                                          float scale, int window, int splits, int blocks_per_split, int* status, cudaStream_t stream,
                                          char* error_message, int error_capacity);
