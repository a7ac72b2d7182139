// An entry point that allocates nothing.  It has no counterpart in the reference, which is a
// CPU program and owns all of its memory.
//
// Who needs it.  Some programs that would call this library may not allocate device memory
// while they run: a serving process that handed the whole GPU to a memory pool at start-up
// and has nothing left for cudaMalloc to give; a loop with a latency bound, where an
// allocation may synchronise the device or fail half-way through a request; a plug-in that
// is called from inside another framework's stream and must not touch that framework's
// allocator.  The split decode attention needs scratch memory (partial sums per split and one
// counter per row and key/value head).  `nb_attention_decode` takes that scratch from the
// caller; `nb_attention_decode_static` below takes none and uses an array that is part of the
// library image instead.  It calls no cudaMalloc, cudaFree or any routine that allocates.
//
// Limits and rules:
//  * The array is NB_STATIC_SCRATCH_BYTES long.  Every GPU on which the library is loaded
//    holds it from load until the process exits, used or not.  A call that needs more
//    (rows x heads x splits x (head size + 2) floats, plus rows x key/value heads counters,
//    each part rounded up to 256 bytes) is refused with an error that says how much it asked
//    for; choose fewer splits, or pass scratch of your own to nb_attention_decode.
//  * The first call on a device looks the array's device address up (cudaGetSymbolAddress,
//    with that device current) and remembers it per device.  Make that first call before any
//    stream capture begins.
//  * All calls on a device share the one array.  It keeps whatever the previous call wrote;
//    each call clears the counters (the only part that must start from zero) with a memset on
//    its stream before its kernel.  Two calls whose kernels overlap on the GPU (different
//    streams without an ordering between them) race on the array and give wrong results:
//    order them.
//
// Arguments are those of nb_attention_decode without the three scratch pointers.
#pragma once

#include <cuda_runtime.h>

#define NB_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of the built-in scratch array.
long long nb_attention_decode_static_capacity(void);

// Decode attention over the paged cache with the library's built-in scratch.  Returns 0 or an
// error code; nb_last_error() has the text.
int nb_attention_decode_static(const void* q, int dtype, int q_stride, int q_col,
                               const int* row_slot, const int* row_pos, const void* k_cache,
                               const void* v_cache, const int* block_table, int max_pages,
                               int page, int n_heads, int n_kv_heads, int head_dim, void* out,
                               int out_dtype, int out_stride, float scale, int window, int n_rows,
                               int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
