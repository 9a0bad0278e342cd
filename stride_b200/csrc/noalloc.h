// Declaration of the one entry point of this library that allocates no memory.
// It has no counterpart in arhaamatiq/stride: that engine allocates all its buffers itself at start-up
// and has no callers that are barred from allocating.
//
// Who needs it: code that runs inside a process whose device memory is already spoken for. A host
// application may have handed the whole GPU to its own arena (another runtime's memory pool, a fixed
// partition under a memory budget), so that a cudaMalloc made on its behalf by a helper library either
// fails or eats into a reserve the host counted on; and a latency-bound serving loop cannot afford
// cudaMalloc or cudaFree at all, because both may synchronise the whole device. Such a caller can still
// run decode attention over its own paged cache with this call: it passes inputs and outputs, and the
// scratch the kernels need between their two passes lives in a fixed array inside the library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// Capacity of the built-in scratch in floats (16 MiB). A call needs
// entries * kv_heads * chunks * 16 * (head_dim + 2) floats, e.g. 32 entries x 8 heads x 8 chunks
// (contexts up to 2,048 tokens) at head_dim 64 need 2.2 M floats. Larger steps are refused.
#define SB_NOALLOC_SCRATCH_FLOATS (4ll * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Decode attention (every entry brings at most 16 / (Hq / Hkv) tokens) over a paged bfloat16 cache, with
// the same arguments and the same result as sb_attention_tc given n_tiles = 0 and a scratch buffer;
// `items` lists the entries (columns of `meta`) to run. Returns 0, or non-zero with a message in
// sb_last_error(); a step that needs more scratch than SB_NOALLOC_SCRATCH_FLOATS is refused before
// anything is launched.
//
// * It calls neither cudaMalloc nor cudaFree nor any routine that allocates. The scratch is a
//   `static __device__` array of this library; every GPU that loads the library holds its 16 MiB until
//   the process exits.
// * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//   device current) and keeps it; make that first call on each device during set-up, before any stream
//   capture is begun.
// * All calls share the one array, and it keeps what the last call left. Nothing in it has to start
//   at zero: the first pass writes every record that the second pass of the same call reads. But two
//   calls that overlap on the GPU (different streams, or one stream per thread) race on it; keep
//   calls on one stream or order them yourself.
int sb_attention_decode_noalloc(const void* q, void* out, const void* k_base, const int32_t* block_table, int max_pages,
                                int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                                const int32_t* meta, int meta_stride, const int32_t* items, int n_items, int chunks,
                                int Hq, int Hkv, int D, int window, float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
