// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in nassor/cuca; it exists for this library's own users.
//
// Who needs it: code that runs where cudaMalloc is off limits. Examples are a plugin called inside another
// program's CUDA graph capture (allocation is not allowed while a stream is capturing), a real-time loop that
// may not take the allocator's lock, or a host whose memory is handed out by a pool it does not control. The
// ordinary entry point, cuca_attention_decode, asks its caller for a scratch buffer and arrival counters that
// somebody had to allocate. This one brings its own: a fixed array that lives inside the library's device
// image.
//
// What it costs: every GPU that loads the library holds CUCA_NOALLOC_SCRATCH_BYTES (4 MiB + 16 KiB) of device
// memory until the process exits, whether or not this function is ever called.
//
// Limits: the split partials must fit the array, i.e.
//     n_rows * nh * n_splits * (d + 2) <= CUCA_NOALLOC_PART_FLOATS   and   n_rows * nkv <= CUCA_NOALLOC_COUNTERS;
// a larger problem is refused with an error (return code 1, text from cuca_last_error()); nothing is launched.
//
// Rules of use:
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that device
//    current. Make that first call outside any stream capture; later calls only launch kernels and a memset.
//  * All calls share the one array, and it keeps what the last call left in it. The counters are cleared on the
//    caller's stream before each launch; the partials need no clearing (each is written before it is read).
//  * Because the array is shared, two calls that overlap on the GPU (different streams, or graphs replayed
//    concurrently) race on it. Keep calls on one stream, or order them with events.
//  * Inputs and outputs are still the caller's: q, out, the key/value pools and the tables are passed as in
//    cuca_attention_decode and have the same meaning.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#define CUCA_NOALLOC_PART_FLOATS (1u << 20)
#define CUCA_NOALLOC_COUNTERS 4096u
#define CUCA_NOALLOC_SCRATCH_BYTES (CUCA_NOALLOC_COUNTERS * 4u + CUCA_NOALLOC_PART_FLOATS * 4u)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as cuca_attention_decode, minus `part` and `counters`.
// Returns 0 on success; 1 if the problem does not fit the built-in scratch or the shape is unsupported;
// 2 if the address lookup or a launch failed.
int cuca_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* kpool,
                                  const void* vpool, int n_blocks, int bs, const int* positions,
                                  const int* seq_of_row, const int* tables, int table_stride, const int* rows,
                                  int n_rows, int nh, int nkv, int d, float scale, int window, int chunk,
                                  int n_splits, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
