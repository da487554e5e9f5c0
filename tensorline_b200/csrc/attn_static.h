// tl_attn_decode_static: split-KV paged decode attention that allocates nothing.
//
// This entry point has no counterpart in tzar-beep/Tensorline.  It exists for callers of this
// library that cannot allocate device memory at the point of the call: code that runs inside
// someone else's memory plan (a host runtime that hands out every device byte itself and forbids
// cudaMalloc after start-up), code on a path where an allocation could block or fail at a bad moment
// (a latency-critical serving loop, a signal-safe or real-time thread), and plain C programs that
// link this library without torch and have no allocator at hand.  Such callers pass their inputs
// and the output buffer as always; what the ordinary entry point (tl_attn_decode) takes as two extra
// scratch buffers for the per-range partial results lives here in one fixed array inside the library.
//
// What to know before calling it:
//   * The scratch is a file-scope device array of TL_ATTN_STATIC_SCRATCH_FLOATS floats (4 MiB).
//     Every GPU on which a process loads this library holds those 4 MiB until the process exits.
//   * A call needs B * nq * splits * (head_dim + 2) floats when splits > 1 (none when splits == 1).
//     Larger requests are refused with a message; nothing is launched.  Use fewer splits.
//   * The key ranges must cover the longest context of the call: chunk * splits >= the largest
//     start_pos[b] + 1, rounded up to a multiple of 64 (with a window: the window + 63).  The lengths
//     live on the device, so this entry point cannot check it; keys beyond chunk * splits are not read
//     and the result is then wrong without an error.
//   * The first call on each device (with that device current) looks up the array's device address
//     (cudaGetSymbolAddress) and raises the kernels' shared-memory limit on that device.  Make that
//     first call outside any stream capture; later calls on the device do no set-up.
//   * All calls on a device share the one array, and it keeps whatever the last call left in it.
//     Nothing in it has to start at zero: a call reads only the partials that the same call wrote.
//     Two calls whose kernels overlap on the GPU (different streams, no ordering between them) race
//     on the array and give wrong results; order them on one stream or with events.
//   * It calls no cudaMalloc, cudaFree or any allocating routine, of CUDA or of any library.
//
// Arguments are those of tl_attn_decode without part_o / part_ml (bfloat16 q, pages and out; int32
// tables and per-request arrays, all device pointers), then `err`: a caller-owned host buffer of
// `err_len` bytes that receives a message when the return value is not 0 (may be NULL).
#pragma once
#include <cuda_runtime.h>

#define TL_ATTN_STATIC_SCRATCH_FLOATS (1 << 20)

extern "C" int tl_attn_decode_static(const void* q, int q_stride, void* out, const void* k_pages,
                                     const void* v_pages, const int* table, int max_pages, int page_size,
                                     const int* q_start, const int* start_pos, const int* slots, int B, int nq,
                                     int nkv, int window, float scale, int chunk, int splits,
                                     cudaStream_t stream, char* err, int err_len);
