// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts that embed
// the kernel library without a device allocator of their own.  Examples: a C or C++ program that
// loads librl_attention_decode.so directly and owns a fixed arena it will not grow; a serving loop
// that forbids cudaMalloc after start-up because an allocation synchronises the whole device and
// stalls every stream; code that runs where the CUDA runtime refuses to allocate at all.
//
// `rl_attn_decode` needs the caller to pass scratch memory for the partial results of its key
// splits.  `rl_attn_decode_static` computes exactly the same thing but keeps that scratch in a
// fixed array inside the library, so the caller passes only inputs and the output.
//
//   * The array holds RL_ATTN_DECODE_STATIC_FLOATS floats (4 MiB).  Every GPU on which this
//     library is loaded carries those 4 MiB from load until the process exits.
//   * A call needs n_seqs * H * n_splits * (hd + 2) floats.  A call that needs more is refused
//     with a negative return code and a message in rl_error_text(); nothing is launched.
//   * The first call on each device looks up the array's device address (once, with that device
//     current).  Make that first call outside of any stream capture.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in
//     it.  Nothing in it has to start at zero: a call writes every element before it reads it.
//     Because the array is shared, two calls that run on the GPU at the same time (different
//     streams, or different host threads) overwrite each other's partial results: run them one
//     after the other.
//   * The function calls no cudaMalloc, no cudaFree and no library routine that allocates.
//
// Arguments are those of rl_attn_decode without `part_o` and `part_ml`; the return value follows
// the library's convention (0, a positive cudaError_t, or a negative refusal code).
#pragma once

#include <cuda_runtime.h>

#define RL_ATTN_DECODE_STATIC_FLOATS (1u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int rl_attn_decode_static(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages,
                          const int* block_table, int table_width, const int* seq_len, void* out, int out_stride,
                          int n_seqs, int H, int K, int hd, int page_size, int window, float scale, int n_splits,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
