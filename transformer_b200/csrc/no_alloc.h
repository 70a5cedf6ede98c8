// An attention entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference project: it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is not an option -- inside a region that must not
// touch the allocator (a latency-critical loop whose memory was fixed at start-up, a host program
// that owns all device memory itself and hands out none, a plug-in loaded into a process whose
// allocator it must not disturb).  Such a caller can still pass its inputs and outputs, but the
// split-key attention kernel also needs scratch memory for the partial results of the key slices.
// tb_attention_split_static keeps that scratch inside the library: a fixed array in device memory
// (TB_STATIC_SCRATCH_BYTES, 8 MiB) that every GPU which loads the library holds until the process
// exits.  The entry point never calls cudaMalloc, cudaFree or any routine that allocates.
//
// Rules for the caller:
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current).  Make that first call outside any stream capture.
//  * A problem whose partial results do not fit, nt * nh * splits * (dh + 2) floats > the array, is
//    refused with TB_ERR_TOO_LARGE; nothing is launched.
//  * All calls share the one array, and it keeps what the last call left in it.  The kernel writes
//    every partial result before the merge step reads it, so nothing has to be cleared between
//    calls; but two calls that run on the GPU at the same time (different streams) race on it.
//    Serialise them.
//  * With splits == 1 no scratch is used at all.
#pragma once
#include <cuda_runtime.h>

#define TB_STATIC_SCRATCH_BYTES (8u << 20)
#define TB_ERR_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif
// Same arguments and results as tb_attention_f32 / tb_attention_bf16 without the `partial`
// pointer; is_bf16 selects the storage type of q, out and the cache (0 = float, 1 = bfloat16).
// Returns 0, a negative TB_ERR_* code, or a cudaError_t.
int tb_attention_split_static(const void* q, void* out, const void* kc, const void* vc, const int* tile_seq,
                              const int* tile_t0, const int* tile_nq, const int* tok_pos, const int* page_table,
                              int tiles, int nt, int max_pages, int q_stride, int nh, int nkvh, int dh, int splits,
                              float scale, int is_bf16, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
