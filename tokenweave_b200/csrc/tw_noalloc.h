// Allocation-free entry point. It has no counterpart in the reference.
//
// Who it is for: code that must run single-query paged attention but is not allowed to allocate
// device memory. Examples are a host process that embeds this library next to a framework owning
// all of the GPU's memory through its own pool (a stray cudaMalloc there can fail or fragment the
// pool), a caller running under a memory budget that was fixed at start-up, and latency-critical
// serving loops in which cudaMalloc's implicit synchronisation is unacceptable. The regular entry
// point, tw_attn_decode, expects the caller to hand it a workspace for the split-KV partial results;
// this one brings its own.
//
// How: the partial results live in a fixed array in the library's device data segment
// (TW_NOALLOC_SCRATCH_BYTES, 4 MiB). Every GPU that loads the library holds that array until the
// process exits. The caller still passes all inputs and the output tensor.
//
// Rules for callers:
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and caches it. Make that first call outside of any stream capture.
//  * n_tok * hq * splits * (D + 2) floats must fit in the array; larger requests are rejected with an
//    error (return value 1, message from tw_last_error()), nothing is launched.
//  * All calls on a device share the one array and it keeps the previous call's contents. The kernels
//    write every partial result they later read, so nothing has to be cleared between calls, but two
//    calls whose kernels may overlap on the GPU (different streams) race on it: serialise them.
//  * No cudaMalloc, cudaFree or other allocating routine is called, here or underneath.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#define TW_NOALLOC_SCRATCH_BYTES (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and semantics as tw_attn_decode (tw_kernels.h) without the two workspace pointers.
int tw_attn_decode_noalloc(const void* q, long long ldq, const void* k_cache, const void* v_cache, int page,
                           void* out, long long ldo, const int* tok_row, const int* tok_seq,
                           const int* tok_kvlen, int n_tok, const int* block_table, int max_blocks, int hq,
                           int hkv, int D, float scale, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
