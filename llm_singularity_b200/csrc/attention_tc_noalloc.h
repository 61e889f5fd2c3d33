// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for
// hosts of this library that cannot call cudaMalloc at the moment they need
// attention: code running inside a memory pool that owns the whole device,
// real-time loops in which an allocation (and the device-wide synchronisation
// it can imply) is not allowed, or plug-in environments where every buffer has
// to be declared up front.  The regular entry point, lsb_decode_attention,
// expects its caller to bring a scratch buffer for the partial results of the
// key splits; this one keeps that scratch inside the library instead, in a
// fixed device array of lsb_decode_attention_noalloc_max_floats() floats
// (4 MiB) that every GPU loading the library holds until the process exits.
//
// Rules for callers:
//   * Inputs and the output are still the caller's buffers.
//   * With up to 8 splits no scratch is used at all (one split needs none, and
//     2 to 8 splits are merged inside a thread-block cluster), so any size is
//     taken.  With more than 8 splits n_requests * nh * splits * (hd + 2) must
//     not exceed the maximum; larger problems are refused with
//     LSB_NOALLOC_TOO_LARGE and nothing is launched.
//   * The first call with more than 8 splits on each device looks up the
//     array's device address (with that device current).  Make that first call
//     before starting any stream capture, and from one thread.
//   * All calls share the one array, and it keeps whatever the previous call
//     left there.  The kernels write every slot before they read it, so nothing
//     has to be cleared, but two calls that overlap on the GPU (different
//     streams, no ordering between them) race on it: order them.
//   * The function calls no cudaMalloc, cudaFree or allocating library routine.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LSB_NOALLOC_TOO_LARGE (-100)   // scratch needed exceeds the built-in array
#define LSB_NOALLOC_BAD_DEVICE (-101)  // device index outside the table of known devices

// Capacity of the built-in scratch array, in floats.
long long lsb_decode_attention_noalloc_max_floats(void);

// Text for a return code of lsb_decode_attention_noalloc (CUDA codes included).
const char* lsb_decode_attention_noalloc_error(int code);

// Same contract as lsb_decode_attention (single decode tokens, bfloat16, head size 64 or
// 128, nh / nkv <= 16) without the scratch argument.  Returns 0, a CUDA error code, or one
// of the LSB_NOALLOC_* codes.
int lsb_decode_attention_noalloc(const void* qkv, int qkv_stride, const void* k_pages,
                                 const void* v_pages, const int* q_start, const int* kv_len,
                                 const int* table_rows, const int* block_table, int table_stride,
                                 void* out, int n_requests, int nh, int nkv, int hd, int page_size,
                                 int num_pages, float scale, int window, int splits,
                                 cudaStream_t stream);

#ifdef __cplusplus
}
#endif
