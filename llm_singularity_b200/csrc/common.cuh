// Shared helpers for the sm_100a kernel libraries.
//
// Every library exports plain C entry points (raw device pointers, sizes, a
// stream) that return 0 or a CUDA error code; the Python side checks shapes and
// dtypes before the call and turns a non-zero return into an exception.  A
// kernel that meets an index it must not follow (a page id outside the pool, a
// token id outside the table) records a code in the library's status word and
// skips the access: it never traps and never reads or writes out of bounds.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LSB_API extern "C" __attribute__((visibility("default")))

enum LsbDtype : int { LSB_F32 = 0, LSB_BF16 = 1 };

// status codes recorded by kernels (first one wins until the host reads it)
enum LsbStatus : int {
    LSB_OK = 0,
    LSB_BAD_PAGE = 1,       // block-table entry outside [0, num_pages)
    LSB_BAD_TOKEN = 2,      // token id outside [0, vocab)
    LSB_BAD_ROW = 3,        // row index outside the tensor
    LSB_WAIT_TIMEOUT = 4,   // a bounded wait on a barrier ran out
};

template <typename T> struct LsbVec;   // 16-byte vectors of T

__device__ __forceinline__ float lsb_to_float(float x) { return x; }
__device__ __forceinline__ float lsb_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T lsb_from_float(float x);
template <> __device__ __forceinline__ float lsb_from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 lsb_from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float lsb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float lsb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a thread block (every thread gets the result). `scratch` holds 33 floats.
__device__ __forceinline__ float lsb_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = lsb_warp_sum(v);
    __syncthreads();                       // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = lsb_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// One status word per library; the host reads and clears it with lsb_take_status().
#define LSB_DEFINE_STATUS()                                                          \
    __device__ int lsb_status_word = 0;                                              \
    __device__ __forceinline__ void lsb_set_status(int code) {                       \
        atomicCAS(&lsb_status_word, 0, code);                                        \
    }                                                                                \
    LSB_API int lsb_take_status(int* out) {                                          \
        int zero = 0;                                                                \
        cudaError_t e = cudaMemcpyFromSymbol(out, lsb_status_word, sizeof(int));     \
        if (e != cudaSuccess) return (int)e;                                         \
        return (int)cudaMemcpyToSymbol(lsb_status_word, &zero, sizeof(int));         \
    }                                                                                \
    LSB_API const char* lsb_error_string(int code) {                                 \
        return cudaGetErrorString((cudaError_t)code);                                \
    }

#define LSB_LAUNCH_CHECK() ((int)cudaGetLastError())

// Programmatic dependent launch.  Every kernel of these libraries is launched with the
// "programmatic stream serialization" attribute: it may become resident while the kernel before
// it in the stream is still running, set itself up, and must call lsb_pdl_wait() before it reads
// or writes anything an earlier kernel of the stream touches (the wait returns once that kernel
// has completed and its writes are visible).  lsb_pdl_launch_dependents() at a kernel's start lets
// the next kernel of the stream do the same.  What this hides is launch latency, block
// scheduling, per-block set-up and, in the matrix products, the first loads of weights.
__device__ __forceinline__ void lsb_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void lsb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#include <stdlib.h>
static inline bool lsb_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("LSB_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the launch attributes above; cluster > 1
// makes that many consecutive blocks one thread-block cluster: along z by default, along x when
// LSB_CLUSTER_ALONG_X is defined before this header is included.
template <typename... KArgs, typename... Args>
static inline int lsb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, int cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (lsb_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
#ifdef LSB_CLUSTER_ALONG_X
        attr[n].val.clusterDim.x = cluster_z;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
#else
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = cluster_z;
#endif
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Calls `body` with `T` bound to the element type named by `dtype`.
#define LSB_DISPATCH_DTYPE(dtype, ...)                                               \
    do {                                                                             \
        if ((dtype) == LSB_F32) { using T = float; __VA_ARGS__; }                    \
        else if ((dtype) == LSB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }      \
        else return (int)cudaErrorInvalidValue;                                      \
    } while (0)
