// SwiGLU on a fused gate/up product whose columns alternate gate_i, up_i:
// out[t, i] = silu(gu[t, 2i]) * gu[t, 2i + 1], silu(g) = g / (1 + exp(-g)), evaluated in 32-bit.
//
// Replaces silu_mul_kernel of the reference (kernels/src/activations.cu:11-21), which
// reads two separate fp32 buffers.  The bfloat16 tensor-core product applies the same formula
// in its epilogue; this kernel serves the 32-bit path and shapes that product does not take.
#include "common.cuh"

LSB_DEFINE_STATUS()

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                              int inter, long long total) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        // out is [tokens, inter] and gate_up [tokens, 2 * inter]: element idx reads 2 idx, 2 idx + 1
        const float g = lsb_to_float(gate_up[2 * idx]);
        const float u = lsb_to_float(gate_up[2 * idx + 1]);
        out[idx] = lsb_from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

LSB_API int lsb_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter,
                       cudaStream_t stream) {
    const long long total = (long long)tokens * inter;
    if (total <= 0) return 0;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(threads), 0, stream, 1,
                                                (const T*)gate_up, (T*)out, inter, total));
    return 0;
}
