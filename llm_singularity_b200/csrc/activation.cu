// The activation of a gated feed-forward on a fused gate/up product whose columns alternate
// gate_i, up_i: out[t, i] = act(gu[t, 2i]) * gu[t, 2i + 1], evaluated in 32-bit.  act: silu(g) =
// g / (1 + exp(-g)); gelu in its tanh form, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)));
// or none (gate * up).
//
// Replaces silu_mul_kernel of the reference (kernels/src/activations.cu:11-21), which
// reads two separate fp32 buffers and knows silu only.  The bfloat16 tensor-core product applies
// the same formulas in its epilogue; this kernel serves the 32-bit path and shapes that product
// does not take.
#include "common.cuh"

LSB_DEFINE_STATUS()

enum : int { LSB_ACT_SILU = 1, LSB_ACT_GELU_TANH = 2, LSB_ACT_NONE = 3 };

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                                 int inter, long long total, int act) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        // out is [tokens, inter] and gate_up [tokens, 2 * inter]: element idx reads 2 idx, 2 idx + 1
        const float g = lsb_to_float(gate_up[2 * idx]);
        const float u = lsb_to_float(gate_up[2 * idx + 1]);
        float a;
        if (act == LSB_ACT_SILU) a = g / (1.f + expf(-g));
        else if (act == LSB_ACT_GELU_TANH)
            a = 0.5f * g * (1.f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
        else a = g;
        out[idx] = lsb_from_float<T>(a * u);
    }
}

LSB_API int lsb_gated_act(const void* gate_up, void* out, int dtype, int tokens, int inter, int act,
                          cudaStream_t stream) {
    const long long total = (long long)tokens * inter;
    if (total <= 0) return 0;
    if (act < LSB_ACT_SILU || act > LSB_ACT_NONE) return (int)cudaErrorInvalidValue;
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return (int)err;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > (long long)sms * 32) blocks = (long long)sms * 32;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(gated_act_kernel<T>, dim3((int)blocks), dim3(threads), 0, stream, 1,
                                                (const T*)gate_up, (T*)out, inter, total, act));
    return 0;
}
