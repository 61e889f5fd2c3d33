// Token embedding gather: out[t, :] = float(table[ids[t], :]).
//
// Replaces the reference's embedding_lookup_kernel (kernels/src/embedding.cu:12-26),
// which copies fp32 rows; here the table is in the compute dtype and the rows are
// widened into the 32-bit residual stream.  One thread block per token.
#include "common.cuh"

LSB_DEFINE_STATUS()

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_TOKEN);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = lsb_to_float(row[i]);
}

LSB_API int lsb_embedding(const void* table, int dtype, const int* ids, float* out,
                          int tokens, int hidden, int vocab, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    int threads = hidden < 256 ? ((hidden + 31) / 32) * 32 : 256;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(embedding_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 1,
                                                (const T*)table, ids, out, hidden, vocab));
    return 0;
}
