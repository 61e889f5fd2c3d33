// Block-table maintenance: dst[idx[i]] = val[i] for the cells that changed since
// the last step.  The reference rebuilds and re-uploads whole padded tables every
// forward (models/llama/llama_model.cpp:441-456); here the tables live on the
// device and only changed cells travel, riding in the step's metadata copy.
#include "common.cuh"

LSB_DEFINE_STATUS()

__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx,
                                   const int* __restrict__ val, int n, long long dst_size) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int j = idx[i];
    if (j < 0 || j >= dst_size) { lsb_set_status(LSB_BAD_ROW); return; }
    dst[j] = val[i];
}

LSB_API int lsb_scatter_i32(int* dst, const int* idx, const int* val, int n, long long dst_size,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    scatter_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, idx, val, n, dst_size);
    return LSB_LAUNCH_CHECK();
}
