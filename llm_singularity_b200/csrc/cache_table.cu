// Block-table maintenance: dst[idx[i]] = val[i] for the cells that changed since
// the last step.  The reference rebuilds and re-uploads whole padded tables every
// forward (models/llama/llama_model.cpp:441-456); here the tables live on the
// device and only changed cells travel, riding in the step's metadata copy.
#include "common.cuh"

LSB_DEFINE_STATUS()

__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx,
                                   const int* __restrict__ val, int n, long long dst_size) {
    // No early launch of what follows: kernels later in the step read the block table before their
    // own wait on their predecessor (the decode attention starts its first copies there), so
    // nothing of the step may start until the table is whole.  The next kernel starts when this
    // one has completed.
    lsb_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int j = idx[i];
    if (j < 0 || j >= dst_size) { lsb_set_status(LSB_BAD_ROW); return; }
    dst[j] = val[i];
}

LSB_API int lsb_scatter_i32(int* dst, const int* idx, const int* val, int n, long long dst_size,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    return lsb_launch(scatter_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 1, dst, idx, val, n,
                      dst_size);
}

// The same with the count on the device: packed = [n, idx[cap], val[cap]].  A captured graph can
// hold this launch and still apply a different number of changes at every replay.
__global__ void scatter_i32_counted_kernel(int* __restrict__ dst, const int* __restrict__ packed,
                                           int cap, long long dst_size) {
    lsb_pdl_wait();              // as above: what follows starts when the table is whole
    int n = packed[0];
    if (n > cap) { if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW); n = cap; }
    const int* idx = packed + 1;
    const int* val = packed + 1 + cap;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int j = idx[i];
        if (j < 0 || j >= dst_size) { lsb_set_status(LSB_BAD_ROW); continue; }
        dst[j] = val[i];
    }
}

LSB_API int lsb_scatter_i32_counted(int* dst, const int* packed, int cap, long long dst_size,
                                    cudaStream_t stream) {
    if (cap <= 0) return 0;
    return lsb_launch(scatter_i32_counted_kernel, dim3(1), dim3(256), 0, stream, 1, dst, packed, cap, dst_size);
}

// dst[dst_idx[i]] = src[src_idx[i]]: the tokens a step sampled on the device become input tokens
// of the next step, which may hold the requests in another order and other tokens beside them.
__global__ void move_i32_kernel(int* __restrict__ dst, const int* __restrict__ dst_idx,
                                const int* __restrict__ src, const int* __restrict__ src_idx, int n,
                                long long dst_size, long long src_size) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int a = dst_idx[i], b = src_idx[i];
    if (a < 0 || a >= dst_size || b < 0 || b >= src_size) { lsb_set_status(LSB_BAD_ROW); return; }
    dst[a] = src[b];
}

LSB_API int lsb_move_i32(int* dst, const int* dst_idx, const int* src, const int* src_idx, int n,
                         long long dst_size, long long src_size, cudaStream_t stream) {
    if (n <= 0) return 0;
    return lsb_launch(move_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 1, dst, dst_idx, src,
                      src_idx, n, dst_size, src_size);
}
