// RMSNorm fused with the residual addition that precedes it.
//
//   residual[t,:] += delta[t,:]                    (32-bit, in place; delta optional)
//   out[t,:] = residual[t,:] * rsqrt(mean(residual[t,:]^2) + eps) * weight
//
// Replaces residual_add_kernel + rms_norm_kernel of the reference
// (kernels/src/residual.cu:11-19, kernels/src/rmsnorm.cu:42-72).  The gathered form
// does the same for selected rows only (the rows whose logits are wanted) and
// leaves the residual stream untouched.  One thread block per row; the row lives
// in registers between the two passes when it fits, else it is re-read.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kNormThreads = 256;
constexpr int kNormRegs = 8;          // rows up to 256*8 = 2048 wide stay in registers

template <typename T, bool GATHER>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                   const int* __restrict__ rows, const float* __restrict__ weight,
                   T* __restrict__ out, int hidden, int n_rows_total, float eps) {
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r_out = blockIdx.x;
    int r_in = r_out;
    if (GATHER) {
        r_in = rows[r_out];
        if (r_in < 0 || r_in >= n_rows_total) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
            for (int i = threadIdx.x; i < hidden; i += blockDim.x)
                out[(size_t)r_out * hidden + i] = lsb_from_float<T>(0.f);
            return;
        }
    }
    float* res = residual + (size_t)r_in * hidden;
    const T* dl = delta ? delta + (size_t)r_in * hidden : nullptr;
    T* o = out + (size_t)r_out * hidden;

    float keep[kNormRegs];
    const bool in_regs = hidden <= kNormThreads * kNormRegs;
    float ss = 0.f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kNormRegs; ++j) {
            const int i = threadIdx.x + j * kNormThreads;
            float x = 0.f;
            if (i < hidden) {
                x = res[i];
                if (dl) x += lsb_to_float(dl[i]);
                if (!GATHER && dl) res[i] = x;
            }
            keep[j] = x;
            ss += x * x;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
            float x = res[i];
            if (dl) x += lsb_to_float(dl[i]);
            if (!GATHER && dl) res[i] = x;
            ss += x * x;
        }
    }
    ss = lsb_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kNormRegs; ++j) {
            const int i = threadIdx.x + j * kNormThreads;
            if (i < hidden) o[i] = lsb_from_float<T>(keep[j] * inv * weight[i]);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
            float x = res[i];
            if (GATHER && dl) x += lsb_to_float(dl[i]);
            o[i] = lsb_from_float<T>(x * inv * weight[i]);
        }
    }
}

// residual: float [rows, hidden] (updated in place when delta is given)
// delta: dtype [rows, hidden] or null; weight: float [hidden]; out: dtype [rows, hidden]
LSB_API int lsb_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out,
                            int dtype, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        add_rmsnorm_kernel<T, false>, dim3(rows), dim3(kNormThreads), 0, stream, 1,
        residual, (const T*)delta, (const int*)nullptr, weight, (T*)out, hidden, rows, eps));
    return 0;
}

// out[i,:] = norm(residual[rows[i],:] + delta[rows[i],:]); residual is not modified.
LSB_API int lsb_gather_add_rmsnorm(const float* residual, const void* delta, const int* rows,
                                   const float* weight, void* out, int dtype, int n_out,
                                   int n_rows_total, int hidden, float eps, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        add_rmsnorm_kernel<T, true>, dim3(n_out), dim3(kNormThreads), 0, stream, 1,
        (float*)residual, (const T*)delta, rows, weight, (T*)out, hidden, n_rows_total, eps));
    return 0;
}
