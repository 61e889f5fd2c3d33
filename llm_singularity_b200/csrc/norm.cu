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

// The same with four elements per thread and step (hidden a multiple of 4, 16-byte aligned
// rows): 16-byte loads of the residual and the weight, 8- or 16-byte loads of the delta.
constexpr int kVecRegs = 4;           // rows up to 256*4*4 = 4096 wide stay in registers

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T, bool GATHER>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_vec4_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                        const int* __restrict__ rows, const float* __restrict__ weight,
                        T* __restrict__ out, int hidden, int n_rows_total, float eps) {
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    const int nvec = hidden >> 2;
    const bool in_regs = nvec <= kNormThreads * kVecRegs;
    // the norm's weight does not depend on the kernel before: it is on its way while that one
    // finishes, instead of costing a second round trip to L2 after the sum of squares
    float4 wv[kVecRegs];
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kVecRegs; ++j) {
            const int v = threadIdx.x + j * kNormThreads;
            wv[j] = v < nvec ? Vec4<float>::load(weight + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
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
    float4 keep[kVecRegs];
    float ss = 0.f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kVecRegs; ++j) {
            const int v = threadIdx.x + j * kNormThreads;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (v < nvec) {
                x = Vec4<float>::load(res + 4 * v);
                if (dl) {
                    const float4 d = Vec4<T>::load(dl + 4 * v);
                    x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
                    if (!GATHER) Vec4<float>::store(res + 4 * v, x);
                }
            }
            keep[j] = x;
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
    } else {
        for (int v = threadIdx.x; v < nvec; v += kNormThreads) {
            float4 x = Vec4<float>::load(res + 4 * v);
            if (dl) {
                const float4 d = Vec4<T>::load(dl + 4 * v);
                x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
                if (!GATHER) Vec4<float>::store(res + 4 * v, x);
            }
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
    }
    ss = lsb_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kVecRegs; ++j) {
            const int v = threadIdx.x + j * kNormThreads;
            if (v < nvec) {
                const float4 w = wv[j];
                const float4 x = keep[j];
                Vec4<T>::store(o + 4 * v, make_float4(x.x * inv * w.x, x.y * inv * w.y, x.z * inv * w.z, x.w * inv * w.w));
            }
        }
    } else {
        for (int v = threadIdx.x; v < nvec; v += kNormThreads) {
            float4 x = Vec4<float>::load(res + 4 * v);
            if (GATHER && dl) {
                const float4 d = Vec4<T>::load(dl + 4 * v);
                x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
            }
            const float4 w = Vec4<float>::load(weight + 4 * v);
            Vec4<T>::store(o + 4 * v, make_float4(x.x * inv * w.x, x.y * inv * w.y, x.z * inv * w.z, x.w * inv * w.w));
        }
    }
}

static inline bool vec4_ok(const void* a, const void* b, const void* c, const void* d, int hidden) {
    return hidden % 4 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0 &&
           ((uintptr_t)c % 16) == 0 && ((uintptr_t)d % 16) == 0;
}

// residual: float [rows, hidden] (updated in place when delta is given)
// delta: dtype [rows, hidden] or null; weight: float [hidden]; out: dtype [rows, hidden]
LSB_API int lsb_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out,
                            int dtype, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vec4_ok(residual, delta, weight, out, hidden))
        LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
            add_rmsnorm_vec4_kernel<T, false>, dim3(rows), dim3(kNormThreads), 0, stream, 1,
            residual, (const T*)delta, (const int*)nullptr, weight, (T*)out, hidden, rows, eps));
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
    if (vec4_ok(residual, delta, weight, out, hidden))
        LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
            add_rmsnorm_vec4_kernel<T, true>, dim3(n_out), dim3(kNormThreads), 0, stream, 1,
            (float*)residual, (const T*)delta, rows, weight, (T*)out, hidden, n_rows_total, eps));
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        add_rmsnorm_kernel<T, true>, dim3(n_out), dim3(kNormThreads), 0, stream, 1,
        (float*)residual, (const T*)delta, rows, weight, (T*)out, hidden, n_rows_total, eps));
    return 0;
}

// The second half of a norm that a product folded in (gemm_stream.cu): values[m, :] holds a
// residual row times the norm's weight, parts[p * 16 + m] the parts of the row's sum of squares;
// out[m, :] = values[m, :] * rsqrt(sum / hidden + eps).  For a consumer that cannot scale its own
// rows; one block per row, parts added in index order within a lane, then across lanes.
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
finish_norm_kernel(const T* __restrict__ values, const float* __restrict__ parts, int n_parts,
                   T* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int m = blockIdx.x;
    float t = 0.f;
    for (int p = threadIdx.x; p < n_parts; p += kNormThreads) t += parts[p * 16 + m];
    t = lsb_block_sum(t, scratch);
    const float inv = rsqrtf(t / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += kNormThreads)
        out[(size_t)m * hidden + i] = lsb_from_float<T>(lsb_to_float(values[(size_t)m * hidden + i]) * inv);
}

LSB_API int lsb_finish_norm(const void* values, const float* parts, int n_parts, void* out, int dtype,
                            int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (rows > 16 || n_parts <= 0) return (int)cudaErrorInvalidValue;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(finish_norm_kernel<T>, dim3(rows), dim3(kNormThreads), 0, stream, 1,
                                                (const T*)values, parts, n_parts, (T*)out, hidden, eps));
    return 0;
}
