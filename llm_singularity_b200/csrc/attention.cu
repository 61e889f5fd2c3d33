// Causal attention over the paged cache, generic form: any mix of prompt portions and
// single decode tokens, any head size that is a multiple of 16 up to 256, any number of
// heads and groups, 32-bit or bfloat16 storage; all arithmetic in 32-bit.
//
// For request r with q_len = q_start[r+1] - q_start[r] new tokens and kv_len tokens in
// the cache after this step, query row i sits at position p = kv_len - q_len + i and
// sees keys at positions [max(0, p - window + 1), p] (window == 0: from 0).  Query
// head h reads kv head h / (nh / nkv).  Scores (q.k) * scale, softmax by running
// maximum and sum, weighted sum of values, division by the sum at the end.
//
// Two score modifiers that other architectures use are taken here (the reference has neither;
// the tensor-core kernels do not take them, so a mixer that asks for one runs this kernel):
// a soft cap, s <- cap * tanh(s / cap), and a linear position bias per head,
// s <- s - slope[h] * (p - key position), applied in that order before the softmax.
//
// Replaces paged_attention_kernel of the reference (kernels/src/attention.cu:27-172:
// 32 threads per (head, row), per-thread v_acc[128] in registers, shared-memory tree
// merge, one launch per request during prefill, models/llama/llama_model.cpp:603-614).
// Here one warp owns a (row, head): lanes split the keys of a 32-key chunk for the
// scores and split the head dims for the weighted sum; one launch covers all requests.
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

constexpr int kAttnWarps = 4;
constexpr int kMaxHeadDim = 256;

// dot of q (shared, float) with one key row (global, 16-byte vector loads)
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q,
                                                const float* __restrict__ k, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + d);
        s += q[d] * kv.x + q[d + 1] * kv.y + q[d + 2] * kv.z + q[d + 3] * kv.w;
    }
    return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            s += q[d + 2 * j] * f.x + q[d + 2 * j + 1] * f.y;
        }
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(kAttnWarps * 32)
paged_attention_generic_kernel(
    const T* __restrict__ qkv, int qkv_stride,              // q of token t at qkv + t*stride
    const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
    const int* __restrict__ table_rows, const int* __restrict__ block_table, int table_stride,
    T* __restrict__ out,                                    // [tokens, nh*hd]
    int nh, int nkv, int hd, int page_size, int num_pages, float scale, int window,
    float softcap, const float* __restrict__ slopes) {
    __shared__ float q_sh[kAttnWarps][kMaxHeadDim];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.z, h = blockIdx.y;
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int i = blockIdx.x * kAttnWarps + warp;            // row within the request
    if (i >= q_len) return;                                  // whole warp leaves together
    const int kv_len = kv_len_arr[r];
    const int p = kv_len - q_len + i;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int g = h / (nh / nkv);
    const int t = qs + i;
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;
    const float slope = slopes ? slopes[h] : 0.f;

    const T* q = qkv + (size_t)t * qkv_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) q_sh[warp][d] = lsb_to_float(q[d]) * scale;
    __syncwarp();

    constexpr int kAccs = kMaxHeadDim / 32;
    float acc[kAccs];
#pragma unroll
    for (int c = 0; c < kAccs; ++c) acc[c] = 0.f;
    float m = -FLT_MAX, l = 0.f;

    for (int base = lo; base <= p; base += 32) {
        const int kj = base + lane;
        float s = -FLT_MAX;
        long long off = -1;                                  // element offset of the key/value row
        if (kj <= p) {
            const int page = bt[kj / page_size];
            if (page < 0 || page >= num_pages) {
                lsb_set_status(LSB_BAD_PAGE);
            } else {
                off = (((long long)page * nkv + g) * page_size + (kj % page_size)) * hd;
                s = dot_row<T>(q_sh[warp], k_pages + off, hd);
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
                s -= slope * (float)(p - kj);
            }
        }
        const float m_new = fmaxf(m, lsb_warp_max(s));
        const float corr = expf(m - m_new);                // m == -FLT_MAX first: exp(-huge) = 0
        const float pj = (off >= 0) ? expf(s - m_new) : 0.f;
        l = l * corr + lsb_warp_sum(pj);
#pragma unroll
        for (int c = 0; c < kAccs; ++c) acc[c] *= corr;
        const int n_valid = min(32, p - base + 1);
        for (int j = 0; j < n_valid; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const long long voff = __shfl_sync(0xffffffffu, off, j);
            if (voff < 0) continue;
            const T* v = v_pages + voff;
#pragma unroll
            for (int c = 0; c < kAccs; ++c) {
                const int d = lane + 32 * c;
                if (d < hd) acc[c] += w * lsb_to_float(v[d]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + (size_t)t * nh * hd + (size_t)h * hd;
#pragma unroll
    for (int c = 0; c < kAccs; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) o[d] = lsb_from_float<T>(acc[c] * inv);
    }
}

// qkv: [tokens, qkv_stride] with the nh*hd query values first in each row.  softcap: 0 for none;
// slopes: float [nh] or null.
LSB_API int lsb_paged_attention_generic(
    const void* qkv, int qkv_stride, const void* k_pages, const void* v_pages,
    const int* q_start, const int* kv_len, const int* table_rows, const int* block_table,
    int table_stride, void* out, int dtype, int n_requests, int max_q_len,
    int nh, int nkv, int hd, int page_size, int num_pages, float scale, int window,
    float softcap, const float* slopes, cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (hd % 16 || hd <= 0 || hd > kMaxHeadDim || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
    if (n_requests > 65535 || nh > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((max_q_len + kAttnWarps - 1) / kAttnWarps, nh, n_requests);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        paged_attention_generic_kernel<T>, grid, dim3(kAttnWarps * 32), 0, stream, 1,
        (const T*)qkv, qkv_stride, (const T*)k_pages, (const T*)v_pages, q_start, kv_len,
        table_rows, block_table, table_stride, (T*)out, nh, nkv, hd, page_size, num_pages,
        scale, window, softcap, slopes));
    return 0;
}
