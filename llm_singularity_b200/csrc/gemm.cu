// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores, 32-bit accumulation, no reduced-precision
// matrix mode: the product of the true 32-bit path, and of any shape the tensor-core
// kernel does not take.  A and W are row-major with K contiguous, the layout checkpoints
// store ([out, in]) and the reference hands to cublasSgemm
// (kernels/src/cublas_provider.cpp:36-51).  Inputs 32-bit or bfloat16; output 32-bit or
// the input type.  64x64 output tile per block, 16-deep slices of K staged through shared
// memory, 4x4 outputs per thread.  The summation order over K is fixed by K alone, so a
// row's result does not depend on M or on where the row sits in the batch.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kGemmThreads = (BM / TM) * (BN / TN);      // 256

template <typename TIn>
__device__ __forceinline__ void load4(const TIn* __restrict__ base, long long row, int rows,
                                      int k0, int K, long long ld, bool vec_ok, float (&v)[4]) {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (row >= rows) return;
    const TIn* p = base + row * ld + k0;
    if (vec_ok && k0 + 3 < K) {
        if constexpr (sizeof(TIn) == 4) {
            const float4 f = *reinterpret_cast<const float4*>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            const uint2 raw = *reinterpret_cast<const uint2*>(p);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (k0 + j < K) v[j] = lsb_to_float(p[j]);
    }
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kGemmThreads)
gemm_nt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ W, TOut* __restrict__ C,
               int M, int N, int K, long long lda, long long ldw, long long ldc, bool vec_ok) {
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Ws[BK][BN + 4];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int tid = threadIdx.x;
    const int ty = tid / (BN / TN), tx = tid % (BN / TN);
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    const int lrow = tid / (BK / 4), lk = (tid % (BK / 4)) * 4;   // 64 rows x 4 quads

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4], w[4];
        load4<TIn>(A, m0 + lrow, M, k0 + lk, K, lda, vec_ok, a);
        load4<TIn>(W, n0 + lrow, N, k0 + lk, K, ldw, vec_ok, w);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 4; ++j) { As[lk + j][lrow] = a[j]; Ws[lk + j][lrow] = w[j]; }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * TM]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * TN]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const long long n = n0 + tx * TN + j;
            if (n < N) C[m * ldc + n] = lsb_from_float<TOut>(acc[i][j]);
        }
    }
}

// in_dtype: element type of A and W; out_dtype: element type of C (LSB_F32 or in_dtype).
LSB_API int lsb_gemm_nt(const void* A, const void* W, void* C, int in_dtype, int out_dtype,
                        int M, int N, int K, long long lda, long long ldw, long long ldc,
                        cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    const int esize = in_dtype == LSB_F32 ? 4 : 2;
    const bool vec_ok = ((uintptr_t)A % (4 * esize) == 0) && ((uintptr_t)W % (4 * esize) == 0) &&
                        lda % 4 == 0 && ldw % 4 == 0;
    const dim3 block(kGemmThreads);
    if (in_dtype == LSB_F32 && out_dtype == LSB_F32)
        return lsb_launch(gemm_nt_kernel<float, float>, grid, block, 0, stream, 1, (const float*)A,
                          (const float*)W, (float*)C, M, N, K, lda, ldw, ldc, vec_ok);
    if (in_dtype == LSB_BF16 && out_dtype == LSB_BF16)
        return lsb_launch(gemm_nt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, 1,
                          (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K,
                          lda, ldw, ldc, vec_ok);
    if (in_dtype == LSB_BF16 && out_dtype == LSB_F32)
        return lsb_launch(gemm_nt_kernel<__nv_bfloat16, float>, grid, block, 0, stream, 1,
                          (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (float*)C, M, N, K, lda, ldw,
                          ldc, vec_ok);
    return (int)cudaErrorInvalidValue;
}
