// out[M, N] = x[M, K] * w[N, K]^T for a handful of rows (M <= 16) and a weight matrix small enough
// to sit in the shared memory of the whole chip: the q/k/v and output projections of a decode step.
//
// Such a product is all latency: a few megabytes of weights, a few rows of activations.  Run on the
// tile kernel (gemm_tc.cu) it needs K split over a cluster and a sum of partial tiles through
// distributed shared memory, and takes 6 us from its predecessor's end to its own, of which the
// weights account for 1 - 2.  Here every block owns N / 148 weight rows and copies ALL of them into
// its shared memory before it waits for the previous kernel (weights depend on nothing), so what is
// left after the wait is: fetch the activations (from L2), a few hundred mma.sync per warp, a sum
// over the block's eight warps through shared memory, one store.  No cluster, no tensor memory, no
// partial tiles outside the block; the summation order is fixed, so results repeat bit for bit.
//
// The eight warps split K; each holds accumulators for the block's rows (one or two 16-row tiles)
// and the batch (one or two 8-column tiles), and copies and waits for its own slice alone.  Operands lie in shared memory row by row with the
// 16-byte chunks of a row XOR-swizzled by the row number, so ldmatrix reads without bank conflicts.
//
// The reference calls cublasSgemm for every projection (kernels/src/cublas_provider.cpp:36-51).
#include "common.cuh"

LSB_DEFINE_STATUS()

typedef __nv_bfloat16 bf16;

constexpr int kThreads = 256, kWarps = 8;
constexpr int kMaxRowTiles = 2;                 // up to 32 weight rows per block
constexpr int kSmemBudget = 200 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                 "{%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Element (row, 16-byte chunk) of a [rows][K] tile whose chunks are swizzled within groups of eight.
__device__ __forceinline__ bf16* at(bf16* base, int K, int row, int chunk) {
    return base + (size_t)row * K + ((chunk ^ (row & 7)) << 3);
}

// NT: 8-column tiles of the batch (M <= 8 * NT).  R: weight rows per block (<= 16 * kMaxRowTiles).
template <int NT, typename TOut>
__global__ void __launch_bounds__(kThreads, 1)
gemm_small_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TOut* __restrict__ out,
                  int M, int N, int K, int R) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sW = reinterpret_cast<bf16*>(smem_raw);                      // [R][K]
    bf16* sX = sW + (size_t)R * K;                                     // [8 * NT][K]
    float* sRed = reinterpret_cast<float*>(sX + (size_t)8 * NT * K);   // [warps][16 * tiles][8 * NT]
    lsb_pdl_launch_dependents();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * R;
    const int rows = min(R, N - n0);
    const int row_tiles = (rows + 15) >> 4;

    // The eight warps split K, and each is on its own until the final sum: it copies its columns of
    // the block's weight rows before the wait on the previous kernel, its columns of the
    // activations after it, and waits for its own copies only.  Which slice of K a warp takes
    // rotates with the block, so that the blocks of the grid, which all want the same few
    // activation rows at the same moment, do not all ask L2 for the same lines at once.
    const int k_steps = K >> 4;
    const int per = (k_steps + kWarps - 1) / kWarps;           // steps of 16 along K per warp
    const int slice = (warp + blockIdx.x) % kWarps;
    const int ks0 = min(slice * per, k_steps), ks1 = min(ks0 + per, k_steps);
    const int c0 = 2 * ks0, nch = 2 * (ks1 - ks0);             // its 16-byte chunks of every row
    for (int idx = lane; idx < rows * nch; idx += 32) {
        const int r = idx / nch, c = c0 + idx - r * nch;
        cp_async16(at(sW, K, r, c), w + (size_t)(n0 + r) * K + (c << 3));
    }
    cp_async_commit();
    for (int idx = lane; idx < (8 * NT - M) * nch; idx += 32) {    // batch rows that do not exist
        const int r = M + idx / nch, c = c0 + idx % nch;
        *reinterpret_cast<uint4*>(at(sX, K, r, c)) = make_uint4(0, 0, 0, 0);
    }

    lsb_pdl_wait();
    for (int idx = lane; idx < M * nch; idx += 32) {
        const int r = idx / nch, c = c0 + idx - r * nch;
        cp_async16(at(sX, K, r, c), x + (size_t)r * K + (c << 3));
    }
    cp_async_commit();
    cp_async_wait_all();
    __syncwarp();

    float acc[kMaxRowTiles][NT][4];
#pragma unroll
    for (int rt = 0; rt < kMaxRowTiles; ++rt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[rt][nt][0] = acc[rt][nt][1] = acc[rt][nt][2] = acc[rt][nt][3] = 0.f;

    // ldmatrix row addresses: A tiles (16 x 16): lanes 0-7 rows 0-7 / 8-15 rows 8-15 of the first
    // eight columns, lanes 16-31 the same rows of the next eight; B tiles (8 batch rows x 16)
    const int a_row = ((lane >> 3) & 1) * 8 + (lane & 7), a_half = lane >> 4;
    const int b_row = lane & 7, b_half = (lane >> 3) & 1;
    for (int ks = ks0; ks < ks1; ++ks) {
        uint32_t b[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) ldmatrix_x2(b[nt], at(sX, K, nt * 8 + b_row, 2 * ks + b_half));
#pragma unroll
        for (int rt = 0; rt < kMaxRowTiles; ++rt) {
            if (rt < row_tiles) {
                uint32_t a[4];
                ldmatrix_x4(a, at(sW, K, min(rt * 16 + a_row, rows - 1), 2 * ks + a_half));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16(acc[rt][nt], a, b[nt][0], b[nt][1]);
            }
        }
    }

    // sum over the warps in warp order (a fixed order for every output), then one store per output
    const int width = 8 * NT, height = 16 * row_tiles;
    float* mine = sRed + (size_t)warp * 16 * kMaxRowTiles * width;
#pragma unroll
    for (int rt = 0; rt < kMaxRowTiles; ++rt) {
        if (rt < row_tiles) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int r = rt * 16 + (lane >> 2), c = nt * 8 + 2 * (lane & 3);
                mine[r * width + c] = acc[rt][nt][0];
                mine[r * width + c + 1] = acc[rt][nt][1];
                mine[(r + 8) * width + c] = acc[rt][nt][2];
                mine[(r + 8) * width + c + 1] = acc[rt][nt][3];
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < M * height; idx += kThreads) {
        const int m = idx / height, r = idx - m * height;
        if (r >= rows) continue;
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < kWarps; ++wi) v += sRed[((size_t)wi * 16 * kMaxRowTiles + r) * width + m];
        out[(size_t)m * N + n0 + r] = lsb_from_float<TOut>(v);
    }
}

// Weight rows per block for N rows in all, and whether the kernel takes the product at all:
// bfloat16, M <= 16, K a multiple of 64 (the swizzle works on groups of eight 16-byte chunks), at
// most 32 rows per block when the rows are dealt over the SMs, and everything within shared memory.
static int plan_rows(int M, int N, int K, int sms, size_t* smem) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 64) return 0;
    const int R = (N + sms - 1) / sms;
    if (R > 16 * kMaxRowTiles) return 0;
    const int nt = M <= 8 ? 1 : 2;
    const size_t bytes = (size_t)R * K * 2 + (size_t)8 * nt * K * 2 +
                         (size_t)kWarps * 16 * kMaxRowTiles * 8 * nt * sizeof(float);
    if (bytes > (size_t)kSmemBudget) return 0;
    *smem = bytes;
    return R;
}

static int sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
}

LSB_API int lsb_gemm_small_supported(const void* x, const void* w, int M, int N, int K) {
    size_t smem;
    return ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && plan_rows(M, N, K, sm_count(), &smem) > 0;
}

template <int NT, typename TOut>
static int launch(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, int R, size_t smem,
                  cudaStream_t stream) {
    static int configured = -1;
    if (configured < 0)
        configured = (int)cudaFuncSetAttribute(gemm_small_kernel<NT, TOut>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (configured) return configured;
    return lsb_launch(gemm_small_kernel<NT, TOut>, dim3((N + R - 1) / R), dim3(kThreads), smem, stream, 1, x, w,
                      out, M, N, K, R);
}

// x [M, K] and w [N, K] bfloat16, out [M, N] bfloat16 or (out_f32) float.
LSB_API int lsb_gemm_small(const void* x, const void* w, void* out, int out_f32, int M, int N, int K,
                           cudaStream_t stream) {
    size_t smem = 0;
    if (!lsb_gemm_small_supported(x, w, M, N, K)) return (int)cudaErrorInvalidValue;
    const int R = plan_rows(M, N, K, sm_count(), &smem);
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (M <= 8)
        return out_f32 ? launch<1, float>(xp, wp, (float*)out, M, N, K, R, smem, stream)
                       : launch<1, bf16>(xp, wp, (bf16*)out, M, N, K, R, smem, stream);
    return out_f32 ? launch<2, float>(xp, wp, (float*)out, M, N, K, R, smem, stream)
                   : launch<2, bf16>(xp, wp, (bf16*)out, M, N, K, R, smem, stream);
}
