// What the pieces of a tcgen05 kernel's inner loop cost a warp on sm_100a, one at a time:
//   * how fast one thread can issue tcgen05.mma of a given N (M = 128, K = 16, bfloat16), alone and
//     with a second issuing thread in another warp, and when the last of them completes;
//   * what a warp waits for a single operation to answer, in a loop of nothing else: a try_wait on
//     a barrier whose phase is long complete, a load of 32 columns from tensor memory with its wait,
//     a store of 32 columns with its wait; with 4, 8 and 12 warps doing the same at once (a figure
//     that does not grow with the number of warps is a latency, one that does is a bandwidth).
// One block, every wait bounded, no operand matters (the tiles hold a constant).  Built and run by
// `python -m llm_singularity_b200.measure.probe tc_latency`; a standalone program, not part of the
// engine's libraries.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t it = 0; it < (1u << 24); ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;                                           // gave up: reported as TIMEOUT
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_smem)), "r"(ncols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
#define REGS32(r) "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), \
    "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), \
    "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), \
    "r"(r[30]), "r"(r[31])
#define OUTS32(r) "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), \
    "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), \
    "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), \
    "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : OUTS32(r) : "r"(taddr));
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), REGS32(r) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) {
    uint64_t d = (uint64_t)((smem_addr(tile) >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D 32-bit, A and B bfloat16, both K-major, M = 128
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

enum : int { OP_NONE = 0, OP_TRY_WAIT = 1, OP_TMEM_LD = 2, OP_TMEM_ST = 3 };

// warp 1: first issuer (and tensor-memory allocation); warp 2: second issuer if `second`; warps 4 ..
// 4 + warps_op - 1: the timed operation `op`.  out[0..2]: first issuer's cycles to issue, to
// completion, and whether its wait came through; out[4..6]: the second's; out[8..11]: cycles per
// operation of the first four operation warps.
__global__ void __launch_bounds__(512, 1) tc_latency(int n, int count, int second, int op, int warps_op, long long* out) {
    extern __shared__ unsigned char raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = base;                 // 128 rows x 64 of K
    unsigned char* sB = base + 16384;         // 256 rows x 64 of K
    __shared__ uint64_t bar[2], done_bar;
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(base)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&done_bar)) : "memory");   // its phase 0 is complete
    }
    if (warp == 1) tmem_alloc(&slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = slot;
    auto issue = [&](int which) {
        const uint32_t idesc = make_idesc(n);
        const uint64_t da = desc_kmajor(sA), db = desc_kmajor(sB);
        const uint32_t d = tm + (which ? 256 : 0);
        const long long t0 = clock64();
        for (int i = 0; i < count; ++i)                      // four k-steps into one accumulator, again and again
            umma_bf16(d, da + 2 * (i & 3), db + 2 * (i & 3), idesc, (i & 3) ? 1u : 0u);
        const long long t1 = clock64();
        umma_commit(&bar[which]);
        const bool ok = mbar_wait(&bar[which], 0);
        const long long t2 = clock64();
        out[which * 4 + 0] = t1 - t0;
        out[which * 4 + 1] = t2 - t0;
        out[which * 4 + 2] = ok ? 1 : 0;
    };
    if (warp == 1 && lane == 0) issue(0);
    else if (warp == 2 && lane == 0 && second) issue(1);
    else if (warp >= 4 && warp < 4 + warps_op && op != OP_NONE) {
        uint32_t v[32];
        for (int x = 0; x < 32; ++x) v[x] = x;
        // columns the issuers do not write: [384, 512)
        const uint32_t ta = tm + ((uint32_t)((warp & 3) * 32) << 16) + 384 + (uint32_t)(((warp >> 2) & 1) * 64);
        const int iters = 200;
        uint32_t acc = 0;
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
            if (op == OP_TRY_WAIT) acc += mbar_try_wait(&done_bar, 0) ? 1 : 0;
            else if (op == OP_TMEM_LD) { tmem_ld_32x32(ta, v); tmem_ld_wait(); acc += v[0] + v[31]; }
            else { v[0] = acc; tmem_st_32x32(ta, v); tmem_st_wait(); acc += 1; }
        }
        const long long t1 = clock64();
        if (lane == 0 && warp < 8) out[8 + (warp & 3)] = (t1 - t0) / iters;
        if (acc == 0x12345) out[15] = acc;                   // (keeps the loop)
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tm, 512);
    }
}

static bool run(int n, int count, int second, int op, int warps_op, long long* dev, long long* host) {
    for (int rep = 0; rep < 2; ++rep) {                      // the second run is the one reported
        cudaMemset(dev, 0, 16 * sizeof(long long));
        tc_latency<<<1, 32 * (4 + (warps_op > 0 ? warps_op : 0)), 60000>>>(n, count, second, op, warps_op, dev);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            printf("error: %s\n", cudaGetErrorString(e));
            return false;
        }
        cudaMemcpy(host, dev, 16 * sizeof(long long), cudaMemcpyDeviceToHost);
    }
    return true;
}

int main() {
    long long* dev = nullptr;
    long long h[16];
    if (cudaMalloc(&dev, 16 * sizeof(long long)) != cudaSuccess ||
        cudaFuncSetAttribute(tc_latency, cudaFuncAttributeMaxDynamicSharedMemorySize, 60000) != cudaSuccess) {
        printf("error: no device, or it does not take the kernel\n");
        return 1;
    }
    const int count = 2048;
    printf("tcgen05.mma, M = 128, K = 16, bfloat16, %d in a row from one thread (cycles each; the tensor pipe alone would need N / 2):\n", count);
    for (int n : {64, 128, 256})
        for (int second = 0; second < 2; ++second) {
            if (!run(n, count, second, OP_NONE, 0, dev, h)) return 1;
            printf("  N = %3d, %s: issued in %6.1f, complete after %6.1f%s", n, second ? "two issuing threads" : "one issuing thread ",
                   (double)h[0] / count, (double)h[1] / count, h[2] ? "" : " TIMEOUT");
            if (second) printf(" (the second thread: %6.1f, %6.1f%s)", (double)h[4] / count, (double)h[5] / count, h[6] ? "" : " TIMEOUT");
            printf("\n");
        }
    printf("one operation and its answer, in a loop of nothing else, no products in flight (cycles, the first four warps):\n");
    const char* names[4] = {"", "try_wait on a completed barrier", "tcgen05.ld 32x32b.x32 + wait::ld", "tcgen05.st 32x32b.x32 + wait::st"};
    for (int op = OP_TRY_WAIT; op <= OP_TMEM_ST; ++op)
        for (int warps_op : {4, 8, 12}) {
            if (!run(64, 0, 0, op, warps_op, dev, h)) return 1;
            printf("  %-34s %2d warps: %lld %lld %lld %lld\n", names[op], warps_op, h[8], h[9], h[10], h[11]);
        }
    cudaFree(dev);
    return 0;
}
