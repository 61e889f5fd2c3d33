// Causal attention for prompt portions on the 5th-generation tensor cores (bfloat16, head 64/128).
//
// One thread block per (128-query tile, head, request).  Per 64-key tile of the request's cache:
//   S = Q K^T      tcgen05.mma, Q and K tiles in shared memory (K-major, 128-byte swizzle, written by
//                  TMA: Q straight from the fused qkv activations, K and V page by page through the
//                  block table from a 4-D tensor map over the page pool), S in TMEM (64 fp32 columns)
//   softmax        four warps, one query row per thread (a row is one TMEM lane, so maximum and sum
//                  need no shuffles): tcgen05.ld, scale, mask, exp2 on the SFU, running max / sum in
//                  32-bit, P rounded to bfloat16 and written to shared memory in the same swizzled
//                  K-major layout
//   O += P V       tcgen05.mma again (V is the MN-major operand: dims contiguous, keys strided),
//                  accumulating in TMEM (HD columns) over all tiles; the softmax warps rescale O only
//                  when a row's maximum has outgrown its reference by 2^8, and read it once at the end
// Warp 0 issues the TMA loads (one lane per page of the tile), warp 1 issues the MMAs and owns the
// TMEM allocation, warps 2-5 do the softmax and the final store.  Three blocks fit per SM (head 64),
// so one block's softmax overlaps the others' matrix products.  All mbarrier waits are bounded.
//
// Query row i of a request with q_len new tokens and kv_len cached tokens sits at position
// p = kv_len - q_len + i and sees keys [max(0, p - window + 1), p].  This kernel takes what the
// reference's paged_attention_kernel (kernels/src/attention.cu:27-172) does one row at a time during
// prefill (models/llama/llama_model.cpp:599-615).  No load in this file uses cluster multicast.
#include "common.cuh"

#include <cuda.h>

LSB_DEFINE_STATUS()

typedef __nv_bfloat16 bf16;

constexpr int kRows = 128;            // queries per block = TMEM lanes
constexpr int kKeys = 64;             // keys per tile
constexpr int kThreads = 224;        // warps: TMA, MMA for S, four softmax warps, MMA for P V
constexpr int kKvStages = 4;          // K/V tiles in flight
constexpr int kBlocksPerSm64 = 2;     // blocks of head size 64 that share an SM (head 128: one)
constexpr int kBtCache = 512;         // block-table entries of this block's key range kept in smem
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kSpinLimit = 1u << 22;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u) {
            if (*abort_flag) return false;
            __nanosleep(128);
        }
    }
    *abort_flag = 1;
    lsb_set_status(LSB_WAIT_TIMEOUT);
    return false;
}
// Is the phase complete?  Never blocks.
__device__ __forceinline__ uint32_t mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok;
}
// A warp waits through its first lane and arrives through it: thirty-two lanes on one barrier are
// thirty-two operations on one shared-memory word.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return ok != 0;
}
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
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
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (rows on lanes, two bfloat16 per 32-bit column).
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The larger of three; two 32-bit floats in a 64-bit register, and a multiply-add and a sum on
// both at once (sm_100: half the instructions of a row's exponents and sums).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) {
    uint64_t d = (uint64_t)((smem_addr(tile) >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand (the contiguous direction is N, here the head dims of V): 64 dims = one 128-byte
// row, rows are consecutive keys (K), groups of 8 keys 1024 bytes apart (stride byte offset), the
// next 64 dims `lbo_bytes` further (leading byte offset).  Same shared-memory image as above.
__device__ __forceinline__ uint64_t desc_mnmajor(const void* tile, uint32_t lbo_bytes) {
    uint64_t d = (uint64_t)((smem_addr(tile) >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D fp32, A and B bf16, M = 128; b_mn = 1 puts B in MN-major form (bit 16)
__host__ __device__ constexpr uint32_t make_idesc(int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(kRows >> 4) << 24);
}

struct AttnParams {
    const int* q_start;
    const int* kv_len;
    const int* table_rows;
    const int* block_table;
    int table_stride;
    bf16* out;
    int nh, nkv, page_size, page_shift, num_pages;
    float scale;
    int window;
    int skip_single;              // requests with one new token are left to the decode kernel
};

template <int HD>
struct Smem {
    static constexpr int kKB = HD / 64;                     // 64-dim blocks of a head
    static constexpr int kQBytes = kRows * HD * 2;
    static constexpr int kKVBytes = kKeys * HD * 2;         // one of K or V, one stage
    static constexpr size_t kTotal = 1024 + kQBytes + 2 * kKvStages * kKVBytes +
                                     kBtCache * 4 + 20 * 8 + 16;
};

template <int HD>
__global__ void __launch_bounds__(kThreads, HD == 64 ? kBlocksPerSm64 : 1)
prefill_attention_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const AttnParams prm) {
    using L = Smem<HD>;
    constexpr int KB = L::kKB;
    // tensor memory: S twice (kKeys columns of 32-bit scores each: even and odd tiles), P twice
    // (kKeys / 2 columns each: two bfloat16 per column), the O tile (HD columns)
    constexpr uint32_t kTmemCols = (3 * kKeys + HD) <= 128 ? 128 : (3 * kKeys + HD) <= 256 ? 256 : 512;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;                                // [KB][128 rows][128 B]
    unsigned char* sK = sQ + L::kQBytes;                     // [stages][KB][128 keys][128 B]
    unsigned char* sV = sK + kKvStages * L::kKVBytes;        // [stages][KB][128 keys][128 B]
    int* sBT = reinterpret_cast<int*>(sV + kKvStages * L::kKVBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sBT + kBtCache);
    uint64_t* q_full = bars;                                 // TMA -> MMA
    uint64_t* kv_full = bars + 1;                            // [stages] TMA -> MMA
    uint64_t* kv_empty = kv_full + kKvStages;                // [stages] MMA -> TMA
    uint64_t* s_full = kv_empty + kKvStages;                 // [2] MMA -> softmax: S of an even / odd tile
    // P of even and of odd tiles has a barrier each: a softmax warp may be a whole tile ahead of
    // another (S of the next tile comes early), and its arrival for tile t + 1 must not count
    // towards tile t, whose P a slower warp has yet to write.  Two tiles ahead it cannot be: P of
    // tile t + 2 waits for the P V product of tile t, which waits for every warp's P of tile t.
    uint64_t* p_full = s_full + 2;                           // [2] softmax -> MMA (an arrival a warp)
    uint64_t* o_full = p_full + 2;                           // [2] MMA -> softmax: P V of an even / odd tile landed
    uint64_t* s_free = o_full + 2;                           // [2] softmax -> MMA: S is in registers (an arrival a warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
    __shared__ int abort_flag;

    lsb_pdl_launch_dependents();
    // What follows up to the wait needs nothing from the kernel before: the step's metadata is on
    // the device before the step's first kernel starts; barriers and tensor memory are this block's.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, r = blockIdx.z;
    const int qs = prm.q_start[r];
    const int q_len = prm.q_start[r + 1] - qs;
    const int n_qt = (q_len + kRows - 1) / kRows;
    if ((int)blockIdx.y >= n_qt || (prm.skip_single && q_len == 1)) return;   // before any barrier
    const int i0 = (n_qt - 1 - (int)blockIdx.y) * kRows;     // heavy tiles first
    const int g = h / (prm.nh / prm.nkv);
    const int kv_len = prm.kv_len[r];
    const int p0 = kv_len - q_len + i0;
    const int rows = min(kRows, q_len - i0);
    const int p_last = p0 + rows - 1;
    const int lo_cta = (prm.window > 0 && p0 - prm.window + 1 > 0) ? p0 - prm.window + 1 : 0;
    const int t0 = lo_cta / kKeys, t1 = p_last / kKeys + 1;
    const int* bt = prm.block_table + (size_t)prm.table_rows[r] * prm.table_stride;
    const int pages_per_tile = kKeys >> prm.page_shift;
    const int page_first = (t0 * kKeys) >> prm.page_shift;
    const int page_last = p_last >> prm.page_shift;          // last page that holds a needed key
    const int n_pages_here = page_last - page_first + 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < kKvStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(&p_full[0], 4);
        mbar_init(&p_full[1], 4);
        mbar_init(&o_full[0], 1);
        mbar_init(&o_full[1], 1);
        mbar_init(&s_free[0], 4);
        mbar_init(&s_free[1], 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    lsb_pdl_wait();
    // this block's slice of the block table (pages outside the pool are caught here)
    // Pages that lie wholly before the first key any row of this block may see (a window has passed
    // them) may have been given back already: their keys are masked, any page stands in for them.
    const int page_needed = lo_cta >> prm.page_shift;
    for (int idx = threadIdx.x; idx < min(n_pages_here, kBtCache); idx += kThreads) {
        int page = (page_first + idx < prm.table_stride) ? bt[page_first + idx] : -1;
        if (page < 0 || page >= prm.num_pages) {
            if (page_first + idx >= page_needed) lsb_set_status(LSB_BAD_PAGE);
            page = 0;
        }
        sBT[idx] = page;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = *tmem_slot;                      // S of even tiles, then of odd tiles
    const uint32_t tmem_p = tmem_s + 2 * kKeys;              // P of even tiles, then of odd tiles
    const uint32_t tmem_o = tmem_s + 3 * kKeys;              // O tile
    const int n_tiles = t1 - t0;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
            mbar_expect_tx(q_full, L::kQBytes);
            for (int kb = 0; kb < KB; ++kb)
                tma_load_2d(sQ + kb * (kRows * 128), &map_q, q_full, h * HD + kb * 64, qs + i0);
        }
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int s = t % kKvStages;
            if (t >= kKvStages) {
                if (lane == 0) ok = mbar_wait(&kv_empty[s], (uint32_t)((t / kKvStages) - 1) & 1, &abort_flag);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
            }
            if (lane == 0) mbar_expect_tx(&kv_full[s], 2 * L::kKVBytes);
            __syncwarp();
            if (lane < pages_per_tile) {
                // pages past the last needed one repeat it: their keys are masked, their bytes finite
                int pi = (((t0 + t) * kKeys) >> prm.page_shift) + lane;
                if (pi > page_last) pi = page_last;
                const int idx = pi - page_first;
                int page;
                if (idx < kBtCache) page = sBT[idx];
                else {
                    page = pi < prm.table_stride ? bt[pi] : -1;
                    if (page < 0 || page >= prm.num_pages) {
                        if (pi >= page_needed) lsb_set_status(LSB_BAD_PAGE);
                        page = 0;
                    }
                }
                const int row_off = lane * prm.page_size * 128;    // bytes into a 64-dim block
                for (int kb = 0; kb < KB; ++kb) {
                    tma_load_4d(sK + s * L::kKVBytes + kb * (kKeys * 128) + row_off, &map_k, &kv_full[s], kb * 64, 0, g, page);
                    tma_load_4d(sV + s * L::kKVBytes + kb * (kKeys * 128) + row_off, &map_v, &kv_full[s], kb * 64, 0, g, page);
                }
            }
        }
        // copies in flight must land before the block may exit
        if (lane == 0) {
            int dummy = 0;
            mbar_wait(q_full, 0, &dummy);
            for (int t = max(0, n_tiles - kKvStages); t < n_tiles; ++t)
                mbar_wait(&kv_full[t % kKvStages], (uint32_t)(t / kKvStages) & 1, &dummy);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kKeys, 0);
            bool ok = mbar_wait(q_full, 0, &abort_flag);
            // S has two buffers: S of tile t + 2 is issued as soon as the softmax warps hold S of
            // tile t in registers, so a tile's scores are complete long before they are wanted and
            // the softmax warps can ask for them early (see there).
            // Descriptors are formed once: the issuer shares its scheduler with busy softmax warps
            // and gets few issue slots, so every instruction saved per tile shortens the wait for S.
            uint64_t da_q[KB], db_k0[KB];
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                da_q[kb] = desc_kmajor(sQ + kb * (kRows * 128));
                db_k0[kb] = desc_kmajor(sK + kb * (kKeys * 128));
            }
            auto issue_s = [&](int t) {
                const uint64_t stage = (uint64_t)((t % kKvStages) * (L::kKVBytes >> 4));    // address field: bytes / 16
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_s + (uint32_t)((t & 1) * kKeys), da_q[kb] + 2 * k, db_k0[kb] + stage + 2 * k,
                                  idesc_qk, (kb | k) ? 1u : 0u);
                }
                umma_commit(&s_full[t & 1]);
            };
            for (int t = 0; t < n_tiles && ok; ++t) {
                ok = mbar_wait(&kv_full[t % kKvStages], (uint32_t)(t / kKvStages) & 1, &abort_flag);
                if (!ok) break;
                if (t >= 2) {                                  // this buffer's last S is in registers
                    ok = mbar_wait(&s_free[t & 1], (uint32_t)((t >> 1) - 1) & 1, &abort_flag);
                    if (!ok) break;
                }
                tc_fence_after();
                issue_s(t);
            }
        }
    } else if (warp == 6) {
        // ---------------------------------------------------------------- MMA issuer for O += P V
        // A thread of its own: issuing one of these small MMAs takes the better part of a hundred
        // cycles, and behind the S products of the other issuer every tile would wait for both.
        if (lane == 0) {
            constexpr uint32_t idesc_pv = make_idesc(HD, 1);
            const uint64_t db_v0 = desc_mnmajor(sV, kKeys * 128);
            bool ok = true;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int s = t % kKvStages;
                // P of this tile (and O rescaled where a row's reference maximum moved)
                ok = mbar_wait(&p_full[t & 1], (uint32_t)(t >> 1) & 1, &abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t db = db_v0 + (uint64_t)(s * (L::kKVBytes >> 4));
                const uint32_t pa = tmem_p + (uint32_t)((t & 1) * (kKeys / 2));
#pragma unroll
                for (int j = 0; j < kKeys / 16; ++j)           // 16 keys per MMA: eight columns of P, 16 rows of V
                    umma_bf16_ts(tmem_o, pa + j * 8, db + (uint64_t)(j * ((16 * 128) >> 4)), idesc_pv, (t | j) ? 1u : 0u);
                umma_commit(&o_full[t & 1]);
                // K of this stage was read by the S product that this P descends from
                umma_commit(&kv_empty[s]);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax, one row per thread
        const int q = warp & 3;
        const int il = q * 32 + lane;
        const int pos = p0 + il;
        const bool live = il < rows;
        const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
        const float sc = prm.scale * kLog2e;
        // m is the reference maximum of the exponents (log2 domain), l the sum of 2^(s - m).  O
        // accumulates in TMEM over all tiles; it is rescaled only when a row's maximum has grown
        // by more than kRescale since its reference was set, so most tiles never touch O here.
        // (softmax is invariant to the shift; with a stale reference the probabilities stay below
        // 2^kRescale, well inside bfloat16 and the 32-bit sums.)
        constexpr float kRescale = 8.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        // A wait on a barrier that is long complete, a load from tensor memory and a store to it
        // each take the warp about a hundred cycles from issue to result when nothing else runs
        // (107, 88 and 77: measure/tc_latency.cu), and several times that in this loop, beside the
        // other block's warps and the products' traffic (clock stamps in a copy of this kernel: 300
        // to 500 cycles for a wait on a barrier that was complete when it was asked).  A tile's chain
        // of them (two waits, a load, a store) was as long as its exponentials.  So the warp asks
        // early and looks late: whether the P buffer is free is asked before the maxima and looked at after
        // them; whether the next S is complete is asked before the exponentials, and if it is, its
        // load is issued behind the store of P, under the wait for that store.
        uint32_t v[kKeys];
        bool loaded = false;                                   // S of tile t is on its way to v already
        for (int t = 0; t < n_tiles && ok; ++t) {
            if (!loaded) {
                ok = warp_wait(&s_full[t & 1], (uint32_t)(t >> 1) & 1, &abort_flag, lane);
                if (!ok) break;
#pragma unroll
                for (int c0 = 0; c0 < kKeys; c0 += 32)
                    tmem_ld_32x32(tmem_s + lane_sel + (uint32_t)((t & 1) * kKeys + c0),
                                  *reinterpret_cast<uint32_t(*)[32]>(&v[c0]));
            }
            const int key0 = (t0 + t) * kKeys;
            const bool full = key0 + kKeys - 1 <= p0 && rows == kRows &&
                              (prm.window <= 0 || key0 > p_last - prm.window);
            // this tile's P buffer was read by the P V of the tile before the previous one
            uint32_t p_free = 1;
            if (t > 1 && lane == 0) p_free = mbar_test(&o_full[t & 1], (uint32_t)((t >> 1) - 1) & 1);
            // S of this row: kKeys values, read from TMEM once.  Tiles wholly below the diagonal (the
            // common case) skip the key tests; partial maxima / sums are independent so that a warp
            // with a scheduler to itself still finds instructions to issue.
            tmem_ld_wait();
            warp_arrive(&s_free[t & 1], lane);                 // S of the tile after the next may overwrite this one
            // columns of this tile the row may see: [c_lo, c_hi]
            const int c_hi = full ? kKeys - 1 : (live ? pos - key0 : -1);
            const int c_lo = (full || prm.window <= 0) ? 0 : pos - prm.window + 1 - key0;
            float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (full) {
#pragma unroll
                for (int x = 0; x < kKeys; x += 2)
                    mxa[(x >> 1) & 3] = max3(mxa[(x >> 1) & 3], __uint_as_float(v[x]), __uint_as_float(v[x + 1]));
            } else {
#pragma unroll
                for (int x = 0; x < kKeys; ++x) {
                    const float sv = (x <= c_hi && x >= c_lo) ? __uint_as_float(v[x]) : -INFINITY;
                    v[x] = __float_as_uint(sv);
                    mxa[x & 3] = fmaxf(mxa[x & 3], sv);
                }
            }
            const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * sc;      // sc > 0
            // move the reference only when needed
            float corr = 1.f;
            bool moved = false;
            if (mx > m + kRescale || (m == -INFINITY && mx > -INFINITY)) {
                corr = (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
                moved = m != -INFINITY;                        // nothing accumulated before: nothing to scale
                m = mx;
                l *= corr;
            }
            const float mref = (m == -INFINITY) ? 0.f : m;
            if (__shfl_sync(0xffffffffu, p_free, 0)) {
                tc_fence_after();
            } else {
                ok = warp_wait(&o_full[t & 1], (uint32_t)((t >> 1) - 1) & 1, &abort_flag, lane);
                if (!ok) break;
            }
            if (t > 0 && __any_sync(0xffffffffu, moved)) {
                // O *= corr for this warp's 32 rows; the P V of the previous tile must have landed
                ok = warp_wait(&o_full[(t - 1) & 1], (uint32_t)((t - 1) >> 1) & 1, &abort_flag, lane);
                if (!ok) break;
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld_32x32(tmem_o + lane_sel + c0, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int x = 0; x < 32; ++x) ov[x] = __float_as_uint(__uint_as_float(ov[x]) * corr);
                    tmem_st_32x32(tmem_o + lane_sel + c0, ov);
                }
                tmem_st_wait();
            }
            uint32_t s_next = 0;
            if (t + 1 < n_tiles && lane == 0) s_next = mbar_test(&s_full[(t + 1) & 1], (uint32_t)((t + 1) >> 1) & 1);
            // probabilities (masked scores are -inf: 2^-inf = 0), rounded to bfloat16, two to a
            // 32-bit column
            uint64_t la[4] = {0ull, 0ull, 0ull, 0ull};         // pairs of partial sums
            const uint64_t sc2 = pack2(sc, sc), mref2 = pack2(-mref, -mref);
            uint32_t pw[kKeys / 2];
#pragma unroll
            for (int x = 0; x < kKeys; x += 2) {
                float ea, eb;
                unpack2(fma2(pack2(__uint_as_float(v[x]), __uint_as_float(v[x + 1])), sc2, mref2), ea, eb);
                const float pa = fast_exp2(ea), pb = fast_exp2(eb);
                la[(x >> 1) & 3] = add2(la[(x >> 1) & 3], pack2(pa, pb));
                __nv_bfloat162 hb = __floats2bfloat162_rn(pa, pb);
                pw[x >> 1] = *reinterpret_cast<uint32_t*>(&hb);
            }
            {
                float s0, s1;
                unpack2(add2(add2(la[0], la[1]), add2(la[2], la[3])), s0, s1);
                l += s0 + s1;
            }
            // P stays in tensor memory: the P V product takes it from there as its A operand
#pragma unroll
            for (int c0 = 0; c0 < kKeys / 2; c0 += 32)
                tmem_st_32x32(tmem_p + lane_sel + (uint32_t)((t & 1) * (kKeys / 2) + c0),
                              *reinterpret_cast<uint32_t(*)[32]>(&pw[c0]));
            loaded = __shfl_sync(0xffffffffu, s_next, 0) != 0;
            if (loaded) {
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < kKeys; c0 += 32)
                    tmem_ld_32x32(tmem_s + lane_sel + (uint32_t)(((t + 1) & 1) * kKeys + c0),
                                  *reinterpret_cast<uint32_t(*)[32]>(&v[c0]));
            }
            tmem_st_wait();
            warp_arrive(&p_full[t & 1], lane);
        }
        // all tiles issued: the last P V closes the accumulator
        if (ok) {
            ok = warp_wait(&o_full[(n_tiles - 1) & 1], (uint32_t)((n_tiles - 1) >> 1) & 1, &abort_flag, lane);
        }
        if (ok) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = prm.out + (size_t)(qs + i0 + il) * prm.nh * HD + (size_t)h * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_o + lane_sel + c0, v);      // the whole warp reads, live rows store
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int y = 0; y < 4; ++y) {
                            __nv_bfloat162 hb = __floats2bfloat162_rn(__uint_as_float(v[d + 2 * y]) * inv,
                                                                      __uint_as_float(v[d + 2 * y + 1]) * inv);
                            w[y] = *reinterpret_cast<uint32_t*>(&hb);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + d) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_s, kTmemCols);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

static int encode(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return (int)cudaErrorNotSupported;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides,
                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Does this kernel take the case?  bf16 is implied by the caller.
LSB_API int lsb_prefill_attention_tc5_supported(const void* qkv, int qkv_stride, const void* k_pages,
                                                const void* v_pages, int nh, int nkv, int hd, int page_size) {
    const bool pow2 = page_size > 0 && (page_size & (page_size - 1)) == 0;
    return (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && pow2 && page_size >= 8 && page_size <= kKeys &&
           qkv_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)k_pages % 16) == 0 &&
           ((uintptr_t)v_pages % 16) == 0;
}

template <int HD>
static int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& prm,
                  dim3 grid, cudaStream_t stream) {
    static int configured = -1;
    constexpr size_t smem = Smem<HD>::kTotal;
    if (configured < 0)
        configured = (int)cudaFuncSetAttribute(prefill_attention_tc5_kernel<HD>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (configured) return configured;
    return lsb_launch(prefill_attention_tc5_kernel<HD>, grid, dim3(kThreads), smem, stream, 1, mq, mk, mv, prm);
}

// Every request of the step is processed (single decode tokens too, as 1-row tiles, unless
// skip_single).
LSB_API int lsb_prefill_attention_tc5(const void* qkv, int qkv_stride, int n_tokens, const void* k_pages,
                                      const void* v_pages, const int* q_start, const int* kv_len,
                                      const int* table_rows, const int* block_table, int table_stride, void* out,
                                      int n_requests, int max_q_len, int nh, int nkv, int hd, int page_size,
                                      int num_pages, float scale, int window, int skip_single,
                                      cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (!lsb_prefill_attention_tc5_supported(qkv, qkv_stride, k_pages, v_pages, nh, nkv, hd, page_size) ||
        n_requests > 65535 || (max_q_len + kRows - 1) / kRows > 65535)
        return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mk, mv;
    int rc;
    {
        cuuint64_t dims[2] = {(cuuint64_t)qkv_stride, (cuuint64_t)n_tokens};
        cuuint64_t strides[1] = {(cuuint64_t)qkv_stride * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)kRows};
        if ((rc = encode(&mq, qkv, 2, dims, strides, box))) return rc;
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)page_size, (cuuint64_t)nkv, (cuuint64_t)num_pages};
        cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)page_size * hd * 2,
                                 (cuuint64_t)nkv * page_size * hd * 2};
        cuuint32_t box[4] = {64, (cuuint32_t)page_size, 1, 1};
        if ((rc = encode(&mk, k_pages, 4, dims, strides, box))) return rc;
        if ((rc = encode(&mv, v_pages, 4, dims, strides, box))) return rc;
    }
    AttnParams prm;
    prm.q_start = q_start; prm.kv_len = kv_len; prm.table_rows = table_rows; prm.block_table = block_table;
    prm.table_stride = table_stride; prm.out = (bf16*)out; prm.nh = nh; prm.nkv = nkv;
    prm.page_size = page_size; prm.num_pages = num_pages; prm.scale = scale; prm.window = window; prm.skip_single = skip_single;
    int sh = 0;
    while ((1 << sh) < page_size) ++sh;
    prm.page_shift = sh;
    dim3 grid(nh, (max_q_len + kRows - 1) / kRows, n_requests);
    return hd == 64 ? launch<64>(mq, mk, mv, prm, grid, stream) : launch<128>(mq, mk, mv, prm, grid, stream);
}
