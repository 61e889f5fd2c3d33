// bfloat16 matrix product on the 5th-generation tensor cores:  D[i, j] = sum_k P[i, k] * Q[j, k].
//
// Both operands are row-major with K contiguous ("K-major"), which is how activations [M, K] and
// checkpoint weights [N, K] already lie in memory (the reference hands the same pair to
// cublasSgemm, kernels/src/cublas_provider.cpp:36-51).  P supplies the 128 rows of a tile (the MMA
// M side, one accumulator row per TMEM lane), Q the BN columns (16..256).  The host picks which
// of activations and weights plays which role:
//   * many tokens (prefill): P = activations, Q = weights, output row-major [M, N];
//   * few tokens (decode): P = weights, Q = activations, so each thread block streams a 128-row
//     slab of the weight matrix exactly once and the batch rides on the narrow N side; the
//     output is written transposed back into [M, N]; K may be split over the blocks of a
//     thread-block cluster, which sum their 32-bit partial tiles through distributed shared
//     memory in rank order (no scratch in global memory, no second kernel, same bits every run).
//
// One thread block = one output tile (x one K split).  Warp 0 (one lane) issues TMA loads of
// [128 x 64] and [BN x 64] bf16 boxes with the 128-byte swizzle into a ring of shared-memory
// stages; warp 1 (one lane) issues tcgen05.mma (kind::f16, 32-bit accumulate in TMEM) and hands
// stages back with tcgen05.commit; warps 2-5 read the accumulator with tcgen05.ld and store it.
// Every wait on an mbarrier is bounded: when it runs out, the block records LSB_WAIT_TIMEOUT,
// all roles leave their loops, outstanding copies are waited for (bounded again), TMEM is freed
// and the block returns.  No load in this file uses cluster multicast.
#include "common.cuh"

#include <cuda.h>

LSB_DEFINE_STATUS()

typedef __nv_bfloat16 bf16;

constexpr int kBM = 128;             // rows of P per tile (TMEM lanes)
constexpr int kBK = 64;              // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;           // K of one tcgen05.mma for 16-bit inputs
constexpr int kGemmThreads = 192;    // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr uint32_t kSpinLimit = 1u << 22;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit = kSpinLimit) {
    for (uint32_t it = 0; it < limit; ++it) {
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
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
// arrives on the mbarrier once all tcgen05.mma issued so far by this thread have finished
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
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// thread-block cluster: rank, barrier over all threads of all blocks, peer shared memory
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_peer_f4(const void* own_smem, uint32_t rank) {
    uint32_t peer;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(smem_addr(own_smem)), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(peer) : "memory");
    return v;
}

// Shared-memory matrix descriptor of a K-major tile written by TMA with the 128-byte swizzle:
// rows of 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), tile base aligned to
// 1024 bytes.  Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30) (unused for
// swizzled K-major, set to 1), stride byte offset >> 4 [32,46), version 1 at [46,48), layout
// type SWIZZLE_128B = 2 at [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
    uint64_t d = (uint64_t)((smem_addr(tile) >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor of kind::f16: D format F32 (1) at [4,6), A and B format BF16 (1) at
// [7,10) and [10,13), both K-major (0 at bits 15, 16), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

struct GemmParams {
    int rows_p, rows_q, K;        // D is [rows_p, rows_q]
    long long ldc_i, ldc_j;       // element strides of the output along i and j
    int kb_per_split;             // 64-wide K blocks each split handles
    int num_kb;                   // ceil(K / 64)
    int splits;                   // > 1: the blocks of one tile form a cluster along z
    int out_f32;                  // output element type
    int swiglu;                   // 0: plain; 1: weight rows alternate gate/up along j; 2: along i.
    int act;                      // gated products: 1 silu, 2 gelu (tanh form), 3 none (gate * up)
                                  // The output then has half as many columns: silu(gate) * up.
    int static_operand;           // 1: P holds weights, 2: Q does (loaded before the PDL wait)
    void* out;                    // bf16 or float
};

template <int BN>
__device__ __forceinline__ void load_acc(uint32_t tmem_base, int q, int c0, bool have, uint32_t (&r)[32]) {
    if (have) {
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        if (BN - c0 >= 32) tmem_ld_32x32(taddr, r);
        else tmem_ld_32x16(taddr, r);
        tmem_ld_wait();
    } else {
#pragma unroll
        for (int x = 0; x < 32; ++x) r[x] = 0u;
    }
}

// act(g) * u for a gated product, with the special-function unit: ex2 and an approximate division
// (each good to about 1e-7 relative, far inside the rounding of the bfloat16 result).  silu(g) =
// g / (1 + e^-g); the tanh form of gelu, 0.5 g (1 + tanh(c (g + 0.044715 g^3))), is the same
// expression with another exponent, g / (1 + e^(-2 c (g + 0.044715 g^3))), c = sqrt(2 / pi).  The
// division must be the approximate one: for very negative gates 1 + e^-g is huge or infinite and
// an IEEE reciprocal drops into its slow denormal path, which cost 15 us per tile on random data.
enum : int { LSB_ACT_SILU = 1, LSB_ACT_GELU_TANH = 2, LSB_ACT_NONE = 3 };
__device__ __forceinline__ float gate_mul(float g, float u, int act) {
    if (act == LSB_ACT_NONE) return g * u;
    const float a = act == LSB_ACT_GELU_TANH ? 1.5957691216f * (g + 0.044715f * g * g * g) : g;
    return __fdividef(g, 1.f + __expf(-a)) * u;
}
#define silu_mul(g, u) gate_mul((g), (u), prm.act)

template <typename T> __device__ __forceinline__ void put(void* base, long long off, float v);
template <> __device__ __forceinline__ void put<float>(void* base, long long off, float v) {
    reinterpret_cast<float*>(base)[off] = v;
}
template <> __device__ __forceinline__ void put<bf16>(void* base, long long off, float v) {
    reinterpret_cast<bf16*>(base)[off] = __float2bfloat16_rn(v);
}

// Store n (<= 32) accumulator values of row i, columns j .. j + n - 1.  The whole warp calls this
// together (the gate/up exchange of swiglu mode 2 is a warp shuffle).
template <int BN>
__device__ __forceinline__ void store_chunk(const GemmParams& prm, uint32_t (&r)[32], int i, int j, int n, int lane) {
    const bool row_ok = i < prm.rows_p;
    const int ncols = min(n, prm.rows_q - j);              // may be <= 0
    if (prm.swiglu == 2) {
        // rows alternate gate, up: even lanes hold gates, their odd neighbours the matching ups
        for (int x = 0; x < n; ++x) {
            const float v = __uint_as_float(r[x]);
            const float other = __shfl_xor_sync(0xffffffffu, v, 1);
            if (!(lane & 1) && row_ok && x < ncols) {
                const long long o = (long long)(i >> 1) * prm.ldc_i + (long long)(j + x) * prm.ldc_j;
                if (prm.out_f32) put<float>(prm.out, o, silu_mul(v, other));
                else put<bf16>(prm.out, o, silu_mul(v, other));
            }
        }
        return;
    }
    if (!row_ok || ncols <= 0) return;
    if (prm.swiglu == 1) {
        // columns alternate gate, up (j is even: tiles start on even columns)
        const long long o = (long long)i * prm.ldc_i + (long long)(j >> 1) * prm.ldc_j;
        bf16* dst = reinterpret_cast<bf16*>(prm.out) + o;
        if (!prm.out_f32 && prm.ldc_j == 1 && ncols == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
            for (int x = 0; x < 32; x += 16) {
                uint32_t w[4];
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const float a = silu_mul(__uint_as_float(r[x + 4 * y]), __uint_as_float(r[x + 4 * y + 1]));
                    const float b = silu_mul(__uint_as_float(r[x + 4 * y + 2]), __uint_as_float(r[x + 4 * y + 3]));
                    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    w[y] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + x / 2) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
            for (int x = 0; x + 1 < ncols; x += 2) {
                const float v = silu_mul(__uint_as_float(r[x]), __uint_as_float(r[x + 1]));
                if (prm.out_f32) put<float>(prm.out, o + (x >> 1) * prm.ldc_j, v);
                else put<bf16>(prm.out, o + (x >> 1) * prm.ldc_j, v);
            }
        }
        return;
    }
    const long long o = (long long)i * prm.ldc_i + (long long)j * prm.ldc_j;
    if (prm.out_f32) {
        float* dst = reinterpret_cast<float*>(prm.out) + o;
        if (prm.ldc_j == 1 && ncols == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
            for (int x = 0; x < 32; x += 4)
                *reinterpret_cast<uint4*>(dst + x) = make_uint4(r[x], r[x + 1], r[x + 2], r[x + 3]);
        } else {
            for (int x = 0; x < ncols; ++x) dst[x * prm.ldc_j] = __uint_as_float(r[x]);
        }
    } else {
        bf16* dst = reinterpret_cast<bf16*>(prm.out) + o;
        if (prm.ldc_j == 1 && ncols == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
            for (int x = 0; x < 32; x += 8) {
                uint32_t w[4];
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[x + 2 * y]), __uint_as_float(r[x + 2 * y + 1]));
                    w[y] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + x) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
            for (int x = 0; x < ncols; ++x) dst[x * prm.ldc_j] = __float2bfloat16_rn(__uint_as_float(r[x]));
        }
    }
}

// Epilogue of a full-width bfloat16 tile in the row-major orientation: every thread converts
// its accumulator row (one TMEM lane), applies the gate if asked, and parks it in shared memory
// (the pipeline's stage buffers are idle by now) in 16-byte chunks XOR-swizzled by row; the warp
// then writes whole rows back with one 16-byte chunk per lane, so global stores are contiguous
// 256- or 512-byte runs instead of 32 scattered 16-byte pieces per instruction.
template <int BN, bool GATED>
__device__ __forceinline__ void epilogue_staged(const GemmParams& prm, unsigned char* stage_base, uint32_t tmem_base,
                                                int q, int lane, int i0, int j0) {
    constexpr int OUT_COLS = GATED ? BN / 2 : BN;
    constexpr int CPROW = OUT_COLS / 8;                       // 16-byte chunks per output row
    static_assert(CPROW >= 8, "the swizzle needs at least eight chunks per row");
    uint4* mine = reinterpret_cast<uint4*>(stage_base) + (size_t)q * 32 * CPROW;
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        if (GATED) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                uint32_t w[4];
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const int x = 16 * k + 4 * y;
                    const float a = silu_mul(__uint_as_float(r[x]), __uint_as_float(r[x + 1]));
                    const float b = silu_mul(__uint_as_float(r[x + 2]), __uint_as_float(r[x + 3]));
                    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    w[y] = *reinterpret_cast<uint32_t*>(&h);
                }
                const int cc = (c0 / 32) * 2 + k;
                mine[lane * CPROW + (cc ^ (lane & 7))] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t w[4];
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * k + 2 * y]),
                                                             __uint_as_float(r[8 * k + 2 * y + 1]));
                    w[y] = *reinterpret_cast<uint32_t*>(&h);
                }
                const int cc = (c0 / 32) * 4 + k;
                mine[lane * CPROW + (cc ^ (lane & 7))] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    __syncwarp();
    bf16* out = reinterpret_cast<bf16*>(prm.out);
    const int jo = GATED ? j0 / 2 : j0;
#pragma unroll
    for (int it = 0; it < CPROW; ++it) {                       // 32 rows x CPROW chunks / 32 lanes
        const int idx = it * 32 + lane;
        const int row = idx / CPROW, c = idx % CPROW;
        const int i = i0 + q * 32 + row;
        if (i < prm.rows_p)
            *reinterpret_cast<uint4*>(out + (long long)i * prm.ldc_i + jo + c * 8) = mine[row * CPROW + (c ^ (row & 7))];
    }
    __syncwarp();                                              // the buffer may be refilled right away
}

// Epilogue of a gated product in the swapped orientation (weights on the tile's 128 rows, gate and up
// rows alternating; the batch on its BN columns; bfloat16 output [batch, n_out]).  A thread owns one
// weight row, so an output row of the batch is spread over all 128 threads: written from there it
// is 2-byte stores 16 KB apart, 8.9 us for a 128 x 64 tile.  Here every pair of lanes forms its 64
// products, parks them in shared memory as [batch row][64 outputs] (the stage buffers are idle by
// now), the four epilogue warps meet, and each output row leaves as one 128-byte run.
template <int BN>
__device__ __forceinline__ void epilogue_swap_gated(const GemmParams& prm, unsigned char* stage_base,
                                                    uint32_t tmem_base, int q, int lane, int i0,
                                                    const int* abort_flag) {
    bf16* tile = reinterpret_cast<bf16*>(stage_base);         // [BN][64]
    const int n_local = (q * 32 + lane) >> 1;                 // this pair's output among the tile's 64
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        load_acc<BN>(tmem_base, q, c0, true, r);
        const int n = BN - c0 >= 32 ? 32 : 16;
#pragma unroll
        for (int x = 0; x < 32; ++x) {
            if (x < n) {
                const float v = __uint_as_float(r[x]);
                const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                if (!(lane & 1)) tile[(c0 + x) * 64 + n_local] = __float2bfloat16_rn(silu_mul(v, other));
            }
        }
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");             // the four epilogue warps
    if (*reinterpret_cast<const volatile int*>(abort_flag)) return;
    const int n_out = prm.rows_p >> 1, n0 = i0 >> 1;
    const int t = q * 32 + lane;
    bf16* out = reinterpret_cast<bf16*>(prm.out);
    for (int idx = t; idx < BN * 8; idx += 128) {              // 16-byte chunks: eight a batch row
        const int m = idx >> 3, c = idx & 7;
        if (m < prm.rows_q && n0 + c * 8 < n_out)
            *reinterpret_cast<uint4*>(out + (long long)m * prm.ldc_j + n0 + c * 8) =
                *reinterpret_cast<const uint4*>(tile + m * 64 + c * 8);
    }
}

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int kPBytes = kBM * kBK * 2;
    static constexpr int kQBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kPBytes + kQBytes;
    static constexpr int kBars = 2 * STAGES + 1;
    static constexpr size_t kTotal = 1024 + (size_t)STAGES * kStageBytes + kBars * 8 + 16;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               const GemmParams prm) {
    using L = SmemLayout<BN, STAGES>;
    constexpr uint32_t kTmemCols = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
    constexpr int kPartSwizzle = BN / 4 >= 8 ? 7 : BN / 4 - 1;     // see the partial tile below
    static_assert((size_t)kBM * BN * 4 <= (size_t)STAGES * L::kStageBytes, "the partial tile lives in the stage buffers");
    extern __shared__ unsigned char smem_raw[];
    // stage buffers need 1024-byte alignment (swizzle atom); the dynamic window is only 16-aligned
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = base;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + (size_t)STAGES * L::kStageBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i0 = blockIdx.x * kBM, j0 = blockIdx.y * BN;
    const int split = blockIdx.z;
    const int kb0 = split * prm.kb_per_split;
    const int kb1 = min(prm.num_kb, kb0 + prm.kb_per_split);
    const int nkb = max(0, kb1 - kb0);

    lsb_pdl_launch_dependents();
    const int pre = min(nkb, STAGES);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // Weights are not written by anything in the stream: their first STAGES boxes are
        // requested at once, before the block meets (tensor memory is being allocated meanwhile)
        // and before the wait on the previous kernel; the activations after it.
        for (int kb = 0; kb < pre; ++kb) {
            unsigned char* st = stages + (size_t)kb * L::kStageBytes;
            mbar_expect_tx(&full[kb], L::kStageBytes);
            if (prm.static_operand == 1) tma_load_2d(st, &map_p, &full[kb], (kb0 + kb) * kBK, i0);
            else tma_load_2d(st + L::kPBytes, &map_q, &full[kb], (kb0 + kb) * kBK, j0);
        }
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x != 0) lsb_pdl_wait();      // thread 0 (the TMA producer) waits after its prefetch

    if (warp == 0) {
        if (lane == 0) {
            lsb_pdl_wait();
            for (int kb = 0; kb < pre; ++kb) {
                unsigned char* st = stages + (size_t)kb * L::kStageBytes;
                if (prm.static_operand == 1) tma_load_2d(st + L::kPBytes, &map_q, &full[kb], (kb0 + kb) * kBK, j0);
                else tma_load_2d(st, &map_p, &full[kb], (kb0 + kb) * kBK, i0);
            }
            int issued = pre;
            for (int kb = pre; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1, &abort_flag)) break;
                mbar_expect_tx(&full[s], L::kStageBytes);
                unsigned char* st = stages + (size_t)s * L::kStageBytes;
                tma_load_2d(st, &map_p, &full[s], (kb0 + kb) * kBK, i0);
                tma_load_2d(st + L::kPBytes, &map_q, &full[s], (kb0 + kb) * kBK, j0);
                issued = kb + 1;
            }
            // copies still in flight must land before the block may exit
            for (int kb = max(0, issued - STAGES); kb < issued; ++kb) {
                int dummy = 0;
                mbar_wait(&full[kb % STAGES], (kb / STAGES) & 1, &dummy);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % STAGES;
                ok = mbar_wait(&full[s], (kb / STAGES) & 1, &abort_flag);
                if (!ok) break;
                tc_fence_after();
                unsigned char* st = stages + (size_t)s * L::kStageBytes;
                const uint64_t dp = make_smem_desc(st), dq = make_smem_desc(st + L::kPBytes);
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k)    // 32 bytes further along K: +2 in 16-byte units
                    umma_bf16(tmem_base, dp + 2 * k, dq + 2 * k, idesc, (kb | k) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);                         // arrives at once if nothing is pending
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int q = warp & 3;
        const int il = q * 32 + lane;                      // row within the tile
        bool ok = true;
        if (nkb > 0) {
            ok = mbar_wait(acc_full, 0, &abort_flag);
            tc_fence_after();
        }
        ok = ok && !abort_flag;
        // the common case of prompts: row-major bfloat16 output, the tile wholly inside the matrix
        const int n_out = prm.swiglu == 1 ? prm.rows_q / 2 : prm.rows_q;
        const bool staged = prm.splits == 1 && !prm.out_f32 && prm.ldc_j == 1 && prm.swiglu != 2 && nkb > 0 &&
                            j0 + BN <= prm.rows_q && (n_out % 8) == 0 && (((uintptr_t)prm.out) & 15) == 0 &&
                            (prm.swiglu == 0 ? BN >= 64 : BN >= 128);
        if (staged) {
            if (ok) {
                if constexpr (BN >= 128) {
                    if (prm.swiglu == 1) epilogue_staged<BN, true>(prm, stages, tmem_base, q, lane, i0, j0);
                    else epilogue_staged<BN, false>(prm, stages, tmem_base, q, lane, i0, j0);
                } else if constexpr (BN >= 64) {
                    epilogue_staged<BN, false>(prm, stages, tmem_base, q, lane, i0, j0);
                }
            }
        } else if (prm.splits == 1 && prm.swiglu == 2 && !prm.out_f32 && prm.ldc_i == 1 && nkb > 0 && j0 == 0 &&
                   ((prm.rows_p >> 1) % 8) == 0 && (prm.ldc_j % 8) == 0 && (((uintptr_t)prm.out) & 15) == 0) {
            // (a condition on the parameters alone: all four warps go in, also after a wait that ran
            // out, because they meet inside; nothing is stored then)
            epilogue_swap_gated<BN>(prm, stages, tmem_base, q, lane, i0, &abort_flag);
        } else if (prm.splits == 1) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                load_acc<BN>(tmem_base, q, c0, nkb > 0, r);
                if (ok) store_chunk<BN>(prm, r, i0 + il, j0 + c0, BN - c0 >= 32 ? 32 : 16, lane);
            }
        } else if (ok) {
            // this block's 32-bit partial tile goes to its own shared memory (the stage buffers
            // are free: every MMA that read them has completed); the cluster sums them below
            // (groups of four floats are swizzled by the row, so that the 32 rows a warp writes at
            // once spread over all banks)
            uint4* part = reinterpret_cast<uint4*>(stages) + (size_t)il * (BN / 4);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                load_acc<BN>(tmem_base, q, c0, nkb > 0, r);
                const int n = BN - c0 >= 32 ? 32 : 16;
                for (int x = 0; x < n; x += 4)
                    part[((c0 + x) / 4) ^ (il & kPartSwizzle)] = make_uint4(r[x], r[x + 1], r[x + 2], r[x + 3]);
            }
        }
    }
    if (prm.splits > 1) {
        // The blocks of a tile (one per K split) are one cluster.  After the barrier every block
        // sums a share of the tile over all blocks' shared memory, in rank order, and stores it.
        __syncwarp();               // lanes that took a role branch rejoin their warp first
        cluster_barrier();
        if (warp >= 2 && !abort_flag) {
            const uint32_t rank = cluster_rank();
            const uint4* part = reinterpret_cast<const uint4*>(stages);
            const int t = (warp - 2) * 32 + lane;
            const bool rows_whole = prm.ldc_j == 1 && (prm.ldc_i & 3) == 0 && (((uintptr_t)prm.out) & 15) == 0;
            for (int g4 = (int)rank * 128 + t; g4 < kBM * BN / 4; g4 += prm.splits * 128) {
                const int row = g4 / (BN / 4), c4 = g4 % (BN / 4);
                const uint4* src = part + (size_t)row * (BN / 4) + (c4 ^ (row & kPartSwizzle));
                float4 v[8];                                  // all peers' loads in flight at once
#pragma unroll
                for (int peer = 0; peer < 8; ++peer)
                    if (peer < prm.splits) v[peer] = ld_peer_f4(src, (uint32_t)peer);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int peer = 0; peer < 8; ++peer)          // summed in rank order
                    if (peer < prm.splits) { acc.x += v[peer].x; acc.y += v[peer].y; acc.z += v[peer].z; acc.w += v[peer].w; }
                const int i = i0 + row, j = j0 + c4 * 4;
                if (i < prm.rows_p) {
                    const long long o0 = (long long)i * prm.ldc_i + (long long)j * prm.ldc_j;
                    if (rows_whole && j + 3 < prm.rows_q) {
                        if (prm.out_f32) {
                            *reinterpret_cast<float4*>(reinterpret_cast<float*>(prm.out) + o0) = acc;
                        } else {
                            const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
                            const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
                            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(prm.out) + o0) =
                                make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                        }
                    } else {
                        const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
                        for (int x = 0; x < 4; ++x) {
                            if (j + x >= prm.rows_q) break;
                            const long long o = o0 + (long long)x * prm.ldc_j;
                            if (prm.out_f32) put<float>(prm.out, o, vals[x]);
                            else put<bf16>(prm.out, o, vals[x]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        cluster_barrier();          // nobody leaves while a peer may still read its shared memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ persistent kernel (prompts)
// One block per SM walks a list of output tiles (row-major orientation, 128 x BN, one K range).
// The accumulator is double-buffered in TMEM (2 x BN columns): while the epilogue warps drain
// tile i from one buffer into global memory, the MMA warp already fills the other with tile i+1,
// and the TMA warp runs ahead through the ring of stages without regard to tile boundaries.  This
// removes the per-tile set-up (barriers, TMEM allocation, first loads) and hides the epilogue.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

constexpr int kEpiCols = 128;                                 // columns drained per pass
constexpr int kEpiBytes = 4 * 32 * kEpiCols * 2;             // 4 warps x 32 rows x 128 bf16

template <int BN, int STAGES>
struct PersistentLayout {
    static constexpr int kPBytes = kBM * kBK * 2;
    static constexpr int kQBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kPBytes + kQBytes;
    static constexpr int kBars = 2 * STAGES + 4;
    static constexpr size_t kTotal = 1024 + (size_t)STAGES * kStageBytes + kEpiBytes + kBars * 8 + 16;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                          const GemmParams prm, int tiles_m, int tiles_n) {
    using L = PersistentLayout<BN, STAGES>;
    static_assert(BN == 16 || BN == 32 || BN == 64 || BN == 128 || BN == 256,
                  "two accumulators of BN columns: a power of two of TMEM columns, at most 512");
    constexpr uint32_t kTmemCols = 2 * BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = base;
    unsigned char* epi = base + (size_t)STAGES * L::kStageBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(epi + kEpiBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;                      // [2]
    uint64_t* acc_empty = acc_full + 2;                       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = tiles_m * tiles_n;
    const int nkb = prm.num_kb;

    lsb_pdl_launch_dependents();
    // tile t -> (row block, column block); neighbouring blocks share the weight columns
    const bool weights_p = prm.static_operand == 1;
    int pre = 0;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // The weights are not written by anything in the stream: the boxes of the first ring fill are
        // requested at once, before the block meets (tensor memory is being allocated meanwhile) and
        // before the wait on the previous kernel; the activations after it.
        for (int t = blockIdx.x; t < n_tiles && pre < STAGES; t += gridDim.x) {
            const int i0 = (t % tiles_m) * kBM, j0 = (t / tiles_m) * BN;
            for (int kb = 0; kb < nkb && pre < STAGES; ++kb, ++pre) {
                unsigned char* st = stages + (size_t)pre * L::kStageBytes;
                mbar_expect_tx(&full[pre], L::kStageBytes);
                if (weights_p) tma_load_2d(st, &map_p, &full[pre], kb * kBK, i0);
                else tma_load_2d(st + L::kPBytes, &map_q, &full[pre], kb * kBK, j0);
            }
        }
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x != 0) lsb_pdl_wait();      // thread 0 (the TMA producer) waits after its first weight boxes

    if (warp == 0) {
        if (lane == 0) {
            lsb_pdl_wait();
            long long it = 0;                                  // K blocks issued so far, over all tiles
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int i0 = (t % tiles_m) * kBM, j0 = (t / tiles_m) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    unsigned char* st = stages + (size_t)s * L::kStageBytes;
                    if (it < pre) {                            // the other half of a box requested above
                        if (weights_p) tma_load_2d(st + L::kPBytes, &map_q, &full[s], kb * kBK, j0);
                        else tma_load_2d(st, &map_p, &full[s], kb * kBK, i0);
                        continue;
                    }
                    if (it >= STAGES && !mbar_wait(&empty[s], (uint32_t)((it / STAGES) - 1) & 1, &abort_flag)) { ok = false; break; }
                    mbar_expect_tx(&full[s], L::kStageBytes);
                    tma_load_2d(st, &map_p, &full[s], kb * kBK, i0);
                    tma_load_2d(st + L::kPBytes, &map_q, &full[s], kb * kBK, j0);
                }
            }
            // copies still in flight must land before the block may exit
            for (long long k = it > STAGES ? it - STAGES : 0; k < it; ++k) {
                int dummy = 0;
                mbar_wait(&full[k % STAGES], (uint32_t)(k / STAGES) & 1, &dummy);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            long long it = 0;
            int local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++local) {
                const int a = local & 1;
                // the epilogue must have drained this accumulator (passes at once the first time)
                ok = mbar_wait(&acc_empty[a], (uint32_t)((local >> 1) & 1) ^ 1u, &abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(a * BN);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    ok = mbar_wait(&full[s], (uint32_t)(it / STAGES) & 1, &abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    unsigned char* st = stages + (size_t)s * L::kStageBytes;
                    const uint64_t dp = make_smem_desc(st), dq = make_smem_desc(st + L::kPBytes);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k)
                        umma_bf16(tmem_d, dp + 2 * k, dq + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    umma_commit(&empty[s]);
                }
                umma_commit(&acc_full[a]);
            }
        }
    } else {
        const int q = warp & 3;
        const int il = q * 32 + lane;
        const int n_out = prm.swiglu == 1 ? prm.rows_q / 2 : prm.rows_q;
        const bool aligned = !prm.out_f32 && (n_out % 8) == 0 && (((uintptr_t)prm.out) & 15) == 0;
        int local = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++local) {
            const int a = local & 1;
            const int i0 = (t % tiles_m) * kBM, j0 = (t / tiles_m) * BN;
            ok = mbar_wait(&acc_full[a], (uint32_t)(local >> 1) & 1, &abort_flag);
            tc_fence_after();
            ok = ok && !abort_flag;
            if (!ok) break;
            const uint32_t tmem_acc = tmem_base + (uint32_t)(a * BN);
            if (BN >= kEpiCols && aligned && j0 + BN <= prm.rows_q) {
#pragma unroll
                for (int h = 0; h < BN / kEpiCols; ++h) {
                    if (prm.swiglu == 1)
                        epilogue_staged<kEpiCols, true>(prm, epi, tmem_acc + h * kEpiCols, q, lane, i0, j0 + h * kEpiCols);
                    else
                        epilogue_staged<kEpiCols, false>(prm, epi, tmem_acc + h * kEpiCols, q, lane, i0, j0 + h * kEpiCols);
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    load_acc<BN>(tmem_acc, q, c0, true, r);
                    store_chunk<BN>(prm, r, i0 + il, j0 + c0, 32, lane);
                }
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[a]);                        // 128 arrivals hand the buffer back
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
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

// [rows, K] bf16 row-major, boxes of [box_rows x 64], 128-byte swizzle, zero fill outside
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int BN, int STAGES>
static int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& prm, dim3 grid,
                  cudaStream_t stream) {
    static int configured = -1;
    constexpr size_t smem = SmemLayout<BN, STAGES>::kTotal;
    if (configured < 0)
        configured = (int)cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (configured) return configured;
    return lsb_launch(gemm_tc_kernel<BN, STAGES>, grid, dim3(kGemmThreads), smem, stream, prm.splits, mp, mq, prm);
}

template <int BN, int STAGES>
static int launch_persistent(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& prm, int tiles_m,
                             int tiles_n, cudaStream_t stream) {
    static int configured = -1;
    static int sms = 0;
    constexpr size_t smem = PersistentLayout<BN, STAGES>::kTotal;
    if (configured < 0) {
        configured = (int)cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    if (configured) return configured;
    const int tiles = tiles_m * tiles_n;
    const int blocks = tiles < sms ? tiles : sms;
    return lsb_launch(gemm_tc_persistent_kernel<BN, STAGES>, dim3(blocks), dim3(kGemmThreads), smem, stream, 1,
                      mp, mq, prm, tiles_m, tiles_n);
}

// What happens when a wait runs out, shown without a fault: one block, a barrier that nothing
// arrives at.  Thread 0 waits on it with a limit of `limit` polls, gives up, raises the block's
// abort flag and records LSB_WAIT_TIMEOUT in the status word; thread 32 waits with the kernels'
// full limit and leaves as soon as it sees the flag.  result[0], result[1]: 1 where the wait
// returned false.  The kernel always ends by itself; the host then reads the status word.
__global__ void wait_timeout_probe_kernel(uint32_t limit, int* __restrict__ result) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) result[0] = mbar_wait(&bar, 0, &abort_flag, limit) ? 0 : 1;
    if (threadIdx.x == 32) result[1] = mbar_wait(&bar, 0, &abort_flag) ? 0 : 1;
}

LSB_API int lsb_gemm_tc_wait_probe(int limit, int* result, cudaStream_t stream) {
    if (limit < 1 || limit > (1 << 16)) return (int)cudaErrorInvalidValue;
    wait_timeout_probe_kernel<<<1, 64, 0, stream>>>((uint32_t)limit, result);
    return LSB_LAUNCH_CHECK();
}

// SMs of the current device (asked once per device).
static int num_sms() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

// Can this kernel take the product?  (TMA needs 16-byte aligned bases and row strides.)
LSB_API int lsb_gemm_tc_supported(const void* x, const void* w, int M, int N, int K) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0;
}

// The plan for a product: orientation (swap = weights on the 128-row side), tile width and K
// splits.  With more than one split the blocks of a tile form a thread-block cluster and sum their
// partial tiles through distributed shared memory, so there is no scratch in global memory; the
// portable cluster size limits the splits to 8.
LSB_API int lsb_gemm_tc_plan(int M, int N, int K, int swiglu, int* swap, int* bn, int* splits) {
    const int num_kb = (K + kBK - 1) / kBK;
    const int sms = num_sms();
    const int most = sms * 13 / 16;              // "nearly every SM has a tile" (120 of 148)
    if (M <= 128) {
        *swap = 1;
        *bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        const int tiles = (N + kBM - 1) / kBM;
        int s = 1;
        if (tiles < most && !swiglu) {           // too few slabs to fill the SMs: split K
            s = (sms + tiles - 1) / tiles;
            if (s > 8) s = 8;
            if (s > num_kb / 4) s = num_kb / 4 > 0 ? num_kb / 4 : 1;   // at least 4 K blocks each
            if (s < 1) s = 1;
        }
        if (s > 1) {                              // no empty splits
            const int per = (num_kb + s - 1) / s;
            s = (num_kb + per - 1) / per;
        }
        *splits = s;
    } else {
        *swap = 0;
        // the widest tile that still fills the machine reasonably
        const int mt = (M + kBM - 1) / kBM;
        int best = 64;
        double best_eff = -1.0;
        const int cands[3] = {256, 128, 64};
        for (int c = 0; c < 3; ++c) {
            const int t = mt * ((N + cands[c] - 1) / cands[c]);
            const int waves = (t + sms - 1) / sms;
            double eff = (double)t / ((double)waves * sms);
            if (cands[c] == 64) eff *= 0.8;      // narrower tiles reuse P less
            else if (cands[c] == 128) eff *= 0.93;
            if (eff > best_eff + 1e-9) { best_eff = eff; best = cands[c]; }
        }
        // persistent blocks walk the tile list, so whole waves no longer matter: take the widest
        // tile unless that leaves SMs without any
        if (mt * ((N + 255) / 256) >= most || N >= 2048) best = 256;
        *bn = best;
        *splits = 1;
        // A few hundred tokens make too few 128 x 256 tiles for the SMs.  Where the walk through K
        // is long (the down projection), K is split over a cluster, as many ways as fit in one
        // wave; summing the partial tiles costs about as much as 2048 of K, so shorter walks stay
        // whole.  (The gated epilogue needs whole sums: gated products stay unsplit too.)
        const int tiles = mt * ((N + 255) / 256);
        if (best == 256 && tiles < most && !swiglu) {
            int s = sms / tiles;
            if (s > 8) s = 8;
            if (s > num_kb / 32) s = num_kb / 32;
            if (s > 1) {
                const int per = (num_kb + s - 1) / s;
                *splits = (num_kb + per - 1) / per;
            }
        }
        // Unsplit and at most half the SMs busy: tiles half as wide bring the rest in (each
        // block's stream of operands, which is what a lone tile waits for, gets shorter).
        if (*splits == 1 && best == 256 && tiles <= sms / 2 && N > 128) *bn = 128;
    }
    return 0;
}

// out[M, N] = x[M, K] * w[N, K]^T, bf16 inputs, bf16 or float output.
// swiglu != 0: w has 2 * N_out rows alternating gate_i, up_i; out is [M, N / 2] with
// out[m, i] = act(d[m, 2i]) * d[m, 2i + 1], act named by swiglu: 1 silu, 2 gelu (tanh form), 3 none.
LSB_API int lsb_gemm_tc(const void* x, const void* w, void* out, int out_f32, int M, int N, int K,
                        int swiglu, cudaStream_t stream) {
    if (!lsb_gemm_tc_supported(x, w, M, N, K)) return (int)cudaErrorInvalidValue;
    if (swiglu && (N % 2)) return (int)cudaErrorInvalidValue;
    if (swiglu < 0 || swiglu > LSB_ACT_NONE) return (int)cudaErrorInvalidValue;
    int swap, bn, splits;
    lsb_gemm_tc_plan(M, N, K, swiglu, &swap, &bn, &splits);
    const int n_out = swiglu ? N / 2 : N;
    GemmParams prm;
    prm.K = K;
    prm.num_kb = (K + kBK - 1) / kBK;
    prm.kb_per_split = (prm.num_kb + splits - 1) / splits;
    prm.splits = splits;
    prm.out_f32 = out_f32;
    prm.out = out;
    prm.act = swiglu;
    const int sms = num_sms();
    CUtensorMap mp, mq;
    int rc;
    dim3 grid;
    if (swap) {
        prm.rows_p = N; prm.rows_q = M; prm.ldc_i = 1; prm.ldc_j = n_out;
        prm.swiglu = swiglu ? 2 : 0;
        prm.static_operand = 1;
        if ((rc = make_map(&mp, w, N, K, kBM))) return rc;
        if ((rc = make_map(&mq, x, M, K, bn))) return rc;
        grid = dim3((N + kBM - 1) / kBM, 1, splits);
    } else {
        prm.rows_p = M; prm.rows_q = N; prm.ldc_i = n_out; prm.ldc_j = 1;
        prm.swiglu = swiglu ? 1 : 0;
        prm.static_operand = 2;
        if ((rc = make_map(&mp, x, M, K, kBM))) return rc;
        if ((rc = make_map(&mq, w, N, K, bn))) return rc;
        grid = dim3((M + kBM - 1) / kBM, (N + bn - 1) / bn, 1);
    }
    // Blocks of a split product are co-scheduled as clusters: four stages keep their shared memory
    // small enough for two or three blocks per SM, so that every cluster finds room at once.
    // Unsplit products run one block per SM and want the deeper ring to keep HBM busy.
    if (!swap && splits > 1) {
        grid.z = splits;
        return launch<256, 4>(mp, mq, prm, grid, stream);
    }
    if (!swap && !out_f32 && bn >= 128) {
        // prompts: persistent blocks, double-buffered accumulator
        const int tm = (M + kBM - 1) / kBM, tn = (N + bn - 1) / bn;
        return bn == 256 ? launch_persistent<256, 4>(mp, mq, prm, tm, tn, stream)
                         : launch_persistent<128, 6>(mp, mq, prm, tm, tn, stream);
    }
    if (splits > 1) {
        switch (bn) {
            case 16: rc = launch<16, 4>(mp, mq, prm, grid, stream); break;
            case 32: rc = launch<32, 4>(mp, mq, prm, grid, stream); break;
            case 64: rc = launch<64, 4>(mp, mq, prm, grid, stream); break;
            case 128: rc = launch<128, 4>(mp, mq, prm, grid, stream); break;
            default: return (int)cudaErrorInvalidValue;
        }
    } else if (swap && !swiglu && (int)grid.x >= 2 * sms) {
        // Many more weight slabs than SMs (the output head): persistent blocks walk the slabs, the
        // loads of the next slab run under the epilogue of this one and no SM idles between waves.
        const int tm = (int)grid.x;
        switch (bn) {
            case 16: rc = launch_persistent<16, 8>(mp, mq, prm, tm, 1, stream); break;
            case 32: rc = launch_persistent<32, 8>(mp, mq, prm, tm, 1, stream); break;
            case 64: rc = launch_persistent<64, 6>(mp, mq, prm, tm, 1, stream); break;
            case 128: rc = launch_persistent<128, 5>(mp, mq, prm, tm, 1, stream); break;
            default: return (int)cudaErrorInvalidValue;
        }
    } else if (swap && (int)grid.x > sms && bn <= 64) {
        // More weight slabs than SMs, fewer than two rounds of them (a wide gated product): with
        // the deep ring one block fits an SM and the second round would run half empty; four
        // stages let two blocks share an SM, so all slabs stream at once (28,672 x 4,096 gated:
        // 54.6 -> 46.7 us at 8 rows, 65.4 -> 51.8 us at 64).  At 128 rows four stages fill an SM
        // by themselves, so that size keeps the deep ring.
        switch (bn) {
            case 16: rc = launch<16, 4>(mp, mq, prm, grid, stream); break;
            case 32: rc = launch<32, 4>(mp, mq, prm, grid, stream); break;
            case 64: rc = launch<64, 4>(mp, mq, prm, grid, stream); break;
            default: return (int)cudaErrorInvalidValue;
        }
    } else {
        // 32 and 64 rows: four stages, so that the blocks of the next product (often split over a
        // cluster) find room beside these and start under their ends (a decode step of 32 or 64
        // rows at 1,024 tokens of context: 2 % shorter than with six and eight stages)
        switch (bn) {
            case 16: rc = launch<16, 8>(mp, mq, prm, grid, stream); break;
            case 32: rc = launch<32, 4>(mp, mq, prm, grid, stream); break;
            case 64: rc = launch<64, 4>(mp, mq, prm, grid, stream); break;
            case 128: rc = launch<128, 6>(mp, mq, prm, grid, stream); break;
            case 256: rc = launch<256, 4>(mp, mq, prm, grid, stream); break;
            default: return (int)cudaErrorInvalidValue;
        }
    }
    return rc;
}

