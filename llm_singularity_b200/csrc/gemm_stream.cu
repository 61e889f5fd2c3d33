// out[M, N] = x[M, K] * w[N, K]^T for a handful of rows (M <= 16) and a weight matrix of any size:
// the feed-forward products of a decode step (gate/up with its activation, down), which are pure
// weight traffic.  What such a product needs is every SM pulling its share of the weights all the
// time, nothing else.
//
// * The weight rows are dealt over one block per SM row by row (pairs of rows for a gated
//   product), not tile by tile: 2,048 rows over 148 SMs are 13 or 14 rows each, where 128-row
//   slabs would leave 20 SMs without work and a K split would need a sum across blocks.  A block
//   walks K for its own rows alone, so there is no cluster, no partial tile outside the block,
//   and the order of every sum is fixed: results repeat bit for bit.
// * One producer thread streams the block's rows through a ring of K chunks in shared memory by
//   TMA: one tiled copy per stage whose box is (64 of K) x (the block's rows) x (the chunk's 64-wide
//   pieces), through a three-dimensional tensor map over the weight matrix, completion counted by
//   an mbarrier per stage; the matching chunk of the activations rides along the same way.  (A
//   bulk copy per row segment was tried first: the copy unit takes some 50 ns per request, however
//   small, and 256-byte requests capped the product at 0.8 TB/s.)  Weights depend on nothing, so
//   the ring is filled before the wait on the previous kernel of the stream (programmatic
//   dependent launch); the activations are requested after it.  The ring takes most of an SM's
//   shared memory (200 KB a block).  Half of that, so that the blocks of two consecutive products
//   share an SM and the second one's ring is full when the first one ends, was slower: what the
//   memory system wants is bytes in flight (gate/up at 8 rows inside a decode step: 15.3 us with
//   112 KB a block, 13.7 us with 200 KB; the down product 14.3 and 11.5 us).
// * Eight consumer warps split each chunk along K and run mma.sync (m16n8k16: sixteen weight rows
//   by up to sixteen activation rows); their partial sums meet in shared memory at the end, in
//   warp order.  Rows of a 16-row tile that are not the block's own, and activation rows beyond
//   M, are never loaded (the latter are filled with zeros by the copy): what the tensor core
//   makes of them lands in outputs nobody stores.  Rows lie in shared memory as 128-byte pieces
//   whose 16-byte chunks the copy swizzles by the piece's index, which spreads the eight rows of
//   an ldmatrix over all banks.
//
// act != 0: w has 2 * N_out rows alternating gate_i, up_i and out is [M, N / 2] with
// out[m, i] = act(d[m, 2i]) * d[m, 2i + 1] (1 silu, 2 gelu in its tanh form, 3 none), in 32-bit.
//
// The reference calls cublasSgemm for every projection (kernels/src/cublas_provider.cpp:36-51) and
// a separate kernel for silu(g) * u (kernels/src/activations.cu:11-21).  No load here uses cluster
// multicast.
#include "common.cuh"
#include "stream_warm.cuh"

#include <cuda.h>

LSB_DEFINE_STATUS()

typedef __nv_bfloat16 bf16;

constexpr int kWarps = 8;                       // consumer warps; warp kWarps is the producer
constexpr int kThreads = 32 * (kWarps + 1);
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 200 * 1024;         // one block per SM; most of it is the ring
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr int kSsPerLane = 5;                  // parts of a row's sum of squares a lane adds up: 160 parts at most
constexpr int kWarmBytes = 112 * 1024;          // of the next product's weights, a block asks L2 for this much
constexpr int kTailBytes = 320;                // barriers, the give-up flag, the rows' scales
static_assert(3 * kMaxStages * 8 + 16 + 16 * 4 <= kTailBytes, "barriers, flag and scales fit the tail");
constexpr int kFoldBytes = (16 * 128 + kWarps * 128 + 16) * 4;   // more shared memory if the product adds to the residual
enum : int { LSB_ACT_SILU = 1, LSB_ACT_GELU_TANH = 2, LSB_ACT_NONE = 3 };

struct StreamParams {
    const bf16* x;
    const bf16* w;
    void* out;
    int M, N, K;
    int out_f32;
    int act;            // 0: plain product; else the activation of a gated product
    int kc;             // K per stage (a multiple of 128)
    int stages;
    int unit;           // rows are dealt in units of this many (2 for a gated product)
    int w_bytes;        // shared memory a stage keeps for weights (a multiple of 1024)
    int rows_a, rows_b, rows_c;   // rows of the boxes of the three weight maps
    int rt, rt_log2;    // 16-row tiles of a pass (1, 2, 4 or 8)
    int rows_hi, rows_lo, n_hi;   // the first n_hi blocks have rows_hi rows, the others rows_lo
    int nk;             // chunks of K
    // A norm folded into the products on either side of it (see lsb_gemm_stream_folded):
    const float* ss_in;     // [ss_parts][16]: sums of squares of the rows x stands for, in parts; or null
    int ss_parts;
    float inv_size, eps;    // the rows' scale is rsqrt(sum * inv_size + eps)
    float* residual;        // [M, N] 32-bit, += the product in place; or null
    const float* norm_w;    // [N]: out = (residual + product) * norm_w
    float* ss_out;          // [blocks][16]: this block's part of the new rows' sums of squares
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the limit ran out or another warp of the block already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    lsb_set_status(LSB_WAIT_TIMEOUT);
    return false;
}
// One box of a three-dimensional tensor map into shared memory (1024-byte aligned).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Byte offset of 16-byte chunk `chunk` of 128-byte piece `piece` of a box (128-byte swizzle; the box
// starts on a 1024-byte boundary).
__device__ __forceinline__ uint32_t swz(int piece, int chunk) {
    return (uint32_t)((piece << 7) + (((chunk ^ piece) & 7) << 4));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                 "{%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kWarps) : "memory"); }

__device__ __forceinline__ float gate_act(float g, int act) {
    if (act == LSB_ACT_SILU) return g / (1.f + __expf(-g));
    if (act == LSB_ACT_GELU_TANH) return 0.5f * g * (1.f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
    return g;
}

// A pass covers 16 * rt rows of the block (rt = 1, 2, 4 or 8 tiles); the eight consumer warps are
// rt tiles x (8 / rt) parts of every chunk's K, one 16-row tile and one part each.  A warp keeps kInFlight
// k-steps going at once, each with an accumulator of its own (one mma at a time on one accumulator
// would wait out the tensor core's latency at every step).  NT: 8-row tiles of activations.
constexpr int kInFlight = 4;

// FOLDS: the kernel can take rows whose norm is still owed (prm.ss_in) and add its product to the
// residual, leaving the next norm half done (prm.residual).  The kernel without that code, for
// plain products, is 0.4 us shorter a launch (gate/up and down of a 1B layer in a chain: 19.4
// against 20.2 us a pair): these kernels run once, cold, and every line of instructions counts.
template <int NT, bool FOLDS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_x,
                   const StreamParams prm, const __grid_constant__ StreamWarm warm) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_raw = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    lsb_pdl_launch_dependents();
    const bool SCALED = FOLDS && prm.ss_in != nullptr, ADDS = FOLDS && prm.residual != nullptr;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kc = prm.kc, stages = prm.stages;
    const int pieces = kc >> 6;                                   // 64-wide pieces of a chunk
    const int w_bytes = prm.w_bytes, x_bytes = pieces * 8 * NT * 128;   // (x_bytes: a multiple of 1024)
    const int stage_bytes = w_bytes + x_bytes;
    constexpr int width = 8 * NT;

    unsigned char* ring = smem_raw;
    float* red = reinterpret_cast<float*>(ring + (size_t)stages * stage_bytes);   // [2][kWarps * 16][width]
    uint64_t* full_w = reinterpret_cast<uint64_t*>(red + 2 * kWarps * 16 * width);   // [kMaxStages] each
    uint64_t* full_x = full_w + kMaxStages;
    uint64_t* empty = full_x + kMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxStages);
    float* scale_s = reinterpret_cast<float*>(empty + kMaxStages) + 4;      // [16]: the rows' scales
    // (only there if the product adds to the residual: the block's piece of the residual [16][128],
    // the norm's weights once per warp [kWarps][128], sums of squares [16])
    float* res_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(full_w) + kTailBytes);
    float* nw_s = res_s + 16 * 128;
    float* ss_s = nw_s + kWarps * 128;

    // this block's rows
    // (worked out without a division: a kernel that lives ten microseconds cannot spend half of one
    // on index arithmetic before its first copy is asked for)
    const int blk = (int)blockIdx.x;
    const bool longer = blk < prm.n_hi;
    const int rows = longer ? prm.rows_hi : prm.rows_lo;
    const int r0 = longer ? blk * prm.rows_hi : prm.n_hi * prm.rows_hi + (blk - prm.n_hi) * prm.rows_lo;
    const int rt = prm.rt, rows_cap = 16 * rt;
    const int passes = (rows + rows_cap - 1) >> (4 + prm.rt_log2);
    const int nk = prm.nk;
    // Every block needs the same activations.  Each starts its walk through K at another chunk, so
    // that at any moment the blocks ask L2 for different lines (all of them on the same few lines
    // at once is a queue at those lines' L2 slices); the order of a block's sums is still fixed.
    const int k_shift = (int)(blockIdx.x % (unsigned)nk);

    if (warp == kWarps) {
        // ------------------------------------------------------------------ producer
        // (one thread: a stage is one copy of weights and one of activations.  It sets up the
        // barriers itself and asks for the first stages before the block meets.)
        // A walk through (pass, chunk of K, stage of the ring), one step at a time; `turn` counts the
        // trips around the ring (its lowest bit is the parity a stage's barriers complete with).
        struct Walk { int pass, kb, s, turn; };
        auto step = [&](Walk& w) {
            if (++w.kb == nk) { w.kb = 0; ++w.pass; }
            if (++w.s == stages) { w.s = 0; ++w.turn; }
        };
        auto chunk_of = [&](const Walk& w) { const int c = w.kb + k_shift; return c >= nk ? c - nk : c; };
        auto issue_w = [&](const Walk& w) {
            const int pr0 = w.pass * rows_cap, prows = min(rows_cap, rows - pr0);
            const CUtensorMap* map = prows == prm.rows_a ? &map_a : prows == prm.rows_b ? &map_b : &map_c;
            mbar_expect_tx(&full_w[w.s], (uint32_t)(prows * kc * 2));
            tma_load_3d(ring + (size_t)w.s * stage_bytes, map, &full_w[w.s], 0, r0 + pr0, chunk_of(w) * pieces);
        };
        auto issue_x = [&](const Walk& w) {
            mbar_expect_tx(&full_x[w.s], (uint32_t)x_bytes);
            tma_load_3d(ring + (size_t)w.s * stage_bytes + w_bytes, &map_x, &full_x[w.s], 0, 0, chunk_of(w) * pieces);
        };
        Walk ww = {0, 0, 0, 0};          // the next weights to ask for
        if (lane == 0) {
            *abort_flag = 0;
            for (int s = 0; s < stages; ++s) {
                mbar_init(&full_w[s], 1);
                mbar_init(&full_x[s], 1);
                mbar_init(&empty[s], kWarps);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            while (ww.turn == 0 && ww.pass < passes) {             // weights depend on nothing
                issue_w(ww);
                step(ww);
            }
        }
        __syncthreads();
        if (lane != 0) return;
        lsb_pdl_wait();
        Walk wx = {0, 0, 0, 0};          // the next activations to ask for
        bool ok = true;
        while (wx.pass < passes) {
            if (wx.turn > 0) {
                ok = mbar_wait(&empty[wx.s], (uint32_t)((wx.turn & 1) ^ 1), abort_flag);
                if (!ok) break;
                issue_w(ww);
                step(ww);
            }
            issue_x(wx);
            step(wx);
        }
        if (ok) stream_warm_issue(warm, blk);      // everything of this product is asked for: on to the next
        if (!ok) {
            // gave up: copies still in flight must land before the block's shared memory goes away
            // (every stage's last copy of weights, and of activations, that was asked for)
            for (int back = 0; back < stages; ++back) {
                Walk w = ww;
                for (int n = 0; n <= back; ++n) { if (w.s == 0) { w.s = stages; --w.turn; } --w.s; }
                if (w.turn < 0) break;
                for (uint32_t n = 0; n < (1u << 16) && !mbar_try_wait(&full_w[w.s], (uint32_t)(w.turn & 1)); ++n)
                    __nanosleep(64);
            }
            for (int back = 0; back < stages; ++back) {
                Walk w = wx;
                for (int n = 0; n <= back; ++n) { if (w.s == 0) { w.s = stages; --w.turn; } --w.s; }
                if (w.turn < 0) break;
                for (uint32_t n = 0; n < (1u << 16) && !mbar_try_wait(&full_x[w.s], (uint32_t)(w.turn & 1)); ++n)
                    __nanosleep(64);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    __syncthreads();         // the barriers are set up
    lsb_pdl_wait();          // before anything of this kernel is stored (its output buffer may be one
                             // that an earlier kernel of the stream still reads)
    const int a_row = ((lane >> 3) & 1) * 8 + (lane & 7), a_half = lane >> 4;
    const int b_row = lane & 7, b_half = (lane >> 3) & 1;
    const int my_tile = warp & (rt - 1), my_part = warp / rt, parts = kWarps / rt;
    // What the end of a pass needs of the kernel's parameters is read now, into registers: a
    // parameter read for the first time costs a trip past the constant cache (some 0.3 us each,
    // one after the other, in a kernel whose whole end is 1 us), and here it hides under the wait
    // for the first weights.
    int e_M = prm.M, e_N = prm.N, e_act = prm.act, e_f32 = prm.out_f32;
    void* e_out = prm.out;
    float e_inv = prm.inv_size, e_eps = prm.eps;
    float* e_res = prm.residual;
    const float* e_nw = prm.norm_w;
    float* e_ss = prm.ss_out;
    asm volatile("" : "+r"(e_M), "+r"(e_N), "+r"(e_act), "+r"(e_f32), "+l"(e_out), "+f"(e_inv), "+f"(e_eps),
                      "+l"(e_res), "+l"(e_nw), "+l"(e_ss));
    const int n_out = e_act ? e_N / 2 : e_N;
    const int k_steps = kc >> 4;               // a multiple of kInFlight (beyond K the copy has filled in zeros)
    // The scale of the rows, if x stands for rows whose norm is still owed: the parts of their sums
    // of squares are asked for now and added up, in a fixed order, when the first pass ends.
    float ssq[2][kSsPerLane];
    if (SCALED) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int q = 0; q < kSsPerLane; ++q) {
                const int m = warp + kWarps * i, part = lane + 32 * q;
                ssq[i][q] = (m < e_M && part < prm.ss_parts) ? prm.ss_in[part * 16 + m] : 0.f;
            }
    }
    if (ADDS && lane == 0) ss_s[warp] = ss_s[warp + kWarps] = 0.f;
    int s = 0;
    uint32_t parity = 0;
    for (int pass = 0; pass < passes; ++pass) {
        float acc[kInFlight][NT][4];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) acc[u][nt][0] = acc[u][nt][1] = acc[u][nt][2] = acc[u][nt][3] = 0.f;
        const int pr0 = pass * rows_cap, prows = min(rows_cap, rows - pr0);
        const bool active = my_tile * 16 < prows;
        for (int kb = 0; kb < nk; ++kb) {
            if (ADDS && kb == 0) {
                // what the outputs of this pass are added to, on its way while the weights are
                // (each thread fetches what it will use itself)
                const size_t first = (size_t)(r0 + pr0);
                for (int m = warp; m < e_M; m += kWarps)
                    for (int j = lane; j < prows; j += 32)
                        cp_async_4(&res_s[m * 128 + j], e_res + (size_t)m * e_N + first + j);
                for (int j = lane; j < prows; j += 32) cp_async_4(&nw_s[warp * 128 + j], e_nw + first + j);
            }
            if (!mbar_wait(&full_w[s], parity, abort_flag) || !mbar_wait(&full_x[s], parity, abort_flag)) return;
            const uint32_t sw = smem_u32(ring + (size_t)s * stage_bytes);
            const uint32_t sx = sw + (uint32_t)w_bytes;
            if (active) {
                for (int ks0 = my_part * kInFlight; ks0 < k_steps; ks0 += parts * kInFlight) {
                    uint32_t a[kInFlight][4], b[kInFlight][NT][2];
#pragma unroll
                    for (int u = 0; u < kInFlight; ++u) {
                        const int ks = ks0 + u, piece = ks >> 2, chunk = (ks & 3) * 2;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            ldmatrix_x2(b[u][nt], sx + swz(piece * 8 * NT + nt * 8 + b_row, chunk + b_half));
                        ldmatrix_x4(a[u], sw + swz(piece * prows + my_tile * 16 + a_row, chunk + a_half));
                    }
#pragma unroll
                    for (int u = 0; u < kInFlight; ++u)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_bf16(acc[u][nt], a[u], b[u][nt][0], b[u][nt][1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == stages) { s = 0; parity ^= 1u; }
        }
        // every warp's sum into shared memory (two buffers by turns: one meeting a pass), then each
        // output is the sum of its tile's K parts, in their order
        float* buf = red + (size_t)(pass & 1) * kWarps * 16 * width;
        {
            float* mine = buf + (size_t)(my_part * rt + my_tile) * 16 * width;
            const int r = lane >> 2;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int c = nt * 8 + 2 * (lane & 3);
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = (acc[0][nt][e] + acc[1][nt][e]) + (acc[2][nt][e] + acc[3][nt][e]);
                *reinterpret_cast<float2*>(&mine[r * width + c]) = make_float2(v[0], v[1]);
                *reinterpret_cast<float2*>(&mine[(r + 8) * width + c]) = make_float2(v[2], v[3]);
            }
        }
        if (SCALED && pass == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float t = ((ssq[i][0] + ssq[i][1]) + (ssq[i][2] + ssq[i][3])) + ssq[i][4];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
                if (lane == 0) scale_s[warp + kWarps * i] = rsqrtf(t * e_inv + e_eps);
            }
        }
        if (ADDS) cp_async_wait_all();
        consumer_sync();
        const int n_local = e_act ? prows >> 1 : prows;
        const size_t first = e_act ? (size_t)((r0 + pr0) >> 1) : (size_t)(r0 + pr0);
        const int part_stride = rt * 16 * width;
        for (int m = warp; m < e_M; m += kWarps) {
        const float scale = SCALED ? scale_s[m] : 1.f;
        float ss_row = 0.f;
        for (int j = lane; j < n_local; j += 32) {
            float v;
            if (e_act) {
                const float* src = buf + (size_t)(2 * j) * width + m;      // (rows of tile t lie at 16 t ...)
                float g = 0.f, u = 0.f;
                for (int p = 0; p < parts; ++p) {
                    g += src[(size_t)p * part_stride];
                    u += src[(size_t)p * part_stride + width];
                }
                v = gate_act(g * scale, e_act) * (u * scale);
            } else {
                const float* src = buf + (size_t)j * width + m;
                v = 0.f;
                for (int p = 0; p < parts; ++p) v += src[(size_t)p * part_stride];
                v *= scale;
            }
            const size_t o = (size_t)m * n_out + first + j;
            if (ADDS) {
                const float h = res_s[m * 128 + j] + v;
                e_res[o] = h;
                ss_row += h * h;
                v = h * nw_s[warp * 128 + j];
            }
            if (e_f32) reinterpret_cast<float*>(e_out)[o] = v;
            else reinterpret_cast<bf16*>(e_out)[o] = __float2bfloat16_rn(v);
        }
        if (ADDS) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ss_row += __shfl_xor_sync(0xffffffffu, ss_row, off);
            if (lane == 0) ss_s[m] += ss_row;
        }
        }
    }
    if (ADDS && lane == 0)
        for (int m = warp; m < e_M; m += kWarps) e_ss[(size_t)blockIdx.x * 16 + m] = ss_s[m];
}

// ------------------------------------------------------------------------------- host
struct Plan {
    int rt, nt, kc, stages, unit, blocks;
    int rows_a, rows_b, rows_c;     // rows of a full pass, of the last pass of the longer blocks, of the shorter
    int rows_hi, rows_lo, n_hi;     // the first n_hi blocks have rows_hi rows, the others rows_lo
    int w_bytes;
    size_t smem;
};

static int sm_count() {
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

// The shape of the launch, or 0 if the kernel does not take the product: bfloat16, M <= 16, K a
// multiple of 64 (the width of a copied piece), an even number of rows for a gated product, and at
// least two stages within the shared-memory budget.
static int make_plan(int M, int N, int K, int act, int fold, int sms, Plan* p) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 64) return 0;
    if (act < 0 || act > LSB_ACT_NONE || (act && (N % 2))) return 0;
    p->unit = act ? 2 : 1;
    const int units = N / p->unit;
    p->blocks = units < sms ? units : sms;
    const int hi = ((units + p->blocks - 1) / p->blocks) * p->unit, lo = (units / p->blocks) * p->unit;
    p->rt = hi <= 16 ? 1 : hi <= 32 ? 2 : hi <= 64 ? 4 : 8;
    p->rows_hi = hi;
    p->rows_lo = lo;
    p->n_hi = hi == lo ? p->blocks : units - (lo / p->unit) * p->blocks;
    const int cap = 16 * p->rt;
    p->rows_a = hi < cap ? hi : cap;
    p->rows_b = hi - ((hi + cap - 1) / cap - 1) * cap;
    p->rows_c = lo - ((lo + cap - 1) / cap - 1) * cap;
    p->nt = M <= 8 ? 1 : 2;
    const size_t red = (size_t)(2 * kWarps * 16) * 8 * p->nt * sizeof(float);   // the warps' sums, two buffers
    const size_t tail = kTailBytes + (fold ? kFoldBytes : 0);
    const size_t room = (size_t)kSmemBudget - 1024 - tail - red;
    p->kc = 0;
    const int cands[5] = {1024, 512, 256, 128, 64};
    for (int c = 0; c < 5; ++c) {
        const int kc = cands[c];
        if (kc > K && kc != 128) continue;
        const size_t w_bytes = ((size_t)p->rows_a * kc * 2 + 1023) & ~(size_t)1023;
        const size_t stage = w_bytes + (size_t)(kc / 64) * 8 * p->nt * 128;
        // three stages at least, unless even the shortest chunk does not allow them
        if (3 * stage <= room || (kc <= 128 && 2 * stage <= room)) {
            p->kc = kc;
            p->w_bytes = (int)w_bytes;
            p->stages = (int)(room / stage);
            if (p->stages > kMaxStages) p->stages = kMaxStages;
            // no more stages than a block has chunks to walk: what a short product leaves of the
            // SM's shared memory lets blocks of the next kernel in beside it, to set themselves up
            const int walk = ((hi + cap - 1) / cap) * ((K + kc - 1) / kc);
            if (p->stages > walk) p->stages = walk < 2 ? 2 : walk;
            p->smem = 1024 + (size_t)p->stages * stage + red + tail;
            break;
        }
    }
    return p->kc != 0;
}

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

// A [rows, K] bf16 row-major matrix seen as (64 of K) x rows x (K / 64 pieces); boxes of
// 64 x box_rows x pieces, 128-byte swizzle, zeros outside.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows, int pieces) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return (int)cudaErrorNotSupported;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)pieces};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

LSB_API int lsb_gemm_stream_supported(const void* x, const void* w, int M, int N, int K, int act) {
    Plan p;
    return ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && make_plan(M, N, K, act, 1, sm_count(), &p) &&
           get_encode() != nullptr;
}

// The number of blocks a product of these sizes runs with: the parts its sums of squares come in.
LSB_API int lsb_gemm_stream_blocks(int M, int N, int K, int act) {
    Plan p;
    return make_plan(M, N, K, act, 1, sm_count(), &p) ? p.blocks : 0;
}

template <int NT, bool FOLDS>
static int launch(const CUtensorMap* maps, const StreamParams& prm, const Plan& p, const StreamWarm& warm,
                  cudaStream_t stream) {
    static int configured = -1;
    if (configured < 0)
        configured = (int)cudaFuncSetAttribute(gemm_stream_kernel<NT, FOLDS>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (configured) return configured;
    return lsb_launch(gemm_stream_kernel<NT, FOLDS>, dim3(p.blocks), dim3(kThreads), p.smem, stream, 1,
                      maps[0], maps[1], maps[2], maps[3], prm, warm);
}

// The product with an RMS norm folded into it on either side, so that the norm needs no kernel of
// its own between two products of a decode step.
//
// ss_in != null: x holds rows r * g (a residual row times the norm's weight, rounded to bfloat16)
// whose normalisation is still owed; ss_in[part * 16 + m] are `ss_parts` (<= 160) parts of
// sum(r[m]^2), and every output row is scaled by rsqrt(sum / size + eps) before the activation,
// which is the same as normalising x first: the scale is one number per row.
//
// residual != null (act == 0): the product is added to residual [M, N] (32-bit, in place), out
// is (residual * norm_w) in bfloat16, the input of the next product in the sense above, and
// ss_out[block * 16 + m] gets this block's part of sum(residual[m]^2) over its own columns;
// lsb_gemm_stream_blocks gives the number of parts.  All sums are taken in a fixed order.
//
// warm != null: a StreamWarm that lsb_gemm_stream_warm filled in for the streaming product that
// follows this one in the stream; its first weights are pulled toward L2 while this one ends.
LSB_API int lsb_gemm_stream_folded(const void* x, const void* w, void* out, int out_f32, int M, int N, int K,
                                   int act, const float* ss_in, int ss_parts, int size, float eps,
                                   float* residual, const float* norm_w, float* ss_out, const void* warm,
                                   cudaStream_t stream) {
    Plan p;
    if (!lsb_gemm_stream_supported(x, w, M, N, K, act)) return (int)cudaErrorInvalidValue;
    if (ss_in && (ss_parts <= 0 || ss_parts > 32 * kSsPerLane || size <= 0)) return (int)cudaErrorInvalidValue;
    if (residual && (act || out_f32 || !norm_w || !ss_out)) return (int)cudaErrorInvalidValue;
    make_plan(M, N, K, act, residual != nullptr, sm_count(), &p);
    StreamParams prm;
    prm.x = (const bf16*)x; prm.w = (const bf16*)w; prm.out = out;
    prm.M = M; prm.N = N; prm.K = K;
    prm.out_f32 = out_f32; prm.act = act;
    prm.kc = p.kc; prm.stages = p.stages; prm.unit = p.unit; prm.w_bytes = p.w_bytes;
    prm.rows_a = p.rows_a; prm.rows_b = p.rows_b; prm.rows_c = p.rows_c;
    prm.rt = p.rt;
    prm.rt_log2 = p.rt == 1 ? 0 : p.rt == 2 ? 1 : p.rt == 4 ? 2 : 3;
    prm.rows_hi = p.rows_hi; prm.rows_lo = p.rows_lo; prm.n_hi = p.n_hi; prm.nk = (K + p.kc - 1) / p.kc;
    prm.ss_in = ss_in; prm.ss_parts = ss_parts; prm.inv_size = ss_in ? 1.f / (float)size : 0.f; prm.eps = eps;
    prm.residual = residual; prm.norm_w = norm_w; prm.ss_out = ss_out;
    CUtensorMap maps[4];
    int rc;
    if ((rc = make_map(&maps[0], w, N, K, p.rows_a, p.kc / 64))) return rc;
    if ((rc = make_map(&maps[1], w, N, K, p.rows_b, p.kc / 64))) return rc;
    if ((rc = make_map(&maps[2], w, N, K, p.rows_c, p.kc / 64))) return rc;
    if ((rc = make_map(&maps[3], x, M, K, 8 * p.nt, p.kc / 64))) return rc;
    StreamWarm none;
    none.base = nullptr;
    none.blocks = 0;
    const StreamWarm& wm = warm ? *reinterpret_cast<const StreamWarm*>(warm) : none;
    if (ss_in || residual)
        return p.nt == 1 ? launch<1, true>(maps, prm, p, wm, stream) : launch<2, true>(maps, prm, p, wm, stream);
    return p.nt == 1 ? launch<1, false>(maps, prm, p, wm, stream) : launch<2, false>(maps, prm, p, wm, stream);
}

// Fills `out` (sizeof(StreamWarm) bytes, see lsb_stream_warm_bytes) with what the kernel before a
// streaming product of these sizes needs to warm it; `adds`: the product adds to the residual.
// Returns 0, or an error if the streaming kernel does not take the product.
LSB_API int lsb_gemm_stream_warm(const void* w, int M, int N, int K, int act, int adds, void* out) {
    Plan p;
    if (((uintptr_t)w % 16) || !make_plan(M, N, K, act, adds, sm_count(), &p)) return (int)cudaErrorInvalidValue;
    StreamWarm* sw = reinterpret_cast<StreamWarm*>(out);
    sw->base = reinterpret_cast<const unsigned char*>(w);
    sw->row_bytes = (long long)K * 2;
    sw->blocks = p.blocks;
    sw->rows_hi = p.rows_hi; sw->rows_lo = p.rows_lo; sw->n_hi = p.n_hi;
    sw->bytes = kWarmBytes;
    return 0;
}

LSB_API int lsb_stream_warm_bytes() { return (int)sizeof(StreamWarm); }

// x [M, K] and w [N, K] bfloat16; out [M, N] (or [M, N / 2] with act != 0) bfloat16 or (out_f32) float.
LSB_API int lsb_gemm_stream(const void* x, const void* w, void* out, int out_f32, int M, int N, int K,
                            int act, cudaStream_t stream) {
    return lsb_gemm_stream_folded(x, w, out, out_f32, M, N, K, act, nullptr, 0, 0, 0.f, nullptr, nullptr,
                                  nullptr, nullptr, stream);
}
