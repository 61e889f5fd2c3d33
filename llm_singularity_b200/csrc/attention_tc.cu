// Tensor-core attention over the paged cache for bfloat16: a split-KV kernel for single
// decode tokens and a tiled causal kernel for prompt portions, head sizes 64 and 128.
//
// Both walk a request's keys in tiles of 64 through its block table, stage K and V tiles in
// shared memory with 16-byte asynchronous copies (two stages, XOR-swizzled so that ldmatrix
// reads are free of bank conflicts), form scores with mma.sync m16n8k16 (bf16 in, 32-bit
// accumulate), keep the running maximum / sum / output of the online softmax in 32-bit
// registers, round the probabilities to bfloat16 only as the left operand of the P.V product,
// and divide by the sum at the end.
//
//  * decode: one thread block per (split, kv head, request).  The nh/nkv query heads that share
//    the kv head are the rows of one 16-row MMA tile, so every key and value is read once for
//    the whole group; each of the four warps pipelines its own 16-key chunks (four in flight,
//    no block barrier in the loop) and the warps merge through shared memory at the end; with
//    more than one split, partial (max, sum, output) go to scratch and a small merge kernel
//    finishes.  The split count depends only on the batch, and each split finds
//    its share of tiles from the request's length on the device, so a captured launch stays
//    valid as sequences grow.
//  * prefill: one thread block per (128-query tile, head, request); warp w of 8 owns rows
//    16w..16w+15; K/V tiles of 64 keys in a three-stage ring; tiles below the diagonal skip the mask.
//    Query row i of a request with q_len new tokens and kv_len cached tokens sits at position
//    p = kv_len - q_len + i and sees keys [max(0, p - window + 1), p].
//
// These replace the reference's paged_attention_kernel (kernels/src/attention.cu:27-172), which
// serves both cases with 32 threads per (head, row) and scalar fp32 loops.  The generic kernel in
// attention.cu remains the 32-bit path and the fallback for other head sizes.
#define LSB_CLUSTER_ALONG_X            // decode splits are blockIdx.x
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

typedef __nv_bfloat16 bf16;

constexpr int kTile = 64;        // keys per tile
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;       // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// D(16x8, f32) += A(16x16, bf16) * B(16x8, bf16)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (one MUFU.EX2; fast_exp2() adds range handling around it that the
// softmax does not need: arguments here are <= 0 and -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Rotates eight split-half pairs: lo holds x[i..i+7], hi holds x[i+half..], cs/sn their cosines
// and sines.
__device__ __forceinline__ void rotate8(uint4& lo, uint4& hi, const float* cs, const float* sn) {
    bf16* a = reinterpret_cast<bf16*>(&lo);
    bf16* b = reinterpret_cast<bf16*>(&hi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float x0 = __bfloat162float(a[e]), x1 = __bfloat162float(b[e]);
        a[e] = __float2bfloat16_rn(x0 * cs[e] - x1 * sn[e]);
        b[e] = __float2bfloat16_rn(x0 * sn[e] + x1 * cs[e]);
    }
}

// thread-block cluster helpers: rank, barrier over all threads of all blocks, a float from a peer
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(const float* own_smem, uint32_t rank) {
    uint32_t peer;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(smem_u32(own_smem)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
    return v;
}

// A tile is rows of HD bf16 = HD/8 chunks of 16 bytes; chunk c of row r lives at chunk c ^ (r & 7).
template <int HD> __device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int chunk) {
    return base + (row * (HD / 8) + (chunk ^ (row & 7))) * 8;
}

// ------------------------------------------------------------------ decode
#ifndef LSB_DEC_CHUNK
#define LSB_DEC_CHUNK 16
#endif
#ifndef LSB_DEC_STAGES
#define LSB_DEC_STAGES 2
#endif
constexpr int kChunk = LSB_DEC_CHUNK;           // keys a warp handles per step
constexpr int kDecStages = LSB_DEC_STAGES;        // chunks in flight per warp
constexpr int kBtCache = 1024;       // block-table entries kept in shared memory per block

__device__ __forceinline__ int div_page(int key, int page_size, int page_shift) {
    return page_shift >= 0 ? key >> page_shift : key / page_size;
}

// Each warp runs its own pipeline over every fourth 16-key chunk of the block's key range:
// asynchronous 16-byte copies of the chunk's K and V rows into the warp's ring of stages, no
// block-wide barrier inside the loop.  The block's slice of the block table is read into shared
// memory first, so that copies are issued without waiting on a table lookup.
#ifndef LSB_DEC_MINBLOCKS
#define LSB_DEC_MINBLOCKS 4
#endif
template <int HD, bool LOW8>
__global__ void __launch_bounds__(kThreads, HD == 64 ? LSB_DEC_MINBLOCKS : 3)
decode_attention_kernel(const bf16* __restrict__ qkv, int qkv_stride,
                        bf16* k_pages, bf16* v_pages,
                        const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
                        const int* __restrict__ table_rows, const int* __restrict__ block_table,
                        int table_stride, bf16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int nh, int nkv, int page_size, int num_pages,
                        float scale, int window, int splits, int cluster_merge,
                        const float* __restrict__ inv_freq, int rotary_dim, int store_kv) {
    constexpr int CPR = HD / 8, KS = HD / 16;
    constexpr int kStageElems = 2 * kChunk * HD;             // K rows then V rows
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);            // [16][HD]
    bf16* sKV = sQ + 16 * HD;                                // [4 warps][stages][K|V][16][HD]
    int* sBT = reinterpret_cast<int*>(sKV + 4 * kDecStages * kStageElems);
    float* sCS = reinterpret_cast<float*>(sBT + kBtCache);   // [cos HD/2][sin HD/2] of the position
    lsb_pdl_launch_dependents();

    // Before the wait on the previous kernel, what does not depend on it.  The step's metadata was
    // copied to the device before the step's first kernel started, and the kernels that patch the
    // block tables let nothing start before they have completed (cache_table.cu), so the block's
    // key range, the sines and cosines of the token's position, its slice of the block table and
    // the first keys and values of every warp can be had while the projection is still being
    // computed.  Only the chunk that holds the token's own position must wait: its last row is
    // written during this step (by this kernel, the rotary kernel or another layer's).
    const int split = blockIdx.x, g = blockIdx.y, r = blockIdx.z;
    const int qs = q_start[r];
    const bool single = q_start[r + 1] - qs == 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = nh / nkv;
    const int kv_len = kv_len_arr[r];
    const int p = kv_len - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    const int first_chunk = lo / kChunk;
    const int n_chunks = p / kChunk + 1 - first_chunk;
    const int per = (n_chunks + splits - 1) / splits;
    const int c0 = first_chunk + split * per;
    const int c1 = min(c0 + per, first_chunk + n_chunks);

    // this block's slice of the block table
    const int page0 = div_page(c0 * kChunk, page_size, page_shift);
    const int n_pages_here = c1 > c0 ? div_page(c1 * kChunk - 1, page_size, page_shift) - page0 + 1 : 0;
    const bool cached = n_pages_here <= kBtCache;
    const int half = rotary_dim >> 1;                        // rotated pairs: dims (i, i + half), i < half
    if (inv_freq && single)
        for (int i = threadIdx.x; i < half; i += kThreads)
            sincosf((float)p * inv_freq[i], &sCS[half + i], &sCS[i]);

    if (single && cached)                                    // from L2: another SM wrote it
        for (int idx = threadIdx.x; idx < n_pages_here; idx += kThreads)
            sBT[idx] = (page0 + idx < table_stride) ? __ldcg(bt + page0 + idx) : -1;
    __syncthreads();

    bf16* ring = sKV + (size_t)warp * kDecStages * kStageElems;
    const int n_mine = (c1 - c0 - warp + 3) / 4;             // chunks c0 + warp, c0 + warp + 4, ...
    auto issue = [&](int i) {
        if (i < n_mine) {
            const int chunk = c0 + warp + 4 * i;
            bf16* dK = ring + (size_t)(i % kDecStages) * kStageElems;
            bf16* dV = dK + kChunk * HD;
            if (page_shift >= 0 && page_size >= kChunk) {
                // the chunk lies inside one page: one table entry, then a contiguous run of rows
                const int key0 = chunk * kChunk;
                const int pi = key0 >> page_shift;
                const int page = cached ? sBT[pi - page0] : (pi < table_stride ? bt[pi] : -1);
                const bool page_ok = page >= 0 && page < num_pages;
                if (!page_ok) lsb_set_status(LSB_BAD_PAGE);
                const long long base = page_ok
                    ? (((long long)page * nkv + g) * page_size + (key0 - (pi << page_shift))) * HD : 0;
                const bf16* srcK = k_pages + base;
                const bf16* srcV = v_pages + base;
#pragma unroll
                for (int idx = lane; idx < kChunk * CPR; idx += 32) {
                    const int kk = idx / CPR, c = idx - kk * CPR;
                    const bool valid = page_ok && key0 + kk >= lo && key0 + kk <= p;
                    const int off = valid ? idx * 8 : 0;
                    cp_async16(tile_ptr<HD>(dK, kk, c), srcK + off, valid);
                    cp_async16(tile_ptr<HD>(dV, kk, c), srcV + off, valid);
                }
            } else
#pragma unroll
            for (int idx = lane; idx < kChunk * CPR; idx += 32) {
                const int kk = idx / CPR, c = idx - kk * CPR;
                const int key = chunk * kChunk + kk;
                bool valid = key >= lo && key <= p;
                long long off = 0;
                if (valid) {
                    const int pi = div_page(key, page_size, page_shift);
                    const int page = cached ? sBT[pi - page0] : (pi < table_stride ? bt[pi] : -1);
                    if (page < 0 || page >= num_pages) {
                        lsb_set_status(LSB_BAD_PAGE);
                        valid = false;
                    } else {
                        const int within = key - pi * page_size;
                        off = (((long long)page * nkv + g) * page_size + within) * HD + c * 8;
                    }
                }
                cp_async16(tile_ptr<HD>(dK, kk, c), k_pages + off, valid);
                cp_async16(tile_ptr<HD>(dV, kk, c), v_pages + off, valid);
            }
        }
        cp_async_commit();
    };

    // the warp's first chunks are on their way before the wait if none of them is the last one
    const bool early = single && cached && c0 + warp + 4 * (kDecStages - 2) < p / kChunk;
    if (early) {
#pragma unroll
        for (int i = 0; i < kDecStages - 1; ++i) issue(i);
    }

    lsb_pdl_wait();
    if (!single) return;                                     // prompt portions go to the other kernel

    const bf16* tok = qkv + (size_t)qs * qkv_stride;          // this token's row of the projection
    if (inv_freq) {
        // The projection comes unrotated: the rotation of the queries and of the new key happens
        // here (split-half pairs (i, i + rotary_dim / 2), angle p * inv_freq[i] in 32-bit, as the
        // separate rotary kernel forms it; dims from rotary_dim on pass through), and the block
        // whose key range holds position p writes the new key and value into their page before
        // anybody's copies start.
        const int HC = half >> 3;                               // 16-byte chunks per rotated half
        const int per_row = CPR - HC;                           // work items a row: HC pairs, then the plain chunks
        __syncthreads();                                        // the sines and cosines formed above
        for (int idx = threadIdx.x; idx < 16 * per_row; idx += kThreads) {
            const int row = idx / per_row, c = idx - row * per_row;
            const bf16* src = tok + (size_t)(g * G + row) * HD;
            if (c < HC) {
                uint4 vlo = make_uint4(0, 0, 0, 0), vhi = make_uint4(0, 0, 0, 0);
                if (row < G) {
                    vlo = *reinterpret_cast<const uint4*>(src + c * 8);
                    vhi = *reinterpret_cast<const uint4*>(src + half + c * 8);
                    rotate8(vlo, vhi, sCS + c * 8, sCS + half + c * 8);
                }
                *reinterpret_cast<uint4*>(tile_ptr<HD>(sQ, row, c)) = vlo;
                *reinterpret_cast<uint4*>(tile_ptr<HD>(sQ, row, c + HC)) = vhi;
            } else {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row < G) v = *reinterpret_cast<const uint4*>(src + (c + HC) * 8);
                *reinterpret_cast<uint4*>(tile_ptr<HD>(sQ, row, c + HC)) = v;
            }
        }
        const int pc = p / kChunk;
        if (store_kv && pc >= c0 && pc < c1) {
            const int pi = div_page(p, page_size, page_shift);
            const int page = pi < table_stride ? bt[pi] : -1;
            if (page < 0 || page >= num_pages) {
                if (threadIdx.x == 0) lsb_set_status(LSB_BAD_PAGE);
            } else {
                const long long dst = (((long long)page * nkv + g) * page_size + (p - pi * page_size)) * HD;
                if (threadIdx.x < HC) {
                    const int c = threadIdx.x;
                    const bf16* src = tok + (size_t)(nh + g) * HD;
                    uint4 vlo = *reinterpret_cast<const uint4*>(src + c * 8);
                    uint4 vhi = *reinterpret_cast<const uint4*>(src + half + c * 8);
                    rotate8(vlo, vhi, sCS + c * 8, sCS + half + c * 8);
                    *reinterpret_cast<uint4*>(k_pages + dst + c * 8) = vlo;
                    *reinterpret_cast<uint4*>(k_pages + dst + half + c * 8) = vhi;
                } else if (threadIdx.x < per_row) {               // the key's dims beyond the rotated ones
                    const int c = threadIdx.x + HC;
                    *reinterpret_cast<uint4*>(k_pages + dst + c * 8) =
                        *reinterpret_cast<const uint4*>(tok + (size_t)(nh + g) * HD + c * 8);
                } else if (threadIdx.x >= 32 && threadIdx.x < 32 + CPR) {
                    const int c = threadIdx.x - 32;
                    *reinterpret_cast<uint4*>(v_pages + dst + c * 8) =
                        *reinterpret_cast<const uint4*>(tok + (size_t)(nh + nkv + g) * HD + c * 8);
                }
            }
        }
    } else {
        // queries of the group: rows 0..G-1 of a 16-row tile, the rest zero
        for (int idx = threadIdx.x; idx < 16 * CPR; idx += kThreads) {
            const int row = idx / CPR, c = idx - row * CPR;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < G)
                v = *reinterpret_cast<const uint4*>(tok + (size_t)(g * G + row) * HD + c * 8);
            *reinterpret_cast<uint4*>(tile_ptr<HD>(sQ, row, c)) = v;
        }
    }
    __syncthreads();            // also orders the new key and value before the copies below

    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], tile_ptr<HD>(sQ, ((lane >> 3) & 1) * 8 + (lane & 7), 2 * ks + (lane >> 4)));

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float sc = scale * kLog2e;

    if (!early) {
#pragma unroll
        for (int i = 0; i < kDecStages - 1; ++i) issue(i);
    }

    for (int i = 0; i < n_mine; ++i) {
        issue(i + kDecStages - 1);
        cp_async_wait<kDecStages - 1>();
        __syncwarp();
        const int chunk = c0 + warp + 4 * i;
        bf16* tK = ring + (size_t)(i % kDecStages) * kStageElems;
        bf16* tV = tK + kChunk * HD;

        constexpr int NT = kChunk / 8;                         // 8-key score tiles per chunk
        float s[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, tile_ptr<HD>(tK, np * 16 + (lane >> 4) * 8 + (lane & 7), 2 * ks + ((lane >> 3) & 1)));
                mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        // Rows 8..15 of the tile hold no query when the group has at most 8 heads: NR is the number
        // of row halves with work, and everything scalar below skips the other one.
        constexpr int NR = LOW8 ? 1 : 2;
        constexpr int NE = 2 * NR;
        float mx[2] = {-INFINITY, -INFINITY};
        const int key0 = chunk * kChunk;
        if (key0 >= lo && key0 + kChunk - 1 <= p) {            // whole chunk in range: no mask
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < NE; ++e) {
                    s[nt][e] *= sc;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
        } else {
            // mask keys outside [lo, p]; scale into the log2 domain
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < NE; ++e) {
                    const int key = key0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                    const float v = (key >= lo && key <= p) ? s[nt][e] * sc : -INFINITY;
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
        }
        float mref[2] = {0.f, 0.f};
        bool moved = false;
#pragma unroll
        for (int h = 0; h < NR; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            moved = moved || mx[h] > m[h];
        }
        if (__any_sync(0xffffffffu, moved)) {                  // rare once the first chunks are in
            float corr[2] = {1.f, 1.f};
#pragma unroll
            for (int h = 0; h < NR; ++h) {
                const float m_new = fmaxf(m[h], mx[h]);
                corr[h] = (m[h] == -INFINITY) ? 0.f : fast_exp2(m[h] - m_new);
                m[h] = m_new;
                l[h] *= corr[h];
            }
#pragma unroll
            for (int i2 = 0; i2 < HD / 8; ++i2) {
                o[i2][0] *= corr[0]; o[i2][1] *= corr[0];
                if (!LOW8) { o[i2][2] *= corr[1]; o[i2][3] *= corr[1]; }
            }
        }
#pragma unroll
        for (int h = 0; h < NR; ++h) mref[h] = m[h] == -INFINITY ? 0.f : m[h];   // ex2(-inf - 0) = 0
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const float pv = fast_exp2(s[nt][e] - mref[e >> 1]);
                s[nt][e] = pv;
                l[e >> 1] += pv;
            }
#pragma unroll
        for (int kt = 0; kt < NT / 2; ++kt) {
            uint32_t pa[4] = {pack_bf16(s[2 * kt][0], s[2 * kt][1]), 0u,
                              pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]), 0u};
            if (!LOW8) {
                pa[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
                pa[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
            }
#pragma unroll
            for (int dt = 0; dt < HD / 16; ++dt) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, tile_ptr<HD>(tV, kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), 2 * dt + (lane >> 4)));
                mma_bf16(o[2 * dt], pa, b[0], b[1]);
                mma_bf16(o[2 * dt + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();                                          // the stage is overwritten next round
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }

    // merge the four warps (each saw different keys) through shared memory
    float* sO = reinterpret_cast<float*>(sKV);                 // [4][16][HD]
    float* sM = sO + 4 * 16 * HD;                              // [4][16]
    float* sL = sM + 4 * 16;
    float* sFin = sL + 4 * 16;                                 // [G][HD] this block's merged output
    float* sFinML = sFin + 16 * HD;                            // [G][2] its (max, sum)
    __syncthreads();
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * (lane & 3);
        float* dst = sO + ((warp * 16 + (lane >> 2)) * HD + d);
        dst[0] = o[i][0]; dst[1] = o[i][1];
        dst[8 * HD] = o[i][2]; dst[8 * HD + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
        sM[warp * 16 + (lane >> 2)] = m[0]; sM[warp * 16 + (lane >> 2) + 8] = m[1];
        sL[warp * 16 + (lane >> 2)] = l[0]; sL[warp * 16 + (lane >> 2) + 8] = l[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += kThreads) {
        const int h = idx / HD, d = idx - h * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 16 + h]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sM[w * 16 + h];
            const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L += sL[w * 16 + h] * f;
            O += sO[(w * 16 + h) * HD + d] * f;
        }
        const int head = g * G + h;
        if (splits == 1) {
            out[(size_t)qs * nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else if (cluster_merge) {
            sFin[idx] = O;
            if (d == 0) { sFinML[2 * h] = M; sFinML[2 * h + 1] = L; }
        } else {
            const size_t slot = ((size_t)r * nh + head) * splits + split;
            part_o[slot * HD + d] = O;
            if (d == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
        }
    }
    if (splits > 1 && cluster_merge) {
        // The splits of one (request, kv head) are one cluster: every block takes a share of the
        // group's outputs and sums all blocks' partial results, read from their shared memory in
        // rank order, so nothing goes through global memory and no second kernel is needed.
        cluster_barrier();
        const uint32_t rank = cluster_rank();
        for (int idx = (int)rank * kThreads + threadIdx.x; idx < G * HD; idx += splits * kThreads) {
            const int h = idx / HD, d = idx - h * HD;
            float M = -INFINITY;
            for (int s2 = 0; s2 < splits; ++s2) M = fmaxf(M, ld_peer_f32(sFinML + 2 * h, (uint32_t)s2));
            float L = 0.f, O = 0.f;
            for (int s2 = 0; s2 < splits; ++s2) {
                const float ms = ld_peer_f32(sFinML + 2 * h, (uint32_t)s2);
                const float f = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
                L += ld_peer_f32(sFinML + 2 * h + 1, (uint32_t)s2) * f;
                O += ld_peer_f32(sFin + idx, (uint32_t)s2) * f;
            }
            out[(size_t)qs * nh * HD + (size_t)(g * G + h) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
        cluster_barrier();          // nobody leaves while a peer may still read its shared memory
    }
}

// out[t, head, :] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
template <int HD>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ q_start, bf16* __restrict__ out, int nh,
                                    int splits) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int head = blockIdx.x, r = blockIdx.y;
    const int qs = q_start[r];
    if (q_start[r + 1] - qs != 1) return;
    const size_t base = ((size_t)r * nh + head) * splits;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float L = 0.f, O = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(base + s) * 2];
            const float f = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
            L += part_ml[(base + s) * 2 + 1] * f;
            O += part_o[(base + s) * HD + d] * f;
        }
        out[(size_t)qs * nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
}

// ------------------------------------------------------------------ prefill
constexpr int kPfRows = 128;         // query rows per block (8 warps x 16)
constexpr int kPfThreads = 256;
constexpr int kPfStages = 3;

// Stage one 64-key tile of K and V for the prefill kernel: 256 threads, the block's slice of the
// block table already in shared memory.
template <int HD>
__device__ __forceinline__ void pf_load_tile(bf16* sK, bf16* sV, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages, const int* __restrict__ bt,
                                             const int* sBT, bool cached, int page0, int table_stride,
                                             int tile, int lo, int hi, int g, int nkv, int page_size,
                                             int page_shift, int num_pages) {
    constexpr int CPR = HD / 8;
#pragma unroll
    for (int idx = threadIdx.x; idx < kTile * CPR; idx += kPfThreads) {
        const int kk = idx / CPR, c = idx - kk * CPR;
        const int key = tile * kTile + kk;
        bool valid = key >= lo && key <= hi;
        long long off = 0;
        if (valid) {
            const int pi = div_page(key, page_size, page_shift);
            const int page = cached ? sBT[pi - page0] : (pi < table_stride ? bt[pi] : -1);
            if (page < 0 || page >= num_pages) {
                lsb_set_status(LSB_BAD_PAGE);
                valid = false;
            } else {
                off = (((long long)page * nkv + g) * page_size + (key - pi * page_size)) * HD + c * 8;
            }
        }
        cp_async16(tile_ptr<HD>(sK, kk, c), k_pages + off, valid);
        cp_async16(tile_ptr<HD>(sV, kk, c), v_pages + off, valid);
    }
}

template <int HD>
__global__ void __launch_bounds__(kPfThreads)
prefill_attention_kernel(const bf16* __restrict__ qkv, int qkv_stride,
                         const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                         const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
                         const int* __restrict__ table_rows, const int* __restrict__ block_table,
                         int table_stride, bf16* __restrict__ out, int nh, int nkv, int page_size,
                         int num_pages, float scale, int window, int skip_single) {
    constexpr int CPR = HD / 8, KS = HD / 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);            // [128][HD]
    bf16* sK = sQ + kPfRows * HD;                            // [stages][64][HD]
    bf16* sV = sK + kPfStages * kTile * HD;
    int* sBT = reinterpret_cast<int*>(sV + kPfStages * kTile * HD);
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();

    // grid: x = head (fastest), y = query tile, z = request, so that across all heads the heavy
    // tiles (late rows see the most keys) are handed out first and the light ones fill the tail
    const int r = blockIdx.z, h = blockIdx.x;
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int n_qt = (q_len + kPfRows - 1) / kPfRows;
    if ((int)blockIdx.y >= n_qt || (skip_single && q_len == 1)) return;
    const int i0 = (n_qt - 1 - (int)blockIdx.y) * kPfRows;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (nh / nkv);
    const int kv_len = kv_len_arr[r];
    const int p0 = kv_len - q_len + i0;                       // position of the tile's first row
    const int rows = min(kPfRows, q_len - i0);
    const int p_last = p0 + rows - 1;
    const int lo_cta = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    const int t0 = lo_cta / kTile, t1 = p_last / kTile + 1;

    const int page0 = div_page(t0 * kTile, page_size, page_shift);
    const int n_pages_here = div_page(p_last, page_size, page_shift) - page0 + 1;
    const bool cached = n_pages_here <= kBtCache;
    if (cached)
        for (int idx = threadIdx.x; idx < n_pages_here; idx += kPfThreads)
            sBT[idx] = (page0 + idx < table_stride) ? bt[page0 + idx] : -1;
    for (int idx = threadIdx.x; idx < kPfRows * CPR; idx += kPfThreads) {
        const int row = idx / CPR, c = idx - row * CPR;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows)
            v = *reinterpret_cast<const uint4*>(qkv + (size_t)(qs + i0 + row) * qkv_stride + (size_t)h * HD + c * 8);
        *reinterpret_cast<uint4*>(tile_ptr<HD>(sQ, row, c)) = v;
    }
    __syncthreads();

    auto issue = [&](int t) {
        if (t < t1) {
            const int st = (t - t0) % kPfStages;
            pf_load_tile<HD>(sK + st * kTile * HD, sV + st * kTile * HD, k_pages, v_pages, bt, sBT, cached, page0,
                             table_stride, t, lo_cta, p_last, g, nkv, page_size, page_shift, num_pages);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < kPfStages - 1; ++i) issue(t0 + i);

    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], tile_ptr<HD>(sQ, warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), 2 * ks + (lane >> 4)));

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float sc = scale * kLog2e;
    // this thread's two rows and their positions
    const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
    const int pos[2] = {p0 + row_a, p0 + row_b};
    const bool live[2] = {row_a < rows, row_b < rows};
    const int warp_first = p0 + warp * 16;                     // position of the warp's first row
    const int warp_hi = p0 + min(warp * 16 + 15, rows - 1);    // last position any row of the warp sees
    const int warp_lo = (window > 0) ? max(0, warp_first - window + 1) : 0;
    const bool warp_live = warp * 16 < rows;

    for (int t = t0; t < t1; ++t) {
        cp_async_wait<kPfStages - 2>();
        __syncthreads();                                       // tile t has landed; tile t-1 is free
        issue(t + kPfStages - 1);
        const int stage = (t - t0) % kPfStages;
        bf16* tK = sK + stage * kTile * HD;
        bf16* tV = sV + stage * kTile * HD;
        const int key0 = t * kTile;
        // a warp whose rows see none of this tile's keys only keeps the barriers
        if (warp_live && key0 <= warp_hi && key0 + kTile - 1 >= warp_lo) {
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, tile_ptr<HD>(tK, np * 16 + (lane >> 4) * 8 + (lane & 7), 2 * ks + ((lane >> 3) & 1)));
                    mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
                }
            // tiles wholly inside every row's range need no mask: all keys <= the warp's first
            // position, all keys inside the window of its last, all 16 rows present
            const bool full = key0 + kTile - 1 <= warp_first && warp * 16 + 15 < rows &&
                              (window <= 0 || key0 > warp_hi - window);
            float mx[2] = {-INFINITY, -INFINITY};
            if (full) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        s[nt][e] *= sc;
                        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                    }
            } else {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                        const int hh = e >> 1;
                        const bool ok = live[hh] && key <= pos[hh] && (window <= 0 || key > pos[hh] - window);
                        const float v = ok ? s[nt][e] * sc : -INFINITY;
                        s[nt][e] = v;
                        mx[hh] = fmaxf(mx[hh], v);
                    }
            }
            float corr[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                const float m_new = fmaxf(m[hh], mx[hh]);
                corr[hh] = (m[hh] == -INFINITY) ? 0.f : fast_exp2(m[hh] - m_new);
                m[hh] = m_new;
                l[hh] *= corr[hh];
            }
            // a row with no key yet keeps m = -inf; fast_exp2(-inf - (-inf)) must not be formed
            const float mref[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = fast_exp2(s[nt][e] - mref[e >> 1]);      // fast_exp2(-inf) = 0
                    s[nt][e] = pv;
                    l[e >> 1] += pv;
                }
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
                uint32_t pa[4] = {pack_bf16(s[2 * kt][0], s[2 * kt][1]), pack_bf16(s[2 * kt][2], s[2 * kt][3]),
                                  pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]),
                                  pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3])};
#pragma unroll
                for (int dt = 0; dt < HD / 16; ++dt) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, tile_ptr<HD>(tV, kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), 2 * dt + (lane >> 4)));
                    mma_bf16(o[2 * dt], pa, b[0], b[1]);
                    mma_bf16(o[2 * dt + 1], pa, b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
    const float inv[2] = {l[0] > 0.f ? 1.f / l[0] : 0.f, l[1] > 0.f ? 1.f / l[1] : 0.f};
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * (lane & 3);
        if (live[0]) {
            bf16* dst = out + (size_t)(qs + i0 + row_a) * nh * HD + (size_t)h * HD + d;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o[i][0] * inv[0], o[i][1] * inv[0]);
        }
        if (live[1]) {
            bf16* dst = out + (size_t)(qs + i0 + row_b) * nh * HD + (size_t)h * HD + d;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o[i][2] * inv[1], o[i][3] * inv[1]);
        }
    }
}

// ------------------------------------------------------------------ host side
template <int HD> constexpr size_t decode_smem() {
    return (16 * HD + 4 * kDecStages * 2 * kChunk * HD) * sizeof(bf16) + kBtCache * sizeof(int) +
           HD * sizeof(float);
}
template <int HD> constexpr size_t prefill_smem() {
    return (kPfRows * HD + 2 * kPfStages * kTile * HD) * sizeof(bf16) + kBtCache * sizeof(int);
}

template <int HD> static int configure_once() {
    static int done = -1;
    if (done >= 0) return done;
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<HD, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<HD>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_attention_kernel<HD, false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<HD>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(prefill_attention_kernel<HD>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem<HD>());
    done = (int)e;
    return done;
}

// The largest cluster the decode kernel may be launched with: 16 (beyond the portable 8) where the
// device says that such a cluster of these blocks can be resident, else 8.
template <int HD> static int max_cluster() {
    static int value = 0;
    if (value) return value;
    value = 8;
    if (configure_once<HD>()) return value;
    bool ok = true;
    for (int low8 = 0; low8 < 2 && ok; ++low8) {
        auto kernel = low8 ? decode_attention_kernel<HD, true> : decode_attention_kernel<HD, false>;
        ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        if (!ok) break;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(16, 1, 1);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = decode_smem<HD>();
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 16; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int n = 0;
        ok = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0;
    }
    (void)cudaGetLastError();
    if (ok) value = 16;
    return value;
}

// Blocks of the decode kernel that fit an SM at once (registers and shared memory), for query groups
// of `group` heads: what the number of key splits is sized by.
LSB_API int lsb_decode_blocks_per_sm(int hd, int group) {
    if ((hd != 64 && hd != 128) || group < 1) return 1;
    if ((hd == 64 ? configure_once<64>() : configure_once<128>())) return 1;
    int n = 0;
    cudaError_t e;
    if (hd == 64)
        e = group <= 8 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_attention_kernel<64, true>, kThreads, decode_smem<64>())
                       : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_attention_kernel<64, false>, kThreads, decode_smem<64>());
    else
        e = group <= 8 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_attention_kernel<128, true>, kThreads, decode_smem<128>())
                       : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_attention_kernel<128, false>, kThreads, decode_smem<128>());
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 1; }
    return n < 1 ? 1 : n;
}

LSB_API int lsb_decode_max_cluster(int hd) { return hd == 64 ? max_cluster<64>() : hd == 128 ? max_cluster<128>() : 8; }

// floats of scratch the decode kernel needs for `splits` > 1: outputs, then (max, sum) pairs
LSB_API long long lsb_decode_scratch_floats(int n_requests, int nh, int hd, int splits) {
    return splits <= 1 ? 0 : (long long)n_requests * nh * splits * (hd + 2);
}

// Single decode tokens (requests with q_len == 1; others are skipped).  bf16, hd 64 or 128,
// nh / nkv <= 16.  `scratch` holds lsb_decode_scratch_floats floats when splits > 1.
static int decode_launch(const void* qkv, int qkv_stride, void* k_pages, void* v_pages,
                         const int* q_start, const int* kv_len, const int* table_rows,
                         const int* block_table, int table_stride, void* out, float* scratch,
                         int n_requests, int nh, int nkv, int hd, int page_size, int num_pages,
                         float scale, int window, int splits, const float* inv_freq, int rotary_dim,
                         int store_kv, int max_cluster_size, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh / nkv > 16 || splits < 1 || n_requests > 65535 || nkv > 65535)
        return (int)cudaErrorInvalidValue;
    // up to this many splits merge inside a thread-block cluster (0: as many as the device takes)
    const int cluster_cap = max_cluster_size > 0 ? max_cluster_size : lsb_decode_max_cluster(hd);
    if (splits > cluster_cap && !scratch) return (int)cudaErrorInvalidValue;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_requests * nh * splits * hd : nullptr;
    dim3 grid(splits, nkv, n_requests);
    const bool in_cluster = splits > 1 && splits <= cluster_cap;      // x is the cluster dimension
#define LAUNCH_DECODE(HD)                                                                          \
    do {                                                                                           \
        int rc = configure_once<HD>();                                                             \
        if (rc) return rc;                                                                         \
        rc = lsb_launch(nh / nkv <= 8 ? decode_attention_kernel<HD, true>                          \
                                      : decode_attention_kernel<HD, false>,                        \
            grid, dim3(kThreads), decode_smem<HD>(), stream,                                       \
            in_cluster ? splits : 1,                                                               \
            (const bf16*)qkv, qkv_stride, (bf16*)k_pages, (bf16*)v_pages, q_start,                \
            kv_len, table_rows, block_table, table_stride, (bf16*)out, part_o, part_ml, nh, nkv,  \
            page_size, num_pages, scale, window, splits, in_cluster ? 1 : 0, inv_freq, rotary_dim,  \
            store_kv);                                                                             \
        if (rc) return rc;                                                                         \
        if (splits > 1 && !in_cluster)                                                             \
            rc = lsb_launch(decode_merge_kernel<HD>, dim3(nh, n_requests), dim3(64), 0, stream, 1, \
                (const float*)part_o, (const float*)part_ml, q_start, (bf16*)out, nh, splits);     \
        if (rc) return rc;                                                                         \
    } while (0)
    if (hd == 64) LAUNCH_DECODE(64);
    else if (hd == 128) LAUNCH_DECODE(128);
    else return (int)cudaErrorInvalidValue;
#undef LAUNCH_DECODE
    return 0;
}

LSB_API int lsb_decode_attention(const void* qkv, int qkv_stride, const void* k_pages, const void* v_pages,
                                 const int* q_start, const int* kv_len, const int* table_rows,
                                 const int* block_table, int table_stride, void* out, float* scratch,
                                 int n_requests, int nh, int nkv, int hd, int page_size, int num_pages,
                                 float scale, int window, int splits, cudaStream_t stream) {
    return decode_launch(qkv, qkv_stride, const_cast<void*>(k_pages), const_cast<void*>(v_pages), q_start,
                         kv_len, table_rows, block_table, table_stride, out, scratch, n_requests, nh, nkv,
                         hd, page_size, num_pages, scale, window, splits, nullptr, 0, 0, 0, stream);
}

// The same over a projection that has not been rotated yet: the kernel rotates the queries and the
// new key by `inv_freq` (rotary_dim / 2 entries; rotary_dim a multiple of 16, at most hd: the dims
// from there on pass through) at position kv_len - 1 and, if `store_kv`, writes the new key and
// value into their page.  Replaces the separate rotary kernel
// for single decode tokens.
LSB_API int lsb_decode_attention_rope(const void* qkv, int qkv_stride, void* k_pages, void* v_pages,
                                      const int* q_start, const int* kv_len, const int* table_rows,
                                      const int* block_table, int table_stride, void* out, float* scratch,
                                      int n_requests, int nh, int nkv, int hd, int page_size,
                                      int num_pages, float scale, int window, int splits,
                                      const float* inv_freq, int rotary_dim, int store_kv,
                                      cudaStream_t stream) {
    if (!inv_freq || rotary_dim < 16 || rotary_dim % 16 || rotary_dim > hd)
        return (int)cudaErrorInvalidValue;
    return decode_launch(qkv, qkv_stride, k_pages, v_pages, q_start, kv_len, table_rows, block_table,
                         table_stride, out, scratch, n_requests, nh, nkv, hd, page_size, num_pages,
                         scale, window, splits, inv_freq, rotary_dim, store_kv, 0, stream);
}

// Prompt portions (and, unless skip_single, single tokens too).  bf16, hd 64 or 128.
LSB_API int lsb_prefill_attention(const void* qkv, int qkv_stride, const void* k_pages, const void* v_pages,
                                  const int* q_start, const int* kv_len, const int* table_rows,
                                  const int* block_table, int table_stride, void* out, int n_requests,
                                  int max_q_len, int nh, int nkv, int hd, int page_size, int num_pages,
                                  float scale, int window, int skip_single, cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (nkv <= 0 || nh % nkv || n_requests > 65535 || (max_q_len + kPfRows - 1) / kPfRows > 65535)
        return (int)cudaErrorInvalidValue;
    dim3 grid(nh, (max_q_len + kPfRows - 1) / kPfRows, n_requests);
#define LAUNCH_PREFILL(HD)                                                                         \
    do {                                                                                           \
        int rc = configure_once<HD>();                                                             \
        if (rc) return rc;                                                                         \
        rc = lsb_launch(prefill_attention_kernel<HD>, grid, dim3(kPfThreads), prefill_smem<HD>(), stream, 1, \
            (const bf16*)qkv, qkv_stride, (const bf16*)k_pages, (const bf16*)v_pages, q_start,    \
            kv_len, table_rows, block_table, table_stride, (bf16*)out, nh, nkv, page_size,        \
            num_pages, scale, window, skip_single);                                                \
        if (rc) return rc;                                                                         \
    } while (0)
    if (hd == 64) LAUNCH_PREFILL(64);
    else if (hd == 128) LAUNCH_PREFILL(128);
    else return (int)cudaErrorInvalidValue;
#undef LAUNCH_PREFILL
    return 0;
}

// ------------------------------------------------------------------ no-allocation entry point
// See attention_tc_noalloc.h for who needs this and the rules that come with it.
#include "attention_tc_noalloc.h"

constexpr long long kNoAllocFloats = 1LL << 20;                // 4 MiB per device
static __device__ __align__(256) float lsb_noalloc_scratch[kNoAllocFloats];

// In host code `lsb_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel could use: the device address is looked up once per device and kept here.
constexpr int kNoAllocMaxDevices = 64;
constexpr int kNoAllocCluster = 8;
static float* g_noalloc_dev_ptr[kNoAllocMaxDevices] = {};

LSB_API long long lsb_decode_attention_noalloc_max_floats(void) { return kNoAllocFloats; }

LSB_API const char* lsb_decode_attention_noalloc_error(int code) {
    if (code == LSB_NOALLOC_TOO_LARGE)
        return "decode attention (no-alloc): n_requests * nh * splits * (hd + 2) exceeds the "
               "built-in scratch array; use at most 8 splits (they need none) or the regular entry point";
    if (code == LSB_NOALLOC_BAD_DEVICE)
        return "decode attention (no-alloc): current device index is outside the library's table";
    return cudaGetErrorString((cudaError_t)code);
}

LSB_API int lsb_decode_attention_noalloc(const void* qkv, int qkv_stride, const void* k_pages,
                                         const void* v_pages, const int* q_start, const int* kv_len,
                                         const int* table_rows, const int* block_table,
                                         int table_stride, void* out, int n_requests, int nh, int nkv,
                                         int hd, int page_size, int num_pages, float scale, int window,
                                         int splits, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh / nkv > 16 || splits < 1 || n_requests > 65535 || nkv > 65535 ||
        (hd != 64 && hd != 128))
        return (int)cudaErrorInvalidValue;
    // Up to kNoAllocCluster splits (the portable cluster size) merge through distributed shared
    // memory and touch no scratch; only more splits than that go through the array.
    float* scratch = nullptr;
    if (splits > kNoAllocCluster) {
        if (lsb_decode_scratch_floats(n_requests, nh, hd, splits) > kNoAllocFloats)
            return LSB_NOALLOC_TOO_LARGE;
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= kNoAllocMaxDevices) return LSB_NOALLOC_BAD_DEVICE;
        if (!g_noalloc_dev_ptr[dev]) {                          // first call on this device
            float* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, lsb_noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            g_noalloc_dev_ptr[dev] = p;
        }
        scratch = g_noalloc_dev_ptr[dev];
    }
    return decode_launch(qkv, qkv_stride, const_cast<void*>(k_pages), const_cast<void*>(v_pages), q_start,
                         kv_len, table_rows, block_table, table_stride, out, scratch, n_requests, nh, nkv,
                         hd, page_size, num_pages, scale, window, splits, nullptr, 0, 0, kNoAllocCluster,
                         stream);
}
