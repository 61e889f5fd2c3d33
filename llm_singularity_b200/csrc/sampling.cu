// Next-token sampling on the device, one thread block per row of logits.
//
// Order of operations is the reference sampler's (core/src/sampling.cpp:11-118):
//   repetition penalty on previously generated tokens (positive logit / penalty, else
//   * penalty, once per occurrence) -> temperature == 0: first maximum -> logits / T ->
//   top-k (others dropped) -> top-p (smallest set of most probable tokens whose mass
//   exceeds p) -> softmax over what is left -> the first index whose cumulative
//   probability reaches the uniform draw u.
// The reference sorts on the host; here the k-th largest value and the top-p cut are found
// by bisection on the order-preserving integer image of the floats (32 passes over the
// row at most), so nothing is sorted and nothing leaves the device.  Ties at the k-th
// value are all kept.  The uniform draw comes from the caller (a counter-based generator
// keyed by the request's seed and its count of generated tokens), which makes a request's
// tokens independent of what else is in the batch.  All arithmetic is 32-bit.
//
// `work` is scratch of the same shape as the logits, used only by rows that apply a
// repetition penalty.
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned int ordered(float f) {
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct BlockScratch {
    float f[33];
    int i[33];
};

__device__ __forceinline__ float block_sum_f(float v, BlockScratch& s) { return lsb_block_sum(v, s.f); }

__device__ __forceinline__ int block_sum_i(int v, BlockScratch& s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) s.i[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = lane < nwarps ? s.i[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) s.i[32] = t;
    }
    __syncthreads();
    return s.i[32];
}

// (value, index) maximum with the lowest index winning ties
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__device__ __forceinline__ void block_argmax(float& v, int& idx, BlockScratch& s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_merge(v, idx, ov, oi);
    }
    __syncthreads();
    if (lane == 0) { s.f[warp] = v; s.i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        float tv = lane < nwarps ? s.f[lane] : -FLT_MAX;
        int ti = lane < nwarps ? s.i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, tv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, ti, o);
            argmax_merge(tv, ti, ov, oi);
        }
        if (lane == 0) { s.f[32] = tv; s.i[32] = ti; }
    }
    __syncthreads();
    v = s.f[32];
    idx = s.i[32];
}

// A greedy row without a repetition penalty is scanned by kGreedyParts blocks (blockIdx.y), each its
// slice; the partial maxima meet in device memory and the block that arrives last picks the first
// maximum among them (the order of arrival does not matter: ties go to the lowest index).  One block
// reading a row of 128,256 logits took 12 - 14 us, as long as a layer of the decode step.  Every other
// row is the work of its first block alone.
constexpr int kGreedyParts = 16;
constexpr int kGreedyRows = 1024;                 // rows beyond this are scanned by one block each
__device__ float greedy_part_v[kGreedyRows * kGreedyParts];
__device__ int greedy_part_i[kGreedyRows * kGreedyParts];
__device__ unsigned int greedy_arrived[kGreedyRows];

// params per row: {temperature, top_p, repetition_penalty, u}
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, float* __restrict__ work, int vocab,
              const float* __restrict__ params, const int* __restrict__ top_ks,
              const int* __restrict__ prev_start, const int* __restrict__ prev_tokens,
              int* __restrict__ out) {
    __shared__ BlockScratch sc;
    __shared__ float chunk_sum[kSampleThreads];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float temperature = params[row * 4 + 0], top_p = params[row * 4 + 1];
    const float penalty = params[row * 4 + 2], u = params[row * 4 + 3];
    const int top_k = top_ks[row];
    const float* src = logits + (size_t)row * vocab;

    const int pb = prev_start ? prev_start[row] : 0, pe = prev_start ? prev_start[row + 1] : 0;
    const int parts = (int)gridDim.y;
    const bool shared_scan = parts > 1 && temperature == 0.0f && !(penalty != 1.0f && pe > pb);
    if (blockIdx.y > 0 && !shared_scan) return;
    if (penalty != 1.0f && pe > pb) {
        float* w = work + (size_t)row * vocab;
        for (int i = tid; i < vocab; i += kSampleThreads) w[i] = src[i];
        __syncthreads();
        if (tid == 0) {
            for (int j = pb; j < pe; ++j) {
                const int t = prev_tokens[j];
                if (t >= 0 && t < vocab) w[t] = w[t] > 0.f ? w[t] / penalty : w[t] * penalty;
            }
        }
        __syncthreads();
        src = w;
    }

    if (temperature == 0.0f) {
        float bv = -FLT_MAX;
        int bi = 0x7fffffff;
        // (one block reads the whole row: four 16-byte loads in flight per thread; with one 4-byte
        // load at a time a row of 128,256 took 14 us, the length of a layer of the decode step)
        if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            const float4* s4 = reinterpret_cast<const float4*>(src);
            int n4 = vocab >> 2, first4 = 0;
            if (shared_scan) {                      // this block's slice of the row
                const int per = (n4 + parts - 1) / parts;
                first4 = min(n4, (int)blockIdx.y * per);
                n4 = min(n4, first4 + per);
            }
            for (int i0 = first4 + tid; i0 < n4; i0 += 4 * kSampleThreads) {
                float4 v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int i = i0 + q * kSampleThreads;
                    v[q] = i < n4 ? s4[i] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int i = 4 * (i0 + q * kSampleThreads);
                    if (i < 4 * n4) {
                        argmax_merge(bv, bi, v[q].x, i);
                        argmax_merge(bv, bi, v[q].y, i + 1);
                        argmax_merge(bv, bi, v[q].z, i + 2);
                        argmax_merge(bv, bi, v[q].w, i + 3);
                    }
                }
            }
        } else {
            int b = 0, e = vocab;
            if (shared_scan) {
                const int per = (vocab + parts - 1) / parts;
                b = min(vocab, (int)blockIdx.y * per);
                e = min(vocab, b + per);
            }
            for (int i = b + tid; i < e; i += kSampleThreads) argmax_merge(bv, bi, src[i], i);
        }
        block_argmax(bv, bi, sc);
        if (!shared_scan) {
            if (tid == 0) out[row] = bi;
            return;
        }
        __shared__ bool last;
        if (tid == 0) {
            greedy_part_v[row * kGreedyParts + blockIdx.y] = bv;
            greedy_part_i[row * kGreedyParts + blockIdx.y] = bi;
            __threadfence();
            last = atomicAdd(&greedy_arrived[row], 1u) == (unsigned int)parts - 1u;
        }
        __syncthreads();
        if (!last) return;
        if (tid < 32) {
            __threadfence();
            float v = -FLT_MAX;
            int idx = 0x7fffffff;
            if (tid < parts) {
                v = __ldcg(&greedy_part_v[row * kGreedyParts + tid]);
                idx = __ldcg(&greedy_part_i[row * kGreedyParts + tid]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                argmax_merge(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
            if (tid == 0) {
                out[row] = idx;
                greedy_arrived[row] = 0u;           // for the next launch
            }
        }
        return;
    }
    // x_i = src[i] / temperature, recomputed in every pass (division as the reference does)
#define X(i) (src[i] / temperature)

    float mx = -FLT_MAX;
    int mi = 0x7fffffff;
    for (int i = tid; i < vocab; i += kSampleThreads) argmax_merge(mx, mi, X(i), i);
    block_argmax(mx, mi, sc);

    unsigned int thr = 0u;                       // keep x with ordered(x) >= thr
    if (top_k > 0 && top_k < vocab) {
        unsigned int lo = 0u, hi = 0xffffffffu;  // count(>= lo) >= k always holds
        while (lo < hi) {
            const unsigned int mid = lo + (hi - lo) / 2u + ((hi - lo) & 1u);
            int c = 0;
            for (int i = tid; i < vocab; i += kSampleThreads) c += ordered(X(i)) >= mid;
            c = block_sum_i(c, sc);
            if (c >= top_k) lo = mid; else hi = mid - 1u;
        }
        thr = lo;
    }
    if (top_p < 1.0f) {
        float tot = 0.f;
        for (int i = tid; i < vocab; i += kSampleThreads) {
            const float x = X(i);
            if (ordered(x) >= thr) tot += expf(x - mx);
        }
        tot = block_sum_f(tot, sc);
        // smallest v with mass(x > v) <= top_p * tot; everything >= v is kept
        unsigned int lo = thr, hi = ordered(mx);
        while (lo < hi) {
            const unsigned int mid = lo + (hi - lo) / 2u;
            float mass = 0.f;
            for (int i = tid; i < vocab; i += kSampleThreads) {
                const float x = X(i);
                if (ordered(x) > mid) mass += expf(x - mx);
            }
            mass = block_sum_f(mass, sc);
            if (mass <= top_p * tot) hi = mid; else lo = mid + 1u;
        }
        thr = lo;
    }

    // inverse CDF in index order: thread t owns the contiguous chunk [t*per, (t+1)*per)
    const int per = (vocab + kSampleThreads - 1) / kSampleThreads;
    const int b = min(vocab, tid * per), e = min(vocab, b + per);
    float mine = 0.f;
    for (int i = b; i < e; ++i) {
        const float x = X(i);
        if (ordered(x) >= thr) mine += expf(x - mx);
    }
    chunk_sum[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int t = 0; t < kSampleThreads; ++t) total += chunk_sum[t];
        const float target = u * total;
        // the first chunk at which the running sum reaches the target; chunks without a kept token
        // are passed over, so that if rounding leaves the sum short of the target at the very end,
        // the scan below ends on the last kept token (the reference's fallback, sampling.cpp:113-116)
        float run = 0.f, before = 0.f;
        int t = -1, last_full = 0;
        for (int c = 0; c < kSampleThreads; ++c) {
            if (!(chunk_sum[c] > 0.f)) continue;
            last_full = c;
            before = run;
            if (run + chunk_sum[c] >= target) { t = c; break; }
            run += chunk_sum[c];
        }
        if (t < 0) t = last_full;
        run = before;
        const int tb = min(vocab, t * per), te = min(vocab, tb + per);
        int pick = -1, last_kept = -1;
        for (int i = tb; i < te; ++i) {
            const float x = X(i);
            if (ordered(x) >= thr) {
                run += expf(x - mx);
                last_kept = i;
                if (run >= target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last_kept >= 0 ? last_kept : mi;   // rounding at the very end
        out[row] = pick;
    }
#undef X
}

// logits: float [rows, vocab]; work: float [rows, vocab] scratch; params: float [rows, 4]
// = {temperature, top_p, repetition_penalty, u}; top_k: int [rows] (0 = off);
// prev_start: int [rows + 1] offsets into prev_tokens, or null; out: int [rows].
LSB_API int lsb_sample(const float* logits, float* work, int rows, int vocab, const float* params,
                       const int* top_k, const int* prev_start, const int* prev_tokens, int* out,
                       cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return (int)cudaErrorInvalidValue;
    // (few rows: their greedy scans are shared out over more blocks; many rows fill the SMs by themselves)
    const int parts = rows <= 64 && vocab >= 16384 ? kGreedyParts : 1;
    static_assert(kGreedyParts <= 32, "the last block merges the parts with one warp");
    return lsb_launch(sample_kernel, dim3(rows, parts), dim3(kSampleThreads), 0, stream, 1, logits, work, vocab,
                      params, top_k, prev_start, prev_tokens, out);
}
