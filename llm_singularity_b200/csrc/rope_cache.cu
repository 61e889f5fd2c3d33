// Rotary position encoding fused with the write of keys and values into cache pages.
//
// Input: the fused projection qkv [tokens, (nh + 2*nkv) * hd] (queries, then keys,
// then values).  For every token at absolute position pos:
//   * each query head and each key head has its first `rotary_dim` dims rotated in
//     split-half pairs (i, i + rotary_dim/2) by the angle pos * inv_freq[i], formed in
//     32-bit; queries are rewritten in place;
//   * the rotated key and the value go to page = table[row][pos / page], offset
//     pos % page of the layer's pools, laid out [page][kv head][offset][hd].
// Replaces rope_kernel + kv_cache_scatter_kernel of the reference
// (kernels/src/rope.cu:13-58, kernels/src/kv_cache.cu:14-45), which recompute powf per
// element and take a per-token page list uploaded each call.  The rotated key is also
// written back into qkv so that a caller who does not store still sees it.
#include "common.cuh"

LSB_DEFINE_STATUS()

template <typename T>
__global__ void rope_kv_store_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_req,
    const int* __restrict__ table_rows, const int* __restrict__ block_table, int table_stride,
    const float* __restrict__ inv_freq, int rotary_dim,
    T* __restrict__ k_pages, T* __restrict__ v_pages,
    int nh, int nkv, int hd, int page_size, int num_pages, int store,
    const int* __restrict__ skip_q_start) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int t = blockIdx.x;
    if (skip_q_start) {           // single decode tokens are rotated and stored by their attention kernel
        const int r = token_req[t];
        if (skip_q_start[r + 1] - skip_q_start[r] == 1) return;
    }
    const int pos = positions[t];
    const int half_hd = hd >> 1;
    const int half_rot = rotary_dim >> 1;
    T* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;

    long long page_base = -1;     // element offset of (page, head 0, offset, 0)
    if (store) {
        const int r = token_req[t];
        const int page_idx = pos / page_size;
        int page = -1;
        if (page_idx < table_stride) page = block_table[(size_t)table_rows[r] * table_stride + page_idx];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_PAGE);
        } else {
            page_base = ((long long)page * nkv * page_size + (pos % page_size)) * hd;
        }
    }

    // work items: (head in [0, nh + nkv), pair index in [0, hd/2))
    const int n_rot = (nh + nkv) * half_hd;
    for (int w = threadIdx.x; w < n_rot; w += blockDim.x) {
        const int head = w / half_hd;
        const int i = w - head * half_hd;
        T* x = row + (size_t)head * hd;
        float a, b;
        int ia, ib;
        if (i < half_rot) {
            ia = i; ib = i + half_rot;
            const float x0 = lsb_to_float(x[ia]), x1 = lsb_to_float(x[ib]);
            float s, c;
            sincosf((float)pos * inv_freq[i], &s, &c);
            a = x0 * c - x1 * s;
            b = x0 * s + x1 * c;
            x[ia] = lsb_from_float<T>(a);
            x[ib] = lsb_from_float<T>(b);
        } else {
            // dims past the rotary part: two unrotated elements per work item
            ia = rotary_dim + 2 * (i - half_rot); ib = ia + 1;
            a = lsb_to_float(x[ia]);
            b = lsb_to_float(x[ib]);
        }
        if (head >= nh && page_base >= 0) {
            T* dst = k_pages + page_base + (long long)(head - nh) * page_size * hd;
            dst[ia] = lsb_from_float<T>(a);
            dst[ib] = lsb_from_float<T>(b);
        }
    }
    if (page_base >= 0) {
        const T* v = row + (size_t)(nh + nkv) * hd;
        for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
            const int head = w / hd, d = w - head * hd;
            v_pages[page_base + (long long)head * page_size * hd + d] = v[w];
        }
    }
}

// Vector form: 16-byte loads and stores, and the sines and cosines of a token computed once per
// block and shared by all its heads (the scalar kernel above evaluates sincosf once per head and
// pair).  Needs head_dim and rotary_dim / 2 to be multiples of the vector width.
template <typename T>
__global__ void rope_kv_store_vec_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_req,
    const int* __restrict__ table_rows, const int* __restrict__ block_table, int table_stride,
    const float* __restrict__ inv_freq, int rotary_dim,
    T* __restrict__ k_pages, T* __restrict__ v_pages,
    int nh, int nkv, int hd, int page_size, int num_pages, int store,
    const int* __restrict__ skip_q_start) {
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float cs[2][128];
    lsb_pdl_launch_dependents();
    // positions and the request index of each token are metadata of the step (on the device before
    // its first kernel starts): the sines and cosines are formed while the projection is computed
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half_rot = rotary_dim >> 1;
    bool skip = false;
    if (skip_q_start) {
        const int r = token_req[t];
        skip = skip_q_start[r + 1] - skip_q_start[r] == 1;
    }
    if (!skip)
        for (int i = threadIdx.x; i < half_rot; i += blockDim.x) sincosf((float)pos * inv_freq[i], &cs[1][i], &cs[0][i]);
    lsb_pdl_wait();
    if (skip) return;
    T* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;

    long long page_base = -1;
    if (store) {
        const int r = token_req[t];
        const int page_idx = pos / page_size;
        int page = -1;
        if (page_idx < table_stride) page = block_table[(size_t)table_rows[r] * table_stride + page_idx];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_PAGE);
        } else {
            page_base = ((long long)page * nkv * page_size + (pos % page_size)) * hd;
        }
    }
    __syncthreads();

    const int per = half_rot / VEC;
    for (int w = threadIdx.x; w < (nh + nkv) * per; w += blockDim.x) {
        const int head = w / per, v = w - head * per;
        T* x = row + (size_t)head * hd;
        T lo[VEC], hi[VEC];
        *reinterpret_cast<uint4*>(lo) = *reinterpret_cast<const uint4*>(x + v * VEC);
        *reinterpret_cast<uint4*>(hi) = *reinterpret_cast<const uint4*>(x + half_rot + v * VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float c = cs[0][v * VEC + e], sn = cs[1][v * VEC + e];
            const float x0 = lsb_to_float(lo[e]), x1 = lsb_to_float(hi[e]);
            lo[e] = lsb_from_float<T>(x0 * c - x1 * sn);
            hi[e] = lsb_from_float<T>(x0 * sn + x1 * c);
        }
        *reinterpret_cast<uint4*>(x + v * VEC) = *reinterpret_cast<const uint4*>(lo);
        *reinterpret_cast<uint4*>(x + half_rot + v * VEC) = *reinterpret_cast<const uint4*>(hi);
        if (head >= nh && page_base >= 0) {
            T* dst = k_pages + page_base + (long long)(head - nh) * page_size * hd;
            *reinterpret_cast<uint4*>(dst + v * VEC) = *reinterpret_cast<const uint4*>(lo);
            *reinterpret_cast<uint4*>(dst + half_rot + v * VEC) = *reinterpret_cast<const uint4*>(hi);
        }
    }
    if (page_base >= 0) {
        // key dims past the rotary part are stored as they are
        const int tail = hd - rotary_dim;
        for (int w = threadIdx.x; w < nkv * tail; w += blockDim.x) {
            const int head = w / tail, d = rotary_dim + (w - head * tail);
            k_pages[page_base + (long long)head * page_size * hd + d] = row[(size_t)(nh + head) * hd + d];
        }
        const T* vsrc = row + (size_t)(nh + nkv) * hd;
        const int vper = hd / VEC;
        for (int w = threadIdx.x; w < nkv * vper; w += blockDim.x) {
            const int head = w / vper, c = w - head * vper;
            *reinterpret_cast<uint4*>(v_pages + page_base + (long long)head * page_size * hd + c * VEC) =
                *reinterpret_cast<const uint4*>(vsrc + (size_t)head * hd + c * VEC);
        }
    }
}

// inv_freq may be null with rotary_dim == 0 (no rotation, only the cache write).  With
// `skip_q_start` (the step's q_start array) tokens of requests that bring a single token are left
// alone: the decode attention kernel rotates and stores those itself.
LSB_API int lsb_rope_kv_store(void* qkv, int dtype, int tokens, int nh, int nkv, int hd,
                              const int* positions, const int* token_req, const int* table_rows,
                              const int* block_table, int table_stride,
                              const float* inv_freq, int rotary_dim,
                              void* k_pages, void* v_pages, int page_size, int num_pages,
                              int store, const int* skip_q_start, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hd % 2 || rotary_dim % 2 || rotary_dim > hd || (rotary_dim > 0 && !inv_freq))
        return (int)cudaErrorInvalidValue;
    int work = (nh + nkv) * (hd / 2);
    int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
    const int vec = dtype == LSB_F32 ? 4 : 8;
    const bool aligned = ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0;
    if (aligned && hd % vec == 0 && (rotary_dim / 2) % vec == 0 && rotary_dim / 2 <= 128) {
        const int items = (nh + nkv) * (rotary_dim / 2 / vec) + nkv * (hd / vec);
        int th = items >= 256 ? 256 : items >= 128 ? 128 : 64;
        LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
            rope_kv_store_vec_kernel<T>, dim3(tokens), dim3(th), 0, stream, 1,
            (T*)qkv, positions, token_req, table_rows, block_table, table_stride, inv_freq, rotary_dim,
            (T*)k_pages, (T*)v_pages, nh, nkv, hd, page_size, num_pages, store, skip_q_start));
    }
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        rope_kv_store_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 1,
        (T*)qkv, positions, token_req, table_rows, block_table, table_stride, inv_freq, rotary_dim,
        (T*)k_pages, (T*)v_pages, nh, nkv, hd, page_size, num_pages, store, skip_q_start));
    return 0;
}
