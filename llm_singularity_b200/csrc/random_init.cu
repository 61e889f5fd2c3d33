// Random weights on the device: out[i] = mean + scale * normal(key, i), a counter-based stream.
//
// The reference has no random-weights mode (app/main.cpp:149-160 needs a checkpoint).  The value
// of element i of a tensor depends on (key, i) alone, key being derived on the host from the seed
// and the tensor's name, so a tensor can be made in any order, in pieces, here or on the CPU
// (weights/random_init.py states the same arithmetic with tensor operations) with the same bits.
//
// normal(key, i): z = splitmix64(key + (i + 1) * golden); a = top 24 bits, b = next 24 bits;
// u = (a + 1) / 2^24 in (0, 1]; Box-Muller: sqrt(-2 ln u) * cos(2 pi b / 2^24).  Both functions
// are evaluated by short polynomials in 32-bit with every product and sum rounded on its own
// (__fmul_rn / __fadd_rn: no fused multiply-add, which the CPU statement does not use either),
// division and square root correctly rounded, so that the two statements agree bit for bit.
#include "common.cuh"

LSB_DEFINE_STATUS()

__device__ __forceinline__ unsigned long long rnd_splitmix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float rnd_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float rnd_add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ float rnd_normal(unsigned long long key, unsigned long long i) {
    const unsigned long long z = rnd_splitmix64(key + (i + 1ull) * 0x9E3779B97F4A7C15ull);
    const unsigned a = (unsigned)(z >> 40);                 // 24 bits
    const unsigned b = (unsigned)(z >> 16) & 0xFFFFFFu;     // 24 bits
    // ln u, u = t / 2^24, t = a + 1 in [1, 2^24]: t = m * 2^e, m in (sqrt(1/2), sqrt(2)]
    const unsigned t = a + 1u;
    int e = 31 - __clz(t);
    float m = rnd_mul(__uint2float_rn(t), __int_as_float((127 - e) << 23));     // exact: m in [1, 2)
    if (m > 1.41421356f) { m = rnd_mul(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(rnd_add(m, -1.0f), rnd_add(m, 1.0f));     // ln m = 2 atanh(s)
    const float s2 = rnd_mul(s, s);
    float p = 1.0f / 9.0f;
    p = rnd_add(rnd_mul(p, s2), 1.0f / 7.0f);
    p = rnd_add(rnd_mul(p, s2), 1.0f / 5.0f);
    p = rnd_add(rnd_mul(p, s2), 1.0f / 3.0f);
    p = rnd_add(rnd_mul(p, s2), 1.0f);
    const float lnm = rnd_mul(rnd_mul(2.0f, s), p);
    const float lnu = rnd_add(rnd_mul(__int2float_rn(e - 24), 0.69314718f), lnm);
    const float r = __fsqrt_rn(rnd_mul(-2.0f, lnu));
    // cos(2 pi b / 2^24): quadrant q, then the sine of an angle in [0, pi/2]
    const unsigned q = b >> 22, f = b & 0x3FFFFFu;
    const unsigned g = (q & 1u) ? f : (0x400000u - f);
    const float x = rnd_mul(__uint2float_rn(g), 3.7450703e-07f);        // (pi / 2) / 2^22
    const float x2 = rnd_mul(x, x);
    float c = 1.0f / 6227020800.0f;
    c = rnd_add(rnd_mul(c, x2), -1.0f / 39916800.0f);
    c = rnd_add(rnd_mul(c, x2), 1.0f / 362880.0f);
    c = rnd_add(rnd_mul(c, x2), -1.0f / 5040.0f);
    c = rnd_add(rnd_mul(c, x2), 1.0f / 120.0f);
    c = rnd_add(rnd_mul(c, x2), -1.0f / 6.0f);
    c = rnd_add(rnd_mul(c, x2), 1.0f);
    float v = rnd_mul(x, c);
    if (q == 1u || q == 2u) v = -v;
    return rnd_mul(r, v);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, unsigned long long key,
                                     float mean, float scale) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = lsb_from_float<T>(rnd_add(mean, rnd_mul(scale, rnd_normal(key, (unsigned long long)i))));
}

LSB_API int lsb_random_normal(void* out, int dtype, long long n, unsigned long long key, float mean,
                              float scale, cudaStream_t stream) {
    if (n <= 0) return 0;
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return (int)err;
    long long blocks = (n + 255) / 256;
    if (blocks > (long long)sms * 32) blocks = (long long)sms * 32;
    LSB_DISPATCH_DTYPE(dtype, random_normal_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(
                                  (T*)out, n, key, mean, scale));
    return LSB_LAUNCH_CHECK();
}
