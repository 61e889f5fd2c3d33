// Warming: a kernel of a decode step asks L2 for some of the weights of the streaming product that
// follows it (gemm_stream.cu).  Between two kernels of a step HBM has nothing to do for two or three
// microseconds (the first one's last sums and stores, the hand-over, the second one's set-up); with
// this it is already fetching bytes the second one will ask for.  Which of its bytes matters
// little, how they are asked for a lot: a few large plain prefetches of consecutive bytes from the
// start of what the next product's block of the same index will read (gate/up and down of a 1B
// layer at 8 rows, in a chain: 19.5 us a pair without, 18.3 us with 96 - 128 KB a block, 19.0 us with
// 256 KB, which delay the kernel's own last copies; the same bytes as tensor-map prefetches in
// the next product's own boxes: 20.3 us; row by row in 1.5 KB pieces: 28 us, the copy unit takes a
// request at a time).  A prefetch changes no result and may be dropped by the hardware.
#pragma once
#include <stdint.h>

struct StreamWarm {
    const unsigned char* base;  // the next product's weights [rows, row_bytes]; null: nothing to warm
    long long row_bytes;
    int blocks;                 // its blocks
    int rows_hi, rows_lo, n_hi; // its first n_hi blocks have rows_hi rows, the others rows_lo
    int bytes;                  // what a block asks for, from the start of its rows
};

constexpr int kWarmPiece = 16 * 1024;           // bytes per prefetch

// One thread of block `b` asks for the first bytes that block `b` of the next product will read.
__device__ __forceinline__ void stream_warm_issue(const StreamWarm& w, int b) {
    if (w.base == nullptr || b >= w.blocks) return;
    const bool longer = b < w.n_hi;
    const long long r0 = longer ? (long long)b * w.rows_hi
                                : (long long)w.n_hi * w.rows_hi + (long long)(b - w.n_hi) * w.rows_lo;
    const long long total = (long long)(longer ? w.rows_hi : w.rows_lo) * w.row_bytes;
    const long long want = total < w.bytes ? total : (long long)w.bytes;      // (a multiple of 16)
    const unsigned char* p = w.base + r0 * w.row_bytes;
    for (long long o = 0; o < want; o += kWarmPiece) {
        const uint32_t n = (uint32_t)(want - o < kWarmPiece ? want - o : kWarmPiece);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + o), "r"(n) : "memory");
    }
}
