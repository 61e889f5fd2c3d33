// Packing a step's metadata on the host: one pass over the entries writes, into one pinned buffer,
// everything the kernels read about the batch, so that one copy brings it to the device.
//
// The reference builds these arrays per request inside its forward pass and copies each on its own
// (models/llama/llama_model.cpp:560-615: positions, the block table row and the lengths of one
// request at a time).  Here a step has many requests with any number of tokens each.
#include <cstdint>

#define LSB_API extern "C" __attribute__((visibility("default")))

// Layout of `out`, in this order: token ids [T], positions [T], the entry of every token [T],
// q_start [R + 1], kv_len [R], block-table rows [R], wanted rows [W].  `offsets` gets the seven
// starts and the end (8 values), `summary` the total T, W, the longest entry and the longest
// sequence.  `tokens` are the entries' tokens one after another; `wants` the wanted places of the
// entries one after another, `want_count[r]` of them for entry r.
// Returns the number of ints written; -1 if `cap` is too small; -(r + 2) if entry r has no tokens
// or wants a place outside its tokens.
LSB_API long long lsbh_pack_step(int R, const int32_t* q_len, const int32_t* starts, const int32_t* rows,
                                 const int32_t* tokens, const int32_t* want_count, const int32_t* wants,
                                 int32_t* out, long long cap, long long* offsets, long long* summary) {
    long long T = 0, W = 0;
    int max_q = 0;
    long long max_kv = 0;
    for (int r = 0; r < R; ++r) {
        if (q_len[r] <= 0) return -(long long)(r + 2);
        T += q_len[r];
        W += want_count[r];
        if (q_len[r] > max_q) max_q = q_len[r];
        const long long kv = (long long)starts[r] + q_len[r];
        if (kv > max_kv) max_kv = kv;
    }
    const long long n = 3 * T + (R + 1) + 2 * (long long)R + W;
    if (n > cap) return -1;
    int32_t* tok = out;
    int32_t* pos = tok + T;
    int32_t* req = pos + T;
    int32_t* q_start = req + T;
    int32_t* kv_len = q_start + R + 1;
    int32_t* row = kv_len + R;
    int32_t* want = row + R;
    long long t = 0, w = 0;
    for (int r = 0; r < R; ++r) {
        q_start[r] = (int32_t)t;
        kv_len[r] = starts[r] + q_len[r];
        row[r] = rows[r];
        for (int i = 0; i < q_len[r]; ++i, ++t) {
            tok[t] = tokens[t];
            pos[t] = starts[r] + i;
            req[t] = r;
        }
        for (int i = 0; i < want_count[r]; ++i, ++w) {
            const int32_t place = wants[w];
            if (place < 0 || place >= q_len[r]) return -(long long)(r + 2);
            want[w] = q_start[r] + place;
        }
    }
    q_start[R] = (int32_t)t;
    offsets[0] = 0;
    offsets[1] = T;
    offsets[2] = 2 * T;
    offsets[3] = 3 * T;
    offsets[4] = offsets[3] + R + 1;
    offsets[5] = offsets[4] + R;
    offsets[6] = offsets[5] + R;
    offsets[7] = offsets[6] + W;
    summary[0] = T;
    summary[1] = W;
    summary[2] = max_q;
    summary[3] = max_kv;
    return n;
}
