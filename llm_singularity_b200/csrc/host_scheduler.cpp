// The scheduler on the host: admits requests, cuts prompts into portions under a token budget,
// decodes, finishes and frees.  Host code only, one object per engine, over the memory layer
// (host_memory.cpp) of the same library.
//
// One call of lsbs_plan plans one step:
//   1. every running request whose prompt is done gets its one decode token;
//   2. running requests still in their prompt get the next portion (at most the portion cap and
//      what is left of the budget);
//   3. waiting requests are admitted first come, first served, as long as a slot is free and the
//      pools can hold the whole prompt plus one token (pages the prefix tree could give up count
//      as free), and get a first portion.
// Pages are reserved here for exactly the tokens the step brings.  When a reservation fails the
// prefix tree is asked to evict; if that is not enough, a decoding request preempts the most
// recently admitted running request (freed, back to the front of the queue, recomputed later from
// everything it has produced so far), while a prompt waits.  A request that can never fit ends
// with an error.  Nothing is random.
//
// Accounting has two halves.  Planning a step advances its requests at once (its tokens count as
// computed; a request whose logits are sampled gets a place-holder at the end of its tokens);
// lsbs_update fills the place-holders in when the sampled tokens have come back, and finishes
// requests.  Between the two the next step can be planned "ahead": a request with a place-holder
// decodes on, its input token being fed on the device.
//
// What happened is reported as a list of events (admitted, preempted, failed, item, token,
// finished) that the Python face replays onto its request records; this file is the authority.
//
// The reference schedules prompts before decode tokens, iterates an unordered map, allocates whole
// prompts at admission, samples after every portion and carries on into page 0 when pages run out
// (core/src/scheduler.cpp:67-272); its stop rules (eos, stop ids, max_new_tokens, the output
// includes the stop token; scheduler.cpp:238-266) are kept.
#include <algorithm>
#include <cstdint>
#include <deque>
#include <string>
#include <vector>

#include "host_memory.h"

#define LSB_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kErr = kLsbHostErr;
constexpr int32_t kPending = -1;     // stands for a token that a step in flight has yet to produce

enum Status { kWaiting = 0, kRunning = 1, kFinished = 2, kFailed = 3 };
enum Event { kAdmit = 1, kPreempt = 2, kFail = 3, kItem = 4, kToken = 5, kFinish = 6 };
enum Stat { kSteps, kPreemptions, kPrefillTokens, kDecodeTokens, kPrefixHitTokens, kEvictedPages, kAdmitted,
            kErrors, kAheadSteps, kNumStats };

struct Req {
    bool used = false;
    long long serial = 0;            // which request this handle stands for (handles are used again)
    std::vector<int32_t> tokens;     // prompt + generated so far (+ place-holders)
    int generated = 0;
    int max_new_tokens = 0;
    bool ignore_eos = false;
    bool penalty = false;            // samples with a repetition penalty: needs every token on the host
    long long computed = 0;          // tokens whose keys and values are cached once the planned steps have run
    int pending = 0;                 // place-holders at the end of tokens
    int status = kWaiting;
    int slot = -1;
    std::vector<int> path;           // prefix-tree nodes it counts as a user of
    std::string error;
};

struct Item {
    int req;
    long long serial;
    long long start;                 // position of the portion's first token
    int n;
    bool sample;                     // the portion ends the known tokens: logits of its last token wanted
    bool decode;                     // one token after a sampled one
};

struct Scheduler {
    void* mem = nullptr;
    bool prefix = false;
    int max_batch_size = 64, max_tokens_per_batch = 512, max_prefill_chunk = 0;
    long long max_model_len = 1LL << 30;
    std::vector<int32_t> stop_ids;
    std::vector<Req> reqs;
    std::vector<int> free_handles;
    std::deque<int> waiting;
    std::vector<int> running;        // admission order
    std::deque<std::vector<Item>> plans;   // steps whose results have not come back, oldest first
    std::vector<long long> events;   // records of 5: kind, request, a, b, c
    long long stats[kNumStats] = {0};
    long long next_serial = 1;
    std::string error;
    std::vector<int> scratch_nodes;

    int fail(const std::string& msg) {
        error = msg;
        return kErr;
    }
    int mem_fail() { return fail(lsbm_last_error(mem)); }
    void emit(int kind, int req, long long a = 0, long long b = 0, long long c = 0) {
        events.insert(events.end(), {(long long)kind, (long long)req, a, b, c});
    }
    long long pages_for(long long n) const {
        const int ps = lsbm_page_size(mem);
        return (n + ps - 1) / ps;
    }
    int free_pages() const { return lsbm_free_pages(mem) + (prefix ? lsbp_evictable(mem) : 0); }
};

Scheduler* S(void* h) { return static_cast<Scheduler*>(h); }

// Pages for new_len tokens of the request, evicting cached prefixes if needed.  1 / 0 / kErr.
int reserve(Scheduler* s, Req& r, long long new_len) {
    int rc = lsbm_reserve(s->mem, r.slot, new_len);
    if (rc == kErr) return s->mem_fail();
    if (rc == 1 || !s->prefix) return rc;
    const long long need = std::max(0LL, s->pages_for(new_len) - lsbm_num_pages(s->mem, r.slot)) - lsbm_free_pages(s->mem);
    if (need > 0) {
        const int freed = lsbp_evict(s->mem, (int)need);
        if (freed == kErr) return s->mem_fail();
        s->stats[kEvictedPages] += freed;
    }
    rc = lsbm_reserve(s->mem, r.slot, new_len);
    return rc == kErr ? s->mem_fail() : rc;
}

// Everything the request holds goes back: its place among the users of its prefix, its pages, its slot.
int release(Scheduler* s, Req& r) {
    if (s->prefix && !r.path.empty()) {
        if (lsbp_release(s->mem, r.path.data(), (int)r.path.size()) == kErr) return s->mem_fail();
        r.path.clear();
    }
    if (lsbm_close(s->mem, r.slot) == kErr) return s->mem_fail();
    r.slot = -1;
    return 0;
}

void drop_running(Scheduler* s, int id) {
    s->running.erase(std::find(s->running.begin(), s->running.end(), id));
}

// Free everything the request holds; it will be recomputed from its tokens so far.
int preempt(Scheduler* s, int id) {
    Req& r = s->reqs[id];
    if (release(s, r) == kErr) return kErr;
    drop_running(s, id);
    r.computed = 0;
    r.status = kWaiting;
    ++s->stats[kPreemptions];
    s->waiting.push_front(id);
    s->emit(kPreempt, id);
    return 0;
}

void fail_request(Scheduler* s, int id, const std::string& why) {
    Req& r = s->reqs[id];
    r.status = kFailed;
    r.error = why;
    ++s->stats[kErrors];
    s->emit(kFail, id);
}

// Why the request can never run (its tokens plus one exceed the model's length or the pool), or "".
std::string never_fits(Scheduler* s, const Req& r) {
    const long long have = (long long)r.tokens.size(), n = have + 1;
    const long long pool = lsbm_smallest_pool(s->mem);
    if (n > s->max_model_len)
        return std::to_string(have) + " tokens plus one exceed max_model_len " + std::to_string(s->max_model_len);
    if (s->pages_for(n) > std::min<long long>(pool, lsbm_max_pages(s->mem)))
        return std::to_string(have) + " tokens plus one need " + std::to_string(s->pages_for(n)) +
               " pages, the pool has " + std::to_string(pool);
    return "";
}

// Largest portion <= n whose pages can be had now (prompts wait rather than preempt).  >= 0 or kErr.
long long fit_portion(Scheduler* s, Req& r, long long n) {
    if (n <= 0) return 0;
    int rc = reserve(s, r, r.computed + n);
    if (rc == kErr) return kErr;
    if (rc == 1) return n;
    const long long ps = lsbm_page_size(s->mem);
    const long long have = s->pages_for(r.computed) * ps;          // tokens its held pages cover
    const long long room = have + (long long)s->free_pages() * ps - r.computed;
    n = std::min(n, room);
    if (n > 0) {
        rc = reserve(s, r, r.computed + n);
        if (rc == kErr) return kErr;
        if (rc == 1) return n;
    }
    return 0;
}

Item portion(const Req& r, int id, long long n) {
    return Item{id, r.serial, r.computed, (int)n, r.computed + n == (long long)r.tokens.size(), false};
}

bool ends_with_token_in_flight(const Scheduler* s, const Req& r) {
    return r.generated + r.pending >= r.max_new_tokens || (long long)r.tokens.size() + 1 > s->max_model_len;
}

}  // namespace

namespace {

// Plans one step (see the head of this file).  Returns the number of items, or kErr.
int plan(Scheduler* s, bool ahead) {
    std::vector<Item> items;
    const long long chunk_cap = s->max_prefill_chunk > 0 ? s->max_prefill_chunk : s->max_tokens_per_batch;

    // 1. decode tokens (requests with exactly one token left to run), oldest first; when pages run
    //    out the youngest running request is preempted (possibly the one asking), or, while a step
    //    is in flight, the request waits
    const std::vector<int> snapshot = s->running;
    for (int id : snapshot) {
        Req& r = s->reqs[id];
        if (r.status != kRunning || (long long)r.tokens.size() - r.computed != 1) continue;
        if (r.pending && ends_with_token_in_flight(s, r)) continue;
        if ((int)items.size() >= s->max_tokens_per_batch) break;
        bool placed = false;
        while (r.status == kRunning) {
            const int rc = reserve(s, r, (long long)r.tokens.size());
            if (rc == kErr) return kErr;
            if (rc == 1) {
                placed = true;
                break;
            }
            if (ahead) break;
            const int victim = s->running.back();
            items.erase(std::remove_if(items.begin(), items.end(), [victim](const Item& it) { return it.req == victim; }),
                        items.end());
            if (preempt(s, victim) == kErr) return kErr;
        }
        if (placed) items.push_back(Item{id, r.serial, r.computed, 1, true, false});
    }
    long long budget = s->max_tokens_per_batch - (long long)items.size();

    // 2. next portions of prompts already running (they wait for pages, never preempt)
    for (int id : s->running) {
        Req& r = s->reqs[id];
        const long long remaining = (long long)r.tokens.size() - r.computed;
        if (remaining <= 1 || budget <= 0) continue;
        const long long n = fit_portion(s, r, std::min({remaining, budget, chunk_cap}));
        if (n == kErr) return kErr;
        if (n > 0) {
            items.push_back(portion(r, id, n));
            budget -= n;
        }
    }

    // 3. admission, first come first served
    while (!s->waiting.empty() && budget > 0 && (int)s->running.size() < s->max_batch_size) {
        const int id = s->waiting.front();
        Req& r = s->reqs[id];
        const std::string why = never_fits(s, r);
        if (!why.empty()) {
            s->waiting.pop_front();
            fail_request(s, id, why);
            continue;
        }
        int n_path = 0;
        if (s->prefix) {
            s->scratch_nodes.resize(lsbm_max_pages(s->mem));
            n_path = lsbp_match(s->mem, r.tokens.data(), (long long)r.tokens.size(), s->scratch_nodes.data(),
                                (int)s->scratch_nodes.size());
            if (n_path == kErr) return s->mem_fail();
        }
        const long long need = s->pages_for((long long)r.tokens.size() + 1) - n_path;
        // pages on the matched path are in use by this request, not evictable for it
        int idle_on_path = 0;
        if (n_path > 0) {
            idle_on_path = lsbp_idle_on(s->mem, s->scratch_nodes.data(), n_path);
            if (idle_on_path == kErr) return s->mem_fail();
        }
        if (need > s->free_pages() - idle_on_path) break;
        const int slot = lsbm_open(s->mem);
        if (slot < 0) break;
        s->waiting.pop_front();
        r.slot = slot;
        if (n_path > 0) {
            const long long got = lsbp_adopt(s->mem, slot, s->scratch_nodes.data(), n_path);
            if (got == kErr) return s->mem_fail();
            r.computed = got;
            r.path.assign(s->scratch_nodes.begin(), s->scratch_nodes.begin() + n_path);
            s->stats[kPrefixHitTokens] += got;
        }
        r.status = kRunning;
        s->running.push_back(id);
        ++s->stats[kAdmitted];
        s->emit(kAdmit, id, r.computed);
        const long long n = fit_portion(s, r, std::min({(long long)r.tokens.size() - r.computed, budget, chunk_cap}));
        if (n == kErr) return kErr;
        if (n > 0) {
            items.push_back(portion(r, id, n));
            budget -= n;
        }
    }

    // nothing could move although requests are live: the youngest gives way
    if (items.empty() && !s->running.empty() && !ahead) {
        if (s->running.size() == 1) {
            const int id = s->running[0];
            if (release(s, s->reqs[id]) == kErr) return kErr;
            drop_running(s, id);
            fail_request(s, id, "the cache pool cannot hold this request");
        } else if (preempt(s, s->running.back()) == kErr) {
            return kErr;
        }
        return plan(s, ahead);
    }

    // the first half of the accounting: the step counts as run
    for (Item& it : items) {
        Req& r = s->reqs[it.req];
        r.computed += it.n;
        it.decode = it.n == 1 && it.start > 0 && (r.generated > 0 || r.pending > 0);
        if (it.sample) {
            if (s->prefix && !it.decode) {
                // The prompt is whole with this step: later prompts may share its full pages from
                // now on (a step that reads them is queued behind this one).
                s->scratch_nodes.resize(lsbm_max_pages(s->mem));
                const int added = lsbp_share(s->mem, r.tokens.data(), r.computed, r.slot, r.path.data(),
                                             (int)r.path.size(), s->scratch_nodes.data(), (int)s->scratch_nodes.size());
                if (added == kErr) return s->mem_fail();
                r.path.insert(r.path.end(), s->scratch_nodes.begin(), s->scratch_nodes.begin() + added);
            }
            r.tokens.push_back(kPending);
            ++r.pending;
        }
        s->emit(kItem, it.req, it.start, it.n, (it.sample ? 1 : 0) | (it.decode ? 2 : 0));
    }
    const int n_items = (int)items.size();
    if (n_items) {
        s->plans.push_back(std::move(items));
        ++s->stats[kSteps];
    }
    return n_items;
}

}  // namespace

// ----------------------------------------------------------------------------- C interface
LSB_API void* lsbs_create(void* memory, int use_prefix, int max_batch_size, int max_tokens_per_batch,
                          int max_prefill_chunk, const int* stop_ids, int n_stop, long long max_model_len) {
    if (!memory || max_batch_size <= 0 || max_tokens_per_batch <= 0) return nullptr;
    Scheduler* s = new Scheduler;
    s->mem = memory;
    s->prefix = use_prefix != 0;
    s->max_batch_size = max_batch_size;
    s->max_tokens_per_batch = max_tokens_per_batch;
    s->max_prefill_chunk = max_prefill_chunk;
    s->stop_ids.assign(stop_ids, stop_ids + n_stop);
    s->max_model_len = max_model_len;
    return s;
}
LSB_API void lsbs_destroy(void* h) { delete S(h); }
// The tokens that end a request, from the next lsbs_update on.
LSB_API void lsbs_set_stop_ids(void* h, const int* stop_ids, int n_stop) {
    S(h)->stop_ids.assign(stop_ids, stop_ids + n_stop);
}
LSB_API const char* lsbs_last_error(void* h) { return S(h)->error.c_str(); }

// A new request joins the queue; returns its handle.
LSB_API int lsbs_add(void* h, const int* tokens, long long n, int max_new_tokens, int ignore_eos, int penalty) {
    Scheduler* s = S(h);
    if (n <= 0) return s->fail("a request needs at least one prompt token");
    if (max_new_tokens < 1) return s->fail("max_new_tokens must be at least 1");
    int id;
    if (!s->free_handles.empty()) {
        id = s->free_handles.back();
        s->free_handles.pop_back();
    } else {
        id = (int)s->reqs.size();
        s->reqs.emplace_back();
    }
    Req& r = s->reqs[id];
    r = Req();
    r.used = true;
    r.serial = s->next_serial++;
    r.tokens.assign(tokens, tokens + n);
    r.max_new_tokens = max_new_tokens;
    r.ignore_eos = ignore_eos != 0;
    r.penalty = penalty != 0;
    s->waiting.push_back(id);
    return id;
}

// The caller has taken note of a finished or failed request: its handle may be used again.
LSB_API int lsbs_forget(void* h, int id) {
    Scheduler* s = S(h);
    if (id < 0 || id >= (int)s->reqs.size() || !s->reqs[id].used) return s->fail("no request " + std::to_string(id));
    if (s->reqs[id].status != kFinished && s->reqs[id].status != kFailed)
        return s->fail("request " + std::to_string(id) + " is still live");
    s->reqs[id] = Req();
    s->free_handles.push_back(id);
    return 0;
}

LSB_API int lsbs_has_work(void* h) { return !S(h)->waiting.empty() || !S(h)->running.empty(); }
LSB_API int lsbs_plans_in_flight(void* h) { return (int)S(h)->plans.size(); }

// Plan the next step.  ahead = 0: the step before it has been accounted (lsbs_update).  ahead = 1:
// the step after the one in flight, before that one's tokens are known; returns 0 when there is
// nothing to run, when two steps would be ahead, or when a request samples with a repetition
// penalty.  Returns the number of items; what happened is in the events.
LSB_API int lsbs_plan(void* h, int ahead) {
    Scheduler* s = S(h);
    s->events.clear();
    if (!ahead) {
        if (!s->plans.empty()) return s->fail("a step is in flight: account it first, or plan ahead");
        return plan(s, false);
    }
    if (s->plans.size() != 1) return 0;
    for (int id : s->running)
        if (s->reqs[id].pending && s->reqs[id].penalty) return 0;
    const int n = plan(s, true);
    if (n > 0) ++s->stats[kAheadSteps];
    return n;
}

// The oldest step still unaccounted has run: requests[i] sampled tokens[i].  Fills the
// place-holders in and finishes requests; what happened is in the events.
LSB_API int lsbs_update(void* h, const int* requests, const int* tokens, int n) {
    Scheduler* s = S(h);
    s->events.clear();
    if (s->plans.empty()) return 0;
    std::vector<Item> items = std::move(s->plans.front());
    s->plans.pop_front();
    std::vector<std::pair<int, long long>> done;
    for (const Item& it : items) {
        Req& r = s->reqs[it.req];
        // planned ahead, but it stopped on the token that was in flight (its handle may be another's by now)
        if (!r.used || r.serial != it.serial || r.status != kRunning) continue;
        const long long end = it.start + it.n;              // tokens cached now that this step has run
        if (lsbm_length(s->mem, r.slot) < end && lsbm_commit(s->mem, r.slot, end) == kErr) return s->mem_fail();
        if (!it.sample) {
            s->stats[kPrefillTokens] += it.n;
            continue;
        }
        if (it.decode) ++s->stats[kDecodeTokens];
        else s->stats[kPrefillTokens] += it.n;
        const int* at = std::find(requests, requests + n, it.req);
        if (at == requests + n) return s->fail("request " + std::to_string(it.req) + ": no token came back for it");
        const int tok = tokens[at - requests];
        if (end >= (long long)r.tokens.size() || r.tokens[end] != kPending)
            return s->fail("request " + std::to_string(it.req) + ": no token is outstanding at place " + std::to_string(end));
        r.tokens[end] = tok;
        --r.pending;
        ++r.generated;
        s->emit(kToken, it.req, tok, end);
        const bool stop_token = !r.ignore_eos && std::find(s->stop_ids.begin(), s->stop_ids.end(), tok) != s->stop_ids.end();
        if (stop_token || r.generated >= r.max_new_tokens || end + 2 > s->max_model_len) done.emplace_back(it.req, end);
    }
    for (auto& [id, end] : done) {
        Req& r = s->reqs[id];
        r.tokens.resize(end + 1);                           // drops a place-holder of a step planned ahead
        r.pending = 0;
        r.computed = end;
        if (s->prefix && lsbp_insert(s->mem, r.tokens.data(), end, r.slot) == kErr) return s->mem_fail();
        if (release(s, r) == kErr) return kErr;
        drop_running(s, id);
        r.status = kFinished;
        s->emit(kFinish, id, end);
    }
    return (int)done.size();
}

// Events of the last lsbs_plan or lsbs_update: records of five (kind, request, a, b, c).
//   admit: a = tokens covered by shared pages; preempt; fail; item: a = start, b = tokens, c = 1 if
//   sampled + 2 if a decode token; token: a = token, b = its place; finish: a = tokens cached.
LSB_API int lsbs_num_events(void* h) { return (int)(S(h)->events.size() / 5); }
LSB_API int lsbs_events(void* h, long long* out, int cap_records) {
    Scheduler* s = S(h);
    const int n = (int)(s->events.size() / 5);
    if (cap_records < n) return s->fail("events: buffer too small");
    std::copy(s->events.begin(), s->events.end(), out);
    return n;
}

LSB_API const char* lsbs_request_error(void* h, int id) { return S(h)->reqs[id].error.c_str(); }
LSB_API int lsbs_request_slot(void* h, int id) { return S(h)->reqs[id].slot; }
// out: status, computed, pending, generated, tokens held, nodes of the prefix tree it uses
LSB_API int lsbs_request_state(void* h, int id, long long* out) {
    Scheduler* s = S(h);
    if (id < 0 || id >= (int)s->reqs.size() || !s->reqs[id].used) return s->fail("no request " + std::to_string(id));
    const Req& r = s->reqs[id];
    out[0] = r.status; out[1] = r.computed; out[2] = r.pending; out[3] = r.generated;
    out[4] = (long long)r.tokens.size(); out[5] = (long long)r.path.size();
    return 0;
}
LSB_API int lsbs_request_tokens(void* h, int id, int* out, long long cap) {
    const Req& r = S(h)->reqs[id];
    if (cap < (long long)r.tokens.size()) return S(h)->fail("tokens: buffer too small");
    std::copy(r.tokens.begin(), r.tokens.end(), out);
    return (int)r.tokens.size();
}
// steps, preemptions, prefill_tokens, decode_tokens, prefix_hit_tokens, evicted_pages, admitted,
// errors, ahead_steps
LSB_API int lsbs_stats(void* h, long long* out) {
    std::copy(S(h)->stats, S(h)->stats + kNumStats, out);
    return kNumStats;
}
