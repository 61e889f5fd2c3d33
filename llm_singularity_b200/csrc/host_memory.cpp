// The memory layer on the host: page pools, block tables, request slots and the prefix tree.
//
// Host code only (no kernel here); built like the other libraries, one shared object with a plain
// C interface.  One `Memory` object serves one engine:
//   * a pool of page ids per group of layers (all keys, or a window of them), with reference
//     counts: a page is free, or held by live requests and/or by nodes of the prefix tree;
//   * a block table per group, [slots x max_pages] int32, whose device copy is patched cell by
//     cell: every change is also appended to the group's list of updates;
//   * request slots (a slot is a request's row in every block table and in every state tensor);
//   * a radix tree over page-sized chunks of token ids whose nodes own one page per group.
// Requests are addressed by slot; the Python wrapper maps request ids to slots.
//
// The reference keeps a bare stack of block indices, a map from whole prompts to block lists and a
// per-request vector in its scheduler (core/src/memory.cpp:5-117, core/include/core/scheduler.h:59-69);
// a block freed twice goes unnoticed there and cached prompts are never evicted.  Here every
// violation is refused with a message.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "host_memory.h"

#define LSB_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int32_t kNoPage = -1;
constexpr int kErr = kLsbHostErr;    // return value of a call that failed (message in last_error)

struct Pool {
    int num_pages = 0;
    std::vector<int32_t> free_list;  // stack: the page freed last is handed out first
    std::vector<int32_t> refs;
    std::vector<int32_t> tree_refs;  // of refs[p], how many belong to prefix-tree nodes
};

struct Group {
    int window = -1;                 // < 0: the group keeps all keys
    Pool pool;
    std::vector<int32_t> table;      // [slots * max_pages], host mirror of the device table
    std::vector<int32_t> first_live; // per slot: pages [0, first_live) were released behind the window
    std::vector<int32_t> updates;    // (flat index, value) pairs not yet taken
    std::vector<uint32_t> taken;     // per cell: the call of take_updates_last that last gave it out
    uint32_t take_call = 0;
};

struct Request {
    bool open = false;
    long long length = 0;
    int num_pages = 0;               // logical pages covered so far (same count in every group)
};

struct Node {
    std::vector<int32_t> key;        // one page of token ids
    std::vector<int32_t> pages;      // one page id per group
    std::map<std::vector<int32_t>, int> children;
    int parent = -1;
    int users = 0;                   // live requests whose prefix runs through here
    long long last_used = 0;
    bool alive = false;
};

struct Memory {
    int page_size = 0, max_requests = 0, max_pages = 0;
    std::vector<Group> groups;
    std::vector<Request> requests;
    std::vector<int32_t> free_slots;
    // prefix tree (node 0 is the root)
    bool tree = false;
    std::vector<Node> nodes;
    std::vector<int> free_nodes;
    long long clock = 0, hits = 0;
    int num_nodes = 0, idle = 0;
    std::string error;

    int fail(const std::string& msg) {
        error = msg;
        return kErr;
    }
    long long pages_for(long long length) const { return (length + page_size - 1) / page_size; }

    // ------------------------------------------------------------------ pool
    int pool_check(int g, int page) {
        if (g < 0 || g >= (int)groups.size()) return fail("no group " + std::to_string(g));
        if (page < 0 || page >= groups[g].pool.num_pages)
            return fail("page id " + std::to_string(page) + " outside pool of " +
                        std::to_string(groups[g].pool.num_pages));
        return 0;
    }
    int pool_allocate(int g) {
        Pool& p = groups[g].pool;
        if (p.free_list.empty()) return -1;
        const int page = p.free_list.back();
        p.free_list.pop_back();
        p.refs[page] = 1;
        return page;
    }
    int pool_retain(int g, int page) {
        if (pool_check(g, page)) return kErr;
        Pool& p = groups[g].pool;
        if (p.refs[page] == 0) return fail("page " + std::to_string(page) + " is free and cannot be retained");
        ++p.refs[page];
        return 0;
    }
    int pool_release(int g, int page) {          // 1: the page went back to the free list
        if (pool_check(g, page)) return kErr;
        Pool& p = groups[g].pool;
        if (p.refs[page] == 0) return fail("page " + std::to_string(page) + " freed twice");
        if (--p.refs[page] == 0) {
            p.free_list.push_back(page);
            return 1;
        }
        return 0;
    }

    void set_cell(Group& g, int slot, int index, int page) {
        const int flat = slot * max_pages + index;
        g.table[flat] = page;
        g.updates.push_back(flat);
        g.updates.push_back(page);
    }
    Request* request(int slot) {
        if (slot < 0 || slot >= max_requests || !requests[slot].open) {
            fail("slot " + std::to_string(slot) + " holds no request");
            return nullptr;
        }
        return &requests[slot];
    }
};

Memory* M(void* h) { return static_cast<Memory*>(h); }

bool no_group(Memory* m, int g) {
    if (g >= 0 && g < (int)m->groups.size()) return false;
    m->fail("no group " + std::to_string(g));
    return true;
}

}  // namespace

// ----------------------------------------------------------------------------- life cycle
// windows[g] < 0: group g keeps all keys.  Returns nullptr on nonsense sizes.
LSB_API void* lsbm_create(int page_size, int max_requests, int max_pages, int n_groups, const int* windows,
                          const int* num_pages) {
    if (page_size <= 0 || max_requests <= 0 || max_pages <= 0 || n_groups < 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (num_pages[g] <= 0) return nullptr;
    Memory* m = new Memory;
    m->page_size = page_size;
    m->max_requests = max_requests;
    m->max_pages = max_pages;
    m->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        Group& gr = m->groups[g];
        gr.window = windows[g];
        gr.pool.num_pages = num_pages[g];
        gr.pool.refs.assign(num_pages[g], 0);
        gr.pool.tree_refs.assign(num_pages[g], 0);
        gr.pool.free_list.resize(num_pages[g]);
        for (int p = 0; p < num_pages[g]; ++p) gr.pool.free_list[p] = num_pages[g] - 1 - p;   // pops 0, 1, 2, ...
        gr.table.assign((size_t)max_requests * max_pages, kNoPage);
        gr.first_live.assign(max_requests, 0);
    }
    m->requests.resize(max_requests);
    m->free_slots.resize(max_requests);
    for (int s = 0; s < max_requests; ++s) m->free_slots[s] = max_requests - 1 - s;
    return m;
}

LSB_API void lsbm_destroy(void* h) { delete M(h); }

LSB_API const char* lsbm_last_error(void* h) { return M(h)->error.c_str(); }
LSB_API int lsbm_page_size(void* h) { return M(h)->page_size; }
LSB_API int lsbm_max_pages(void* h) { return M(h)->max_pages; }
// Pages of the smallest pool (1 << 30 if there is none): what a single request can ever hold.
LSB_API int lsbm_smallest_pool(void* h) {
    int n = 1 << 30;
    for (Group& g : M(h)->groups) n = std::min(n, g.pool.num_pages);
    return n;
}

// ----------------------------------------------------------------------------- pools
LSB_API int lsbm_pool_allocate(void* h, int g) {
    if (g < 0 || g >= (int)M(h)->groups.size()) return M(h)->fail("no group " + std::to_string(g));
    return M(h)->pool_allocate(g);
}
LSB_API int lsbm_pool_retain(void* h, int g, int page) { return M(h)->pool_retain(g, page); }
LSB_API int lsbm_pool_release(void* h, int g, int page) { return M(h)->pool_release(g, page); }
LSB_API int lsbm_pool_refcount(void* h, int g, int page) {
    if (M(h)->pool_check(g, page)) return kErr;
    return M(h)->groups[g].pool.refs[page];
}
LSB_API int lsbm_pool_num_free(void* h, int g) { return no_group(M(h), g) ? kErr : (int)M(h)->groups[g].pool.free_list.size(); }
LSB_API int lsbm_pool_num_pages(void* h, int g) { return no_group(M(h), g) ? kErr : M(h)->groups[g].pool.num_pages; }

// Free list and reference counts agree: no page on the list twice, free exactly when unreferenced.
static int pool_invariants(Memory* m, int g) {
    Pool& p = m->groups[g].pool;
    std::vector<char> on_list(p.num_pages, 0);
    for (int page : p.free_list) {
        if (on_list[page]) return m->fail("a page is on the free list twice");
        on_list[page] = 1;
    }
    for (int page = 0; page < p.num_pages; ++page)
        if ((p.refs[page] == 0) != (on_list[page] != 0))
            return m->fail("page " + std::to_string(page) + ": refcount " + std::to_string(p.refs[page]) +
                           " disagrees with free list");
    return 0;
}
LSB_API int lsbm_pool_check(void* h, int g) { return no_group(M(h), g) ? kErr : pool_invariants(M(h), g); }

// ----------------------------------------------------------------------------- requests
// A free slot (block-table row and state row) for a new request, or -1 if all are taken.
LSB_API int lsbm_open(void* h) {
    Memory* m = M(h);
    if (m->free_slots.empty()) return -1;
    const int slot = m->free_slots.back();
    m->free_slots.pop_back();
    m->requests[slot] = Request();
    m->requests[slot].open = true;
    for (Group& g : m->groups) g.first_live[slot] = 0;
    return slot;
}

LSB_API long long lsbm_length(void* h, int slot) {
    Request* r = M(h)->request(slot);
    return r ? r->length : kErr;
}
LSB_API int lsbm_num_pages(void* h, int slot) {
    Request* r = M(h)->request(slot);
    return r ? r->num_pages : kErr;
}
LSB_API int lsbm_first_live(void* h, int g, int slot) {
    if (no_group(M(h), g) || slot < 0 || slot >= M(h)->max_requests) return kErr;
    return M(h)->groups[g].first_live[slot];
}

// Pages free in the tightest group.
LSB_API int lsbm_free_pages(void* h) {
    int n = 1 << 30;
    for (Group& g : M(h)->groups) n = std::min(n, (int)g.pool.free_list.size());
    return n;
}

// Cover positions [0, new_length) with pages in every group, or change nothing.
// 1: covered; 0: a pool is short; kErr: the block table cannot hold that many pages.
LSB_API int lsbm_reserve(void* h, int slot, long long new_length) {
    Memory* m = M(h);
    Request* r = m->request(slot);
    if (!r) return kErr;
    const long long want = m->pages_for(new_length);
    if (want > m->max_pages)
        return m->fail(std::to_string(new_length) + " tokens need " + std::to_string(want) +
                       " pages, a block table holds " + std::to_string(m->max_pages));
    const int need = (int)want - r->num_pages;
    if (need <= 0) return 1;
    for (Group& g : m->groups)
        if ((int)g.pool.free_list.size() < need) return 0;
    for (size_t gi = 0; gi < m->groups.size(); ++gi)
        for (int i = r->num_pages; i < (int)want; ++i) m->set_cell(m->groups[gi], slot, i, m->pool_allocate((int)gi));
    r->num_pages = (int)want;
    return 1;
}

// The request now holds new_length tokens; pages that a window has passed go back to their pool.
LSB_API int lsbm_commit(void* h, int slot, long long new_length) {
    Memory* m = M(h);
    Request* r = m->request(slot);
    if (!r) return kErr;
    if (m->pages_for(new_length) > r->num_pages)
        return m->fail("length " + std::to_string(new_length) + " is not covered by its pages");
    r->length = new_length;
    for (size_t gi = 0; gi < m->groups.size(); ++gi) {
        Group& g = m->groups[gi];
        if (g.window < 0) continue;
        // the next query sits at position >= new_length and sees keys > position - window
        const long long first_needed = std::max(0LL, new_length - g.window + 1);
        const int dead = (int)std::min<long long>(first_needed / m->page_size, r->num_pages);
        for (int i = g.first_live[slot]; i < dead; ++i) {
            if (m->pool_release((int)gi, g.table[(size_t)slot * m->max_pages + i]) == kErr) return kErr;
            m->set_cell(g, slot, i, kNoPage);
        }
        g.first_live[slot] = std::max(g.first_live[slot], dead);
    }
    return 0;
}

// The request is over: every page it holds and its slot go back.
LSB_API int lsbm_close(void* h, int slot) {
    Memory* m = M(h);
    Request* r = m->request(slot);
    if (!r) return kErr;
    for (size_t gi = 0; gi < m->groups.size(); ++gi) {
        Group& g = m->groups[gi];
        for (int i = g.first_live[slot]; i < r->num_pages; ++i) {
            if (m->pool_release((int)gi, g.table[(size_t)slot * m->max_pages + i]) == kErr) return kErr;
            m->set_cell(g, slot, i, kNoPage);
        }
        g.first_live[slot] = 0;
    }
    r->open = false;
    m->free_slots.push_back(slot);
    return 0;
}

// Start a fresh request on pages that already hold its first `length` tokens; one reference is
// taken on each.  pages: [groups][n].
LSB_API int lsbm_adopt(void* h, int slot, const int* pages, int n, long long length) {
    Memory* m = M(h);
    Request* r = m->request(slot);
    if (!r) return kErr;
    if (r->num_pages || length % m->page_size) return m->fail("adopt needs a fresh request and a whole number of pages");
    if ((long long)n * m->page_size != length) return m->fail("adopt: page list does not match the length");
    if (n > m->max_pages) return m->fail("adopt: more pages than a block table holds");
    const int G = (int)m->groups.size();
    for (int g = 0; g < G; ++g)
        for (int i = 0; i < n; ++i) {
            const int p = pages[(size_t)g * n + i];
            if (m->pool_check(g, p)) return kErr;
            if (m->groups[g].pool.refs[p] == 0)
                return m->fail("page " + std::to_string(p) + " is free and cannot be retained");
        }
    for (int g = 0; g < G; ++g)
        for (int i = 0; i < n; ++i) {
            const int p = pages[(size_t)g * n + i];
            ++m->groups[g].pool.refs[p];
            m->set_cell(m->groups[g], slot, i, p);
        }
    r->num_pages = n;
    r->length = length;
    return 0;
}

// out[0 .. num_pages) = the request's pages in `group`; returns their number.
LSB_API int lsbm_pages_of(void* h, int slot, int group, int* out, int cap) {
    Memory* m = M(h);
    Request* r = m->request(slot);
    if (!r || no_group(m, group)) return kErr;
    if (cap < r->num_pages) return m->fail("pages_of: buffer too small");
    const int32_t* row = &m->groups[group].table[(size_t)slot * m->max_pages];
    for (int i = 0; i < r->num_pages; ++i) out[i] = row[i];
    return r->num_pages;
}

// ----------------------------------------------------------------------------- tables
LSB_API int32_t* lsbm_table(void* h, int group) { return no_group(M(h), group) ? nullptr : M(h)->groups[group].table.data(); }
LSB_API int lsbm_num_updates(void* h, int group) {
    return no_group(M(h), group) ? kErr : (int)(M(h)->groups[group].updates.size() / 2);
}
// Block-table cells changed since the last call, as (flat index, value) pairs, oldest first.
LSB_API int lsbm_take_updates(void* h, int group, int* out, int cap_pairs) {
    if (no_group(M(h), group)) return kErr;
    Group& g = M(h)->groups[group];
    const int n = (int)(g.updates.size() / 2);
    if (cap_pairs < n) return M(h)->fail("take_updates: buffer too small");
    std::copy(g.updates.begin(), g.updates.end(), out);
    g.updates.clear();
    return n;
}

// The same as two arrays, cells and values, with one entry per cell: where a cell changed more than
// once since the last call only its last value is given (the device applies the entries in no
// particular order).  Returns the number of entries.
LSB_API int lsbm_take_updates_last(void* h, int group, int* cells, int* values, int cap) {
    if (no_group(M(h), group)) return kErr;
    Group& g = M(h)->groups[group];
    const int n = (int)(g.updates.size() / 2);
    if (cap < n) return M(h)->fail("take_updates_last: buffer too small");
    int out = 0;
    // newest first: a cell that this call has given out already is an older write
    if (g.taken.size() != g.table.size()) g.taken.assign(g.table.size(), 0u);
    if (++g.take_call == 0) {                       // the counter came round: start afresh
        std::fill(g.taken.begin(), g.taken.end(), 0u);
        g.take_call = 1;
    }
    for (int i = n - 1; i >= 0; --i) {
        const int32_t cell = g.updates[2 * i];
        if (cell < 0 || (size_t)cell >= g.taken.size()) return M(h)->fail("take_updates_last: a cell outside the table");
        if (g.taken[cell] == g.take_call) continue;
        g.taken[cell] = g.take_call;
        cells[out] = cell;
        values[out] = g.updates[2 * i + 1];
        ++out;
    }
    g.updates.clear();
    return out;
}

// ----------------------------------------------------------------------------- prefix tree
// A node owns one page per group: the keys and values of its chunk of tokens after the path above
// it.  Only whole pages are shared and a match never covers the last token of a prompt, so there is
// always something to run.  Nodes that no live request uses can be evicted, leaves first, least
// recently used first.
namespace {

int new_node(Memory* m, int parent, const int32_t* key, const std::vector<int32_t>& pages) {
    int id;
    if (!m->free_nodes.empty()) {
        id = m->free_nodes.back();
        m->free_nodes.pop_back();
    } else {
        id = (int)m->nodes.size();
        m->nodes.emplace_back();
    }
    Node& n = m->nodes[id];
    n = Node();
    n.key.assign(key, key + m->page_size);
    n.pages = pages;
    n.parent = parent;
    n.alive = true;
    for (size_t g = 0; g < pages.size(); ++g) {
        ++m->groups[g].pool.refs[pages[g]];          // the caller has checked that they are held
        ++m->groups[g].pool.tree_refs[pages[g]];
    }
    m->nodes[parent].children[n.key] = id;
    ++m->num_nodes;
    ++m->idle;
    return id;
}

int node_check(Memory* m, int id) {
    if (!m->tree) return m->fail("the prefix tree is not enabled");
    if (id <= 0 || id >= (int)m->nodes.size() || !m->nodes[id].alive)
        return m->fail("no prefix node " + std::to_string(id));
    return 0;
}

// The pages of the request's i-th logical page, one per group.
void pages_at(Memory* m, int slot, int i, std::vector<int32_t>& out) {
    out.resize(m->groups.size());
    for (size_t g = 0; g < m->groups.size(); ++g) out[g] = m->groups[g].table[(size_t)slot * m->max_pages + i];
}

}  // namespace

// Sharing needs every layer to keep all its keys: refused if a group has a window.
LSB_API int lsbp_enable(void* h) {
    Memory* m = M(h);
    for (Group& g : m->groups)
        if (g.window >= 0) return m->fail("prefix sharing needs every layer to keep all its keys");
    if (!m->tree) {
        m->tree = true;
        m->nodes.assign(1, Node());
        m->nodes[0].alive = true;
    }
    return 0;
}

// Nodes of the longest cached prefix of tokens[0 .. n): whole pages, never the last token.
LSB_API int lsbp_match(void* h, const int* tokens, long long n, int* out, int cap) {
    Memory* m = M(h);
    if (!m->tree) return m->fail("the prefix tree is not enabled");
    const long long limit = n > 0 ? (n - 1) / m->page_size : 0;
    int node = 0, found = 0;
    std::vector<int32_t> key(m->page_size);
    for (long long i = 0; i < limit && found < cap; ++i) {
        key.assign(tokens + i * m->page_size, tokens + (i + 1) * m->page_size);
        auto it = m->nodes[node].children.find(key);
        if (it == m->nodes[node].children.end()) break;
        node = it->second;
        out[found++] = node;
    }
    return found;
}

// Start the request in `slot` (open, no pages yet) on the pages of the path; returns tokens covered.
LSB_API long long lsbp_adopt(void* h, int slot, const int* path, int n) {
    Memory* m = M(h);
    if (n <= 0) return 0;
    for (int i = 0; i < n; ++i)
        if (node_check(m, path[i])) return kErr;
    const int G = (int)m->groups.size();
    std::vector<int> pages((size_t)G * n);
    for (int g = 0; g < G; ++g)
        for (int i = 0; i < n; ++i) pages[(size_t)g * n + i] = m->nodes[path[i]].pages[g];
    if (lsbm_adopt(h, slot, pages.data(), n, (long long)n * m->page_size) == kErr) return kErr;
    const long long now = ++m->clock;
    for (int i = 0; i < n; ++i) {
        Node& nd = m->nodes[path[i]];
        if (nd.users == 0) --m->idle;
        ++nd.users;
        nd.last_used = now;
    }
    m->hits += n;
    return (long long)n * m->page_size;
}

// The request that used these nodes is gone (its page references are dropped by close).
LSB_API int lsbp_release(void* h, const int* path, int n) {
    Memory* m = M(h);
    for (int i = 0; i < n; ++i) {
        if (node_check(m, path[i])) return kErr;
        if (m->nodes[path[i]].users <= 0) return m->fail("prefix node " + std::to_string(path[i]) + " has no user to release");
    }
    const long long now = ++m->clock;
    for (int i = 0; i < n; ++i) {
        Node& nd = m->nodes[path[i]];
        if (--nd.users == 0) ++m->idle;
        nd.last_used = now;
    }
    return 0;
}

// Keep the full pages of the request in `slot`, which holds tokens[0 .. n), for later prompts.  Call
// before the request is closed.  Returns the number of pages newly kept.
LSB_API int lsbp_insert(void* h, const int* tokens, long long n, int slot) {
    Memory* m = M(h);
    if (!m->tree) return m->fail("the prefix tree is not enabled");
    Request* r = m->request(slot);
    if (!r) return kErr;
    const long long n_full = std::min(n, r->length) / m->page_size;
    const long long now = ++m->clock;
    int node = 0, kept = 0;
    std::vector<int32_t> key(m->page_size), mine;
    for (long long i = 0; i < n_full; ++i) {
        key.assign(tokens + i * m->page_size, tokens + (i + 1) * m->page_size);
        auto it = m->nodes[node].children.find(key);
        int child;
        if (it == m->nodes[node].children.end()) {
            pages_at(m, slot, (int)i, mine);
            child = new_node(m, node, key.data(), mine);
            ++kept;
        } else {
            child = it->second;
        }
        m->nodes[child].last_used = now;
        node = child;
    }
    return kept;
}

// Like insert, for a request that goes on running: the pages that tokens[0 .. n) fill become visible
// to later prompts now.  held: nodes the request already counts as a user of.  added receives the
// further nodes whose pages are the request's own; it is a user of those too until release, so that
// they are not offered for eviction while evicting them would free nothing.
LSB_API int lsbp_share(void* h, const int* tokens, long long n, int slot, const int* held, int n_held,
                       int* added, int cap) {
    Memory* m = M(h);
    if (!m->tree) return m->fail("the prefix tree is not enabled");
    Request* r = m->request(slot);
    if (!r) return kErr;
    // (the step that fills these pages may only be planned yet: whoever reads them is queued
    // behind it, so the pages count as full as soon as they are the request's)
    const long long n_full = std::min<long long>(n / m->page_size, r->num_pages);
    const long long now = ++m->clock;
    int node = 0, n_added = 0;
    std::vector<int32_t> key(m->page_size), mine;
    for (long long i = 0; i < n_full; ++i) {
        key.assign(tokens + i * m->page_size, tokens + (i + 1) * m->page_size);
        pages_at(m, slot, (int)i, mine);
        auto it = m->nodes[node].children.find(key);
        const int child = it == m->nodes[node].children.end() ? new_node(m, node, key.data(), mine) : it->second;
        Node& nd = m->nodes[child];
        nd.last_used = now;
        if (nd.pages == mine && std::find(held, held + n_held, child) == held + n_held) {
            if (n_added >= cap) return m->fail("share: buffer too small");
            if (nd.users == 0) --m->idle;
            ++nd.users;
            added[n_added++] = child;
        }
        node = child;
    }
    return n_added;
}

LSB_API int lsbp_evictable(void* h) { return M(h)->idle; }
LSB_API int lsbp_num_nodes(void* h) { return M(h)->num_nodes; }
LSB_API long long lsbp_hits(void* h) { return M(h)->hits; }

// Give back up to `wanted` pages per group: unused leaves, least recently used first; a parent
// that becomes a leaf is looked at in the next round.  Returns how many nodes were freed.
LSB_API int lsbp_evict(void* h, int wanted) {
    Memory* m = M(h);
    if (!m->tree) return 0;
    int freed = 0;
    std::vector<int> leaves;
    while (freed < wanted) {
        leaves.clear();
        for (int id = 1; id < (int)m->nodes.size(); ++id) {
            const Node& nd = m->nodes[id];
            if (nd.alive && nd.children.empty() && nd.users == 0) leaves.push_back(id);
        }
        if (leaves.empty()) break;
        std::stable_sort(leaves.begin(), leaves.end(),
                         [m](int a, int b) { return m->nodes[a].last_used < m->nodes[b].last_used; });
        for (int id : leaves) {
            if (freed >= wanted) break;
            Node& nd = m->nodes[id];
            for (size_t g = 0; g < nd.pages.size(); ++g) {
                --m->groups[g].pool.tree_refs[nd.pages[g]];
                if (m->pool_release((int)g, nd.pages[g]) == kErr) return kErr;
            }
            m->nodes[nd.parent].children.erase(nd.key);
            nd.alive = false;
            nd.children.clear();
            m->free_nodes.push_back(id);
            --m->num_nodes;
            --m->idle;
            ++freed;
        }
    }
    return freed;
}

LSB_API int lsbp_node_users(void* h, int id) { return node_check(M(h), id) ? kErr : M(h)->nodes[id].users; }
LSB_API int lsbp_node_pages(void* h, int id, int* out) {
    if (node_check(M(h), id)) return kErr;
    const Node& nd = M(h)->nodes[id];
    std::copy(nd.pages.begin(), nd.pages.end(), out);
    return (int)nd.pages.size();
}
// How many nodes of the path no live request uses (they count as evictable, but not for a request
// that is about to adopt them).
LSB_API int lsbp_idle_on(void* h, const int* path, int n) {
    int idle = 0;
    for (int i = 0; i < n; ++i) {
        if (node_check(M(h), path[i])) return kErr;
        idle += M(h)->nodes[path[i]].users == 0;
    }
    return idle;
}

// ----------------------------------------------------------------------------- invariants
// No page lost, none held without a reference, none freed twice, no slot lost or held twice; the
// counters of the prefix tree agree with the tree.  0 if all holds, else kErr with a message.
LSB_API int lsbm_check(void* h) {
    Memory* m = M(h);
    for (size_t gi = 0; gi < m->groups.size(); ++gi) {
        Group& g = m->groups[gi];
        if (pool_invariants(m, (int)gi)) return kErr;
        std::vector<int32_t> held(g.pool.num_pages, 0);
        for (int slot = 0; slot < m->max_requests; ++slot) {
            const int32_t* row = &g.table[(size_t)slot * m->max_pages];
            const Request& r = m->requests[slot];
            const int covered = r.open ? r.num_pages : 0;
            for (int i = 0; i < covered; ++i) {
                const int p = row[i];
                if (i < g.first_live[slot]) {
                    if (p != kNoPage) return m->fail("released cell still names page " + std::to_string(p));
                    continue;
                }
                if (p == kNoPage) return m->fail("slot " + std::to_string(slot) + " lacks page " + std::to_string(i));
                if (p < 0 || p >= g.pool.num_pages) return m->fail("a block table names page " + std::to_string(p));
                ++held[p];
            }
            for (int i = covered; i < m->max_pages; ++i)
                if (row[i] != kNoPage) return m->fail("slot " + std::to_string(slot) + ": cells past its pages are set");
        }
        for (int p = 0; p < g.pool.num_pages; ++p)
            if (g.pool.refs[p] != held[p] + g.pool.tree_refs[p])
                return m->fail("page " + std::to_string(p) + ": refcount " + std::to_string(g.pool.refs[p]) +
                               " but " + std::to_string(held[p] + g.pool.tree_refs[p]) + " owners known");
    }
    std::vector<char> seen(m->max_requests, 0);
    for (int s : m->free_slots) {
        if (s < 0 || s >= m->max_requests || seen[s] || m->requests[s].open) return m->fail("a slot is held twice");
        seen[s] = 1;
    }
    int open = 0;
    for (const Request& r : m->requests) open += r.open;
    if (open + (int)m->free_slots.size() != m->max_requests) return m->fail("a slot was lost");
    if (m->tree) {
        int alive = 0, idle = 0;
        std::vector<std::vector<int32_t>> owned(m->groups.size());
        for (size_t g = 0; g < m->groups.size(); ++g) owned[g].assign(m->groups[g].pool.num_pages, 0);
        for (int id = 1; id < (int)m->nodes.size(); ++id) {
            const Node& nd = m->nodes[id];
            if (!nd.alive) continue;
            ++alive;
            idle += nd.users == 0;
            if (nd.users < 0) return m->fail("prefix tree: a node has fewer than zero users");
            if (!m->nodes[nd.parent].alive) return m->fail("prefix tree: a node hangs on a node that is gone");
            auto it = m->nodes[nd.parent].children.find(nd.key);
            if (it == m->nodes[nd.parent].children.end() || it->second != id)
                return m->fail("prefix tree: a node is not among its parent's children");
            for (size_t g = 0; g < nd.pages.size(); ++g) ++owned[g][nd.pages[g]];
        }
        if (alive != m->num_nodes || idle != m->idle)
            return m->fail("prefix tree: " + std::to_string(alive) + " nodes / " + std::to_string(m->num_nodes) +
                           " counted, " + std::to_string(idle) + " idle / " + std::to_string(m->idle) + " counted");
        for (size_t g = 0; g < m->groups.size(); ++g)
            if (owned[g] != m->groups[g].pool.tree_refs) return m->fail("prefix tree: page ownership counters are off");
    }
    return 0;
}
