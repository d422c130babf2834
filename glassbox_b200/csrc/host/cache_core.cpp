// Host-side bookkeeping of the paged cache and the layout of a step's metadata block, in C++.
//
// The device only ever sees block tables and slots; every decision about pages is taken here. The
// semantics follow crates/glassbox-core/src/kv.rs: pages of a fixed number of tokens (kv.rs:11), a
// free stack from which page 0 pops first (kv.rs:67), reference counts, copy-on-write of a shared
// partial last page (kv.rs:161-196), fork (kv.rs:260-266), truncate (kv.rs:237-257), and prefix
// sharing by a chained FNV-1a hash of whole pages (kv.rs:45-55, 135-157, 205-233) with unreferenced
// hashed pages kept for reuse until space is needed, oldest evicted first (kv.rs:96-110).
//
// Beyond the reference: several *groups* of layers, each with a page pool and block tables of its
// own (a group with a window gives pages back as soon as the window has passed them), all-or-nothing
// reservation across the groups, and one fixed-size *state slot* per live request.
//
// The interface is a C ABI over an opaque handle, loaded with ctypes; requests are named by 64-bit
// ids that the caller chooses. Every function returns 0 on success, 1 when pages or slots ran out
// (nothing was changed), 2 for a bad argument, 3 for an unknown request; gbh_last_error() has the text.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

#define GBH_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local char g_error[512];

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

enum { OK = 0, OUT_OF_PAGES = 1, BAD_VALUE = 2, UNKNOWN_REQUEST = 3 };

constexpr uint64_t FNV_OFFSET = 0xCBF29CE484222325ull, FNV_PRIME = 0x100000001B3ull;

// FNV-1a over the previous hash and one page of token ids as little-endian u32 bytes (kv.rs:45-55)
uint64_t chain_hash(uint64_t prev, const int32_t* tokens, int n) {
    uint64_t h = prev ^ FNV_OFFSET;
    for (int i = 0; i < n; ++i) {
        const uint32_t t = (uint32_t)tokens[i];
        for (int b = 0; b < 4; ++b) {
            h ^= (t >> (8 * b)) & 0xFFu;
            h *= FNV_PRIME;
        }
    }
    return h;
}

struct Group {
    int num_pages, page_size, window;   // window < 0: keep every token
    bool share;
    std::vector<int> refs;
    std::vector<int> free;              // a stack; page 0 pops first
    std::deque<int> cached;             // unreferenced hashed pages kept for reuse, oldest first
    std::vector<char> hashed;
    std::vector<uint64_t> page_hash;
    std::unordered_map<uint64_t, int> by_hash;
    std::unordered_map<int64_t, std::vector<int>> tables;

    int free_pages() const { return (int)(free.size() + cached.size()); }

    int alloc() {   // the caller has checked that a page is free
        int p;
        if (!free.empty()) {
            p = free.back();
            free.pop_back();
        } else {
            p = cached.front();
            cached.pop_front();
            if (hashed[p]) {
                hashed[p] = 0;
                by_hash.erase(page_hash[p]);
            }
        }
        refs[p] = 1;
        return p;
    }

    void release(int p) {
        if (--refs[p] == 0) {
            if (hashed[p]) cached.push_back(p);
            else free.push_back(p);
        }
    }

    void retain(int p) {
        if (refs[p] == 0) cached.erase(std::find(cached.begin(), cached.end(), p));
        ++refs[p];
    }

    // index of the first page that a query at position >= length can still see
    int first_live_page(int length) const {
        if (window < 0) return 0;
        return std::max(0, length - window + 1) / page_size;
    }

    // (new pages, copy-on-write needed) to write positions length .. length+n-1
    void plan(const std::vector<int>& table, int length, int n, int* fresh, bool* cow) const {
        const int need = (length + n + page_size - 1) / page_size;
        *fresh = std::max(0, need - (int)table.size());
        *cow = false;
        if (n > 0 && length % page_size && length / page_size < (int)table.size()) {
            const int last = table[length / page_size];
            *cow = last >= 0 && refs[last] > 1;
        }
    }
};

struct Request {
    int length = 0;                 // tokens whose keys/values (or state) are written
    std::vector<int32_t> tokens;
    int slot = -1;
};

struct Cache {
    std::vector<Group> groups;
    std::unordered_map<int64_t, Request> requests;
    int max_requests = 0;
    bool share = false;
    std::vector<int> free_slots;    // a stack; slot 0 pops first
    std::vector<int> fresh_slots;   // handed out since the last drain: to be zeroed on the device
};

Request* find(Cache* c, int64_t rid) {
    auto it = c->requests.find(rid);
    return it == c->requests.end() ? nullptr : &it->second;
}

}  // namespace

GBH_EXPORT const char* gbh_last_error() { return g_error; }

GBH_EXPORT uint64_t gbh_chain_hash(uint64_t prev, const int32_t* tokens, int n) { return chain_hash(prev, tokens, n); }

// window[g] < 0: the group keeps every token. Prefix sharing is only sound when what a page holds is a pure
// function of the token prefix for every mixer: it is switched off when a group has a window or a request has state.
GBH_EXPORT void* gbh_cache_new(int n_groups, const int* num_pages, const int* page_size, const int* window,
                               int max_requests, int share_prefixes, int has_state) {
    for (int g = 0; g < n_groups; ++g)
        if (num_pages[g] <= 0 || page_size[g] <= 0) {
            fail(BAD_VALUE, "a cache group needs a positive number of pages and a positive page size");
            return nullptr;
        }
    Cache* c = new Cache();
    bool sound = share_prefixes && !has_state;
    for (int g = 0; g < n_groups; ++g) sound = sound && window[g] < 0;
    c->share = sound;
    c->max_requests = max_requests;
    c->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        Group& gr = c->groups[g];
        gr.num_pages = num_pages[g];
        gr.page_size = page_size[g];
        gr.window = window[g];
        gr.share = sound;
        gr.refs.assign(gr.num_pages, 0);
        gr.hashed.assign(gr.num_pages, 0);
        gr.page_hash.assign(gr.num_pages, 0);
        gr.free.resize(gr.num_pages);
        for (int p = 0; p < gr.num_pages; ++p) gr.free[p] = gr.num_pages - 1 - p;
    }
    c->free_slots.resize(std::max(max_requests, 0));
    for (int s = 0; s < max_requests; ++s) c->free_slots[s] = max_requests - 1 - s;
    return c;
}

GBH_EXPORT void gbh_cache_delete(void* h) { delete static_cast<Cache*>(h); }

GBH_EXPORT int gbh_cache_shares_prefixes(void* h) { return static_cast<Cache*>(h)->share ? 1 : 0; }

// Start a request. With prefix sharing, whole leading pages whose token prefix is already cached are
// shared; never the page that holds the last prompt token, which must still run to give logits
// (kv.rs:135-157). *present receives the number of tokens already in the cache.
GBH_EXPORT int gbh_cache_add(void* h, int64_t rid, const int32_t* prompt, int n, int* present) {
    Cache* c = static_cast<Cache*>(h);
    if (find(c, rid)) return fail(BAD_VALUE, "the request exists");
    if (c->free_slots.empty()) return fail(OUT_OF_PAGES, "no free state slot");
    Request req;
    req.tokens.assign(prompt, prompt + n);
    req.slot = c->free_slots.back();
    c->free_slots.pop_back();
    c->fresh_slots.push_back(req.slot);
    for (Group& g : c->groups) g.tables[rid].clear();
    if (c->share && !c->groups.empty()) {
        const int ps = c->groups[0].page_size;
        bool same = true;
        for (const Group& g : c->groups) same = same && g.page_size == ps;
        if (same) {
            uint64_t hash = 0;
            int reused = 0;
            std::vector<int> pages(c->groups.size());
            for (int i = 0; i < n / ps; ++i) {
                if ((i + 1) * ps >= n) break;
                hash = chain_hash(hash, prompt + i * ps, ps);
                bool all = true;
                for (size_t g = 0; g < c->groups.size() && all; ++g) {
                    auto it = c->groups[g].by_hash.find(hash);
                    if (it == c->groups[g].by_hash.end()) all = false;
                    else pages[g] = it->second;
                }
                if (!all) break;
                for (size_t g = 0; g < c->groups.size(); ++g) {
                    c->groups[g].retain(pages[g]);
                    c->groups[g].tables[rid].push_back(pages[g]);
                }
                ++reused;
            }
            req.length = reused * ps;
        }
    }
    *present = req.length;
    c->requests.emplace(rid, std::move(req));
    return OK;
}

// Make room to write positions length .. length+n-1 in every group, all or nothing. copies receives the
// copy-on-write work as (group, source page, destination page) triples (at most one per group) that the
// caller must carry out on the device before the step (kv.rs:161-196).
GBH_EXPORT int gbh_cache_reserve(void* h, int64_t rid, int n, int* copies, int* n_copies) {
    Cache* c = static_cast<Cache*>(h);
    Request* req = find(c, rid);
    if (!req) return fail(UNKNOWN_REQUEST, "unknown request");
    if (n < 0) return fail(BAD_VALUE, "cannot reserve a negative number of tokens");
    const size_t G = c->groups.size();
    std::vector<int> fresh(G);
    std::vector<char> cow(G);
    for (size_t g = 0; g < G; ++g) {
        bool w;
        c->groups[g].plan(c->groups[g].tables[rid], req->length, n, &fresh[g], &w);
        cow[g] = w;
        if (fresh[g] + (w ? 1 : 0) > c->groups[g].free_pages()) return fail(OUT_OF_PAGES, "out of pages");
    }
    int nc = 0;
    for (size_t g = 0; g < G; ++g) {
        Group& gr = c->groups[g];
        std::vector<int>& table = gr.tables[rid];
        if (cow[g]) {
            const int i = req->length / gr.page_size;
            const int old = table[i];
            const int page = gr.alloc();
            copies[3 * nc] = (int)g;
            copies[3 * nc + 1] = old;
            copies[3 * nc + 2] = page;
            ++nc;
            gr.release(old);
            table[i] = page;
        } else if (n > 0 && req->length % gr.page_size && req->length / gr.page_size < (int)table.size()) {
            // The write lands in a partly filled page that this request holds alone. If the page is still
            // indexed under the hash of what it held when it was full (a fork truncated into it while the
            // other holder was alive, then that holder went away), the index must forget it now: its
            // contents are about to change.
            const int p = table[req->length / gr.page_size];
            if (p >= 0 && gr.hashed[p]) {
                gr.by_hash.erase(gr.page_hash[p]);
                gr.hashed[p] = 0;
            }
        }
        for (int k = 0; k < fresh[g]; ++k) table.push_back(gr.alloc());
    }
    *n_copies = nc;
    return OK;
}

// Mark n more positions as written; hash pages that became full (kv.rs:205-233); give back pages that a
// window has passed.
GBH_EXPORT int gbh_cache_commit(void* h, int64_t rid, const int32_t* tokens, int n) {
    Cache* c = static_cast<Cache*>(h);
    Request* req = find(c, rid);
    if (!req) return fail(UNKNOWN_REQUEST, "unknown request");
    const int start = req->length;
    req->length += n;
    // The tokens named at admission are what the caller expected to run; what is hashed must be what ran.
    const bool as_expected = (int)req->tokens.size() >= req->length &&
                             (n == 0 || std::memcmp(req->tokens.data() + start, tokens, sizeof(int32_t) * (size_t)n) == 0);
    if (!as_expected) {
        req->tokens.resize(std::min<size_t>(req->tokens.size(), (size_t)start));
        req->tokens.insert(req->tokens.end(), tokens, tokens + n);
    }
    for (Group& g : c->groups) {
        std::vector<int>& table = g.tables[rid];
        if (g.share) {
            const int ps = g.page_size, first = start / ps, last = req->length / ps;
            uint64_t hash = 0;
            bool chained = false;
            for (int bi = first; bi < last; ++bi) {
                const int p = table[bi];
                if (g.hashed[p]) { chained = false; continue; }
                if (!chained) {   // the chain over pages 0 .. bi-1
                    hash = 0;
                    for (int k = 0; k < bi; ++k) hash = chain_hash(hash, req->tokens.data() + (size_t)k * ps, ps);
                    chained = true;
                }
                hash = chain_hash(hash, req->tokens.data() + (size_t)bi * ps, ps);
                if (g.by_hash.find(hash) == g.by_hash.end()) {
                    g.by_hash[hash] = p;
                    g.page_hash[p] = hash;
                    g.hashed[p] = 1;
                }
            }
        }
        if (g.window >= 0) {
            const int live = std::min(g.first_live_page(req->length), (int)table.size());
            for (int bi = 0; bi < live; ++bi)
                if (table[bi] >= 0) {
                    g.release(table[bi]);
                    table[bi] = -1;
                }
        }
    }
    return OK;
}

// commit for several requests in one call: request e brings counts[e] tokens, flat in `tokens`.
GBH_EXPORT int gbh_cache_commit_many(void* h, int n, const int64_t* rids, const int* counts, const int32_t* tokens) {
    int at = 0;
    for (int e = 0; e < n; ++e) {
        const int code = gbh_cache_commit(h, rids[e], tokens + at, counts[e]);
        if (code) return code;
        at += counts[e];
    }
    return OK;
}

// Forget everything after the first `length` tokens (kv.rs:237-257). Not available once a window has
// given pages back behind `length`.
GBH_EXPORT int gbh_cache_truncate(void* h, int64_t rid, int length) {
    Cache* c = static_cast<Cache*>(h);
    Request* req = find(c, rid);
    if (!req) return fail(UNKNOWN_REQUEST, "unknown request");
    if (length > req->length || length < 0) return fail(BAD_VALUE, "cannot truncate to more than is written");
    for (Group& g : c->groups)
        if (g.window >= 0) {
            const std::vector<int>& table = g.tables[rid];
            for (size_t i = (size_t)g.first_live_page(length); i < table.size(); ++i)
                if (table[i] < 0)
                    return fail(BAD_VALUE, "a windowed group has already released pages that the shorter request would need");
        }
    req->length = length;
    if ((int)req->tokens.size() > length) req->tokens.resize(length);
    for (Group& g : c->groups) {
        std::vector<int>& table = g.tables[rid];
        const int keep = std::min((int)table.size(), (length + g.page_size - 1) / g.page_size);
        std::vector<int> dropped(table.begin() + keep, table.end());
        table.resize(keep);
        if (length % g.page_size) {
            const int p = table[length / g.page_size];
            if (p >= 0 && g.refs[p] == 1 && g.hashed[p]) {
                g.by_hash.erase(g.page_hash[p]);
                g.hashed[p] = 0;
            }
        }
        for (int p : dropped)
            if (p >= 0) g.release(p);
    }
    return OK;
}

// New request sharing every page of the parent (kv.rs:260-266). Its state slot is a copy, not a share:
// slots receives (parent slot, child slot) for the device copy.
GBH_EXPORT int gbh_cache_fork(void* h, int64_t parent, int64_t child, int* slots) {
    Cache* c = static_cast<Cache*>(h);
    if (find(c, child)) return fail(BAD_VALUE, "the request exists");
    Request* src = find(c, parent);
    if (!src) return fail(UNKNOWN_REQUEST, "unknown request");
    if (c->free_slots.empty()) return fail(OUT_OF_PAGES, "no free state slot");
    Request req;
    req.length = src->length;
    req.tokens = src->tokens;
    req.slot = c->free_slots.back();
    c->free_slots.pop_back();
    for (Group& g : c->groups) {
        std::vector<int> table = g.tables[parent];
        for (int p : table)
            if (p >= 0) g.retain(p);
        g.tables[child] = std::move(table);
    }
    slots[0] = src->slot;
    slots[1] = req.slot;
    c->requests.emplace(child, std::move(req));
    return OK;
}

// Give back everything the request holds (kv.rs:268-274). Unknown ids are ignored.
GBH_EXPORT int gbh_cache_free(void* h, int64_t rid) {
    Cache* c = static_cast<Cache*>(h);
    auto it = c->requests.find(rid);
    if (it == c->requests.end()) return OK;
    for (Group& g : c->groups) {
        auto t = g.tables.find(rid);
        for (int p : t->second)
            if (p >= 0) g.release(p);
        g.tables.erase(t);
    }
    const int slot = it->second.slot;
    c->free_slots.push_back(slot);
    auto f = std::find(c->fresh_slots.begin(), c->fresh_slots.end(), slot);
    if (f != c->fresh_slots.end()) c->fresh_slots.erase(f);
    c->requests.erase(it);
    return OK;
}

// ------------------------------------------------------------------------------------------ queries
GBH_EXPORT int gbh_cache_has(void* h, int64_t rid) { return find(static_cast<Cache*>(h), rid) ? 1 : 0; }

GBH_EXPORT int gbh_cache_length(void* h, int64_t rid) {
    Request* r = find(static_cast<Cache*>(h), rid);
    return r ? r->length : -1;
}

// Lengths of several requests in one call (-1 for an unknown one).
GBH_EXPORT void gbh_cache_lengths(void* h, int n, const int64_t* rids, int* out) {
    for (int e = 0; e < n; ++e) out[e] = gbh_cache_length(h, rids[e]);
}

GBH_EXPORT int gbh_cache_slot(void* h, int64_t rid) {
    Request* r = find(static_cast<Cache*>(h), rid);
    return r ? r->slot : -1;
}

GBH_EXPORT int gbh_cache_free_pages(void* h, int group) { return static_cast<Cache*>(h)->groups[group].free_pages(); }

GBH_EXPORT int gbh_cache_ref_count(void* h, int group, int page) { return static_cast<Cache*>(h)->groups[group].refs[page]; }

// The request's block table in a group: returns its length (or -1) and copies up to cap entries.
GBH_EXPORT int gbh_cache_table(void* h, int group, int64_t rid, int* out, int cap) {
    Cache* c = static_cast<Cache*>(h);
    auto it = c->groups[group].tables.find(rid);
    if (it == c->groups[group].tables.end()) return -1;
    const int n = (int)it->second.size();
    if (out) std::memcpy(out, it->second.data(), sizeof(int) * std::min(n, cap));
    return n;
}

// The request's known tokens: returns their number and copies up to cap.
GBH_EXPORT int gbh_cache_tokens(void* h, int64_t rid, int32_t* out, int cap) {
    Request* r = find(static_cast<Cache*>(h), rid);
    if (!r) return -1;
    const int n = (int)r->tokens.size();
    if (out) std::memcpy(out, r->tokens.data(), sizeof(int32_t) * std::min(n, cap));
    return n;
}

// which: 0 free state slots, 1 fresh state slots (drained by the call when drain != 0)
GBH_EXPORT int gbh_cache_slots(void* h, int which, int drain, int* out, int cap) {
    Cache* c = static_cast<Cache*>(h);
    std::vector<int>& v = which == 0 ? c->free_slots : c->fresh_slots;
    const int n = (int)v.size();
    if (out) std::memcpy(out, v.data(), sizeof(int) * std::min(n, cap));
    if (drain && which == 1) v.clear();
    return n;
}

// The pool of a group for an outside check of the invariants. which: 0 reference counts [num_pages],
// 1 free stack, 2 cached pages oldest first, 3 hashed flags [num_pages]. Returns the count.
GBH_EXPORT int gbh_cache_pool(void* h, int group, int which, int* out, int cap) {
    Group& g = static_cast<Cache*>(h)->groups[group];
    std::vector<int> tmp;
    const std::vector<int>* src = &tmp;
    if (which == 0) src = &g.refs;
    else if (which == 1) src = &g.free;
    else if (which == 2) tmp.assign(g.cached.begin(), g.cached.end());
    else tmp.assign(g.hashed.begin(), g.hashed.end());
    const int n = (int)src->size();
    if (out) std::memcpy(out, src->data(), sizeof(int) * std::min(n, cap));
    return n;
}

// The hash index of a group as (hash, page) pairs and each page's own hash; returns the number of pairs.
GBH_EXPORT int gbh_cache_hashes(void* h, int group, uint64_t* hashes, int* pages, int cap, uint64_t* page_hash) {
    Group& g = static_cast<Cache*>(h)->groups[group];
    int i = 0;
    for (const auto& kv : g.by_hash) {
        if (i < cap && hashes && pages) {
            hashes[i] = kv.first;
            pages[i] = kv.second;
        }
        ++i;
    }
    if (page_hash) std::memcpy(page_hash, g.page_hash.data(), sizeof(uint64_t) * g.page_hash.size());
    return i;
}

// The ids of the requests of a group's tables (which < 0: of the request map); returns the count.
GBH_EXPORT int gbh_cache_ids(void* h, int group, int64_t* out, int cap) {
    Cache* c = static_cast<Cache*>(h);
    int i = 0;
    if (group < 0) {
        for (const auto& kv : c->requests) {
            if (i < cap && out) out[i] = kv.first;
            ++i;
        }
    } else {
        for (const auto& kv : c->groups[group].tables) {
            if (i < cap && out) out[i] = kv.first;
            ++i;
        }
    }
    return i;
}

// ------------------------------------------------------------------------------ a scheduler step's plan
// What one step of continuous batching computes, and with which pages (the policy of
// crates/glassbox-server/src/scheduler.rs:283-330). The running requests are given in admission order with the
// number of tokens each still has to run. Requests with one token left (decoding) come first, then the others
// (prompt portions), each taking what is left of the token budget. Room is then reserved entry by entry; when the
// pages run out, the most recently admitted request is preempted (everything it holds is given back, its plan
// entry dropped) and the entry tried again; a lone request that does not fit is reported instead.
// Out: plan_idx / plan_n (index into the running list, tokens), *n_plan; copies (group, source page, destination
// page triples of copy-on-write work, at most one per group and entry), *n_copies; *n_preempted (the last that
// many running requests, latest first); *lone_failed.
GBH_EXPORT int gbh_plan_step(void* h, int n_running, const int64_t* rids, const int* remaining, int budget, int* plan_idx,
                             int* plan_n, int* n_plan, int* copies, int* n_copies, int* n_preempted, int* lone_failed) {
    Cache* c = static_cast<Cache*>(h);
    std::vector<std::pair<int, int>> plan;
    for (int pass = 0; pass < 2 && budget > 0; ++pass)
        for (int i = 0; i < n_running && budget > 0; ++i) {
            if ((remaining[i] > 1) != (pass == 1)) continue;
            const int n = std::min(remaining[i], budget);
            plan.emplace_back(i, n);
            budget -= n;
        }
    int live = n_running, pre = 0;
    *lone_failed = 0;
    size_t k = 0;
    std::vector<int> one(3 * std::max<size_t>(c->groups.size(), 1));
    std::vector<std::vector<int>> work(plan.size());   // copy-on-write triples of each reserved plan entry
    while (k < plan.size()) {
        int got = 0;
        const int code = gbh_cache_reserve(h, rids[plan[k].first], plan[k].second, one.data(), &got);
        if (code == OK) {
            work[k].assign(one.begin(), one.begin() + 3 * got);
            ++k;
            continue;
        }
        if (code != OUT_OF_PAGES) return code;
        if (live == 1) {
            *lone_failed = 1;
            plan.clear();
            work.clear();
            break;
        }
        const int victim = --live;
        gbh_cache_free(h, rids[victim]);
        ++pre;
        for (size_t p = 0; p < plan.size(); ++p)
            if (plan[p].first == victim) {
                // Its destination pages went back to the pool with everything else it held and may be handed
                // out again in this very plan: its copies must not run.
                plan.erase(plan.begin() + p);
                work.erase(work.begin() + p);
                if (p < k) --k;
                break;
            }
    }
    int nc = 0;
    for (size_t p = 0; p < plan.size(); ++p) {
        plan_idx[p] = plan[p].first;
        plan_n[p] = plan[p].second;
        std::memcpy(copies + 3 * nc, work[p].data(), sizeof(int) * work[p].size());
        nc += (int)work[p].size() / 3;
    }
    *n_plan = (int)plan.size();
    *n_copies = nc;
    *n_preempted = pre;
    return OK;
}

// A step in which every running request decodes one token, planned in one call: the requests must all have room below
// `max_position` (else BAD_VALUE: the caller's general path ends the request that has none), a slot for one more token
// is reserved for each, all or nothing (else OUT_OF_PAGES and nothing is held that was not held before: the caller's
// general path decides whom to preempt). Out: copy-on-write triples, and the widest block table among the requests.
GBH_EXPORT int gbh_decode_plan(void* h, int n, const int64_t* rids, int max_position, int* copies, int* n_copies, int* max_pages) {
    Cache* c = static_cast<Cache*>(h);
    for (int e = 0; e < n; ++e) {
        Request* req = find(c, rids[e]);
        if (!req) return fail(UNKNOWN_REQUEST, "unknown request");
        if (req->length + 1 > max_position) return fail(BAD_VALUE, "a request has reached max_position");
    }
    std::vector<int> one(3 * std::max<size_t>(c->groups.size(), 1));
    int nc = 0;
    for (int e = 0; e < n; ++e) {
        int got = 0;
        const int code = gbh_cache_reserve(h, rids[e], 1, one.data(), &got);
        if (code != OK) {
            for (int k = 0; k < e; ++k) gbh_cache_truncate(h, rids[k], find(c, rids[k])->length);   // give the new pages back
            return code;
        }
        std::memcpy(copies + 3 * nc, one.data(), sizeof(int) * 3 * got);
        nc += got;
    }
    int widest = 1;
    for (const Group& g : c->groups)
        for (int e = 0; e < n; ++e) widest = std::max(widest, (int)g.tables.find(rids[e])->second.size());
    *n_copies = nc;
    *max_pages = widest;
    return OK;
}

// ------------------------------------------------------------------------------ a step's metadata
// Fills the int32 block that a step copies to the device. Its sections start at the offsets given:
//   off[0..8]: tokens [n], positions [n], row_seq [n], want [n_want], seq_first_row [S+1], seq_start_pos [S],
//   seq_slots [S], want_slots [n_want], token_slots [n]; then per group g: off[9+2g] slots [n], off[10+2g] tables
//   [S, max_pages].
// want_slots names, for each wanted row that is to be sampled from its request's own sampling state (sample_mask,
// one byte per wanted row of the entries, or null: none), the request's state slot, and -1 for every other wanted row.
// token_slots names, for the one row of each entry whose byte in feedback_mask is set, the request's state slot (the
// device puts the token it sampled for the request in the step before into that row), and -1 for every other row.
// The E entries bring tok_count[e] tokens each (flat in tokens) and ask for want_count[e] of their rows
// (indices within the entry, flat in want). The step has a fixed shape of S >= E sequences and n rows:
// pad_after padding sequences follow the first `lead` entries (so that a batch whose leading single-token
// requests are counted in round numbers keeps its shape while their number changes), the rest follow the last
// entry; a padding sequence has one padding row. Padding rows, the rows behind the last sequence and the
// padding sequences get position -1 (the sequences: start position -1), slot -1 and empty tables: every kernel
// skips them. The wanted rows of the
// entries come first, in entry order; the remaining want slots name padding rows (row 0 when there are none
// left), whose logits nobody reads. seq_info receives (start position, slot, first row) per entry, *max_ctx
// the longest context of the step.
GBH_EXPORT int gbh_fill_step(void* h, int E, const int64_t* rids, const int* tok_count, const int32_t* tokens,
                             const int* want_count, const int* want, int lead, int pad_after, int n, int S, int n_want,
                             int max_pages, const long long* off, long long size, int32_t* host,
                             const unsigned char* sample_mask, int n_mask, const unsigned char* feedback_mask,
                             int* seq_info, int* max_ctx) {
    Cache* c = static_cast<Cache*>(h);
    const int G = (int)c->groups.size();
    if (S < E + pad_after || lead < 0 || lead > E || pad_after < 0) return fail(BAD_VALUE, "fewer sequences than entries");
    long long rows = 0, wanted = 0;
    for (int e = 0; e < E; ++e) {
        rows += tok_count[e];
        wanted += want_count[e];
    }
    if (rows + (S - E) > n || wanted > n_want) return fail(BAD_VALUE, "the entries do not fit the step's shape");
    std::memset(host, 0, sizeof(int32_t) * (size_t)size);
    int32_t* h_tokens = host + off[0];
    int32_t* h_pos = host + off[1];
    int32_t* h_row_seq = host + off[2];
    int32_t* h_want = host + off[3];
    int32_t* h_first = host + off[4];
    int32_t* h_start = host + off[5];
    int32_t* h_slots = host + off[6];
    int32_t* h_want_slots = host + off[7];
    int32_t* h_token_slots = host + off[8];
    std::fill(h_pos, h_pos + n, -1);
    std::fill(h_want_slots, h_want_slots + n_want, -1);
    std::fill(h_token_slots, h_token_slots + n, -1);
    for (int g = 0; g < G; ++g) {
        std::fill(host + off[9 + 2 * g], host + off[9 + 2 * g] + n, -1);
        std::fill(host + off[10 + 2 * g], host + off[10 + 2 * g] + (long long)S * max_pages, -1);
    }
    std::vector<int> pad_rows;
    int row = 0, wi = 0, longest = 0, tcur = 0, wcur = 0, seq = 0;
    auto pad_seq = [&]() {   // a padding sequence: one padding row, start position -1
        h_row_seq[row] = seq;
        h_first[seq] = row;
        h_start[seq] = -1;
        pad_rows.push_back(row);
        ++row;
        ++seq;
    };
    for (int e = 0; e < E; ++e) {
        if (e == lead)
            for (int p = 0; p < pad_after; ++p) pad_seq();
        Request* req = find(c, rids[e]);
        if (!req) return fail(UNKNOWN_REQUEST, "unknown request");
        const int k = tok_count[e], start = req->length;
        seq_info[3 * e] = start;
        seq_info[3 * e + 1] = req->slot;
        seq_info[3 * e + 2] = row;
        for (int i = 0; i < k; ++i) {
            h_tokens[row + i] = tokens[tcur + i];
            h_pos[row + i] = start + i;
            h_row_seq[row + i] = seq;
        }
        for (int i = 0; i < want_count[e]; ++i) {
            if (sample_mask && wi < n_mask && sample_mask[wi]) h_want_slots[wi] = req->slot;
            h_want[wi++] = row + want[wcur + i];
        }
        h_first[seq] = row;
        h_start[seq] = start;
        h_slots[seq] = req->slot;
        if (feedback_mask && feedback_mask[e] && k == 1) h_token_slots[row] = req->slot;
        for (int g = 0; g < G; ++g) {
            const Group& gr = c->groups[g];
            const std::vector<int>& table = gr.tables.find(rids[e])->second;
            if ((int)table.size() > max_pages) return fail(BAD_VALUE, "a block table is wider than the step's tables");
            if ((start + k + gr.page_size - 1) / gr.page_size > (int)table.size())
                return fail(BAD_VALUE, "a request brings tokens for which no page was reserved");
            std::memcpy(host + off[10 + 2 * g] + (long long)seq * max_pages, table.data(), sizeof(int) * table.size());
            int32_t* sl = host + off[9 + 2 * g] + row;
            for (int i = 0; i < k; ++i) {
                const int pos = start + i;
                sl[i] = table[pos / gr.page_size] * gr.page_size + pos % gr.page_size;
            }
        }
        row += k;
        tcur += k;
        wcur += want_count[e];
        longest = std::max(longest, start + k);
        ++seq;
    }
    if (lead == E)
        for (int p = 0; p < pad_after; ++p) pad_seq();
    while (seq < S) pad_seq();
    h_first[S] = row;
    for (int r = row; r < n; ++r) h_row_seq[r] = S - 1;   // rows behind the last sequence: skipped by their position
    for (size_t p = 0; wi < n_want; ++p) h_want[wi++] = p < pad_rows.size() ? pad_rows[p] : 0;
    *max_ctx = longest;
    return OK;
}
