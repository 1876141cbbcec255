// Host-side bookkeeping of the paged key/value cache, and the flattening of a step's description: plain C++
// behind a C interface (no CUDA, no Python headers), loaded by cache/pages.py and engine/engine.py through ctypes.
//
// The reference gives every sequence one contiguous K and V buffer of the whole context (src/model.c:3089-3101);
// "which rows are valid" is the sequence's position (src/engine.h:40).  Here a request holds fixed-size pages.
// Layers are collected in groups by what they keep: all keys (window < 0) or the last `window` keys (the
// reference's per-layer sliding flag, src/model.h:229-235).  Every group has a pool of pages of its own and every
// request slot a row of page numbers per group (the block table, -1 where no page is held).  Pages go back to
// their pool when a request ends and, in a window group, as soon as every position in the page lies behind the
// window of every query still to come.  The block tables live in memory that the caller owns (numpy arrays), so
// that the engine copies rows of them into the step description without asking this library.
//
// A request is known here by its slot.  Return codes: XRH_OK, or one of the errors below; nothing is changed
// by a call that returns an error, except where a comment says otherwise.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#define XRH_EXPORT extern "C" __attribute__((visibility("default")))

enum { XRH_OK = 0, XRH_OUT_OF_PAGES = 1, XRH_TOO_LONG = 2, XRH_NO_SLOT = 3, XRH_BAD_ARG = -1, XRH_NOT_OPEN = -2, XRH_NOT_HELD = -3 };

namespace {

struct Pool {
    int n_pages = 0;
    std::vector<int> free_;           // a stack; page 0 is handed out first
    std::vector<uint8_t> held;
    explicit Pool(int n) : n_pages(n), held((size_t)n, 0) {
        free_.reserve((size_t)n);
        for (int p = n - 1; p >= 0; p--) free_.push_back(p);
    }
    int n_free() const { return (int)free_.size(); }
    int take() {
        if (free_.empty()) return -1;
        int p = free_.back();
        free_.pop_back();
        held[(size_t)p] = 1;
        return p;
    }
    bool give(int p) {
        if (p < 0 || p >= n_pages || !held[(size_t)p]) return false;
        held[(size_t)p] = 0;
        free_.push_back(p);
        return true;
    }
};

struct Request {
    bool open = false;
    long long length = 0;             // tokens whose keys are in the cache
    long long reserved = 0;           // tokens reserved beyond `length` for the step in flight
    std::vector<int> first_live;      // per group: table entries below this were released
};

struct Cache {
    int groups, page_size, max_requests, max_pages;
    std::vector<int> window;          // per group, < 0: every key is kept
    std::vector<Pool> pools;
    std::vector<int32_t*> tables;     // per group [max_requests][max_pages], owned by the caller
    std::vector<Request> reqs;
    std::vector<int> free_slots;
    std::vector<int> high_water;

    int32_t* row(int g, int slot) { return tables[(size_t)g] + (size_t)slot * (size_t)max_pages; }
    long long ceil_pages(long long tokens) const { return (tokens + page_size - 1) / page_size; }
    // lowest page index that a query at `query_pos` (or any later one) can read in group g
    long long first_needed_page(int g, long long query_pos) const {
        int w = window[(size_t)g];
        if (w < 0) return 0;
        long long first_key = query_pos - w + 1;
        if (first_key < 0) first_key = 0;
        return first_key / page_size;
    }
    Request* req(int slot) {
        if (slot < 0 || slot >= max_requests || !reqs[(size_t)slot].open) return nullptr;
        return &reqs[(size_t)slot];
    }
    // pages per group that reserving n_new more tokens would take, after releasing what the window has passed
    void pages_needed(const Request& r, long long n_new, int* out) const {
        long long start = r.length + r.reserved, end = start + n_new;
        for (int g = 0; g < groups; g++) {
            long long have_upto = ceil_pages(start), want_upto = ceil_pages(end);
            long long first = first_needed_page(g, start);
            if (r.first_live[(size_t)g] > first) first = r.first_live[(size_t)g];
            long long lo = have_upto > first ? have_upto : first;
            out[g] = (int)(want_upto > lo ? want_upto - lo : 0);
        }
    }
    // pages that the window lets go before a query at the request's next position
    long long releasable(const Request& r, int g) const {
        long long pos = r.length + r.reserved;
        long long first = first_needed_page(g, pos), held_upto = ceil_pages(pos);
        long long upto = first < held_upto ? first : held_upto;
        long long n = upto - r.first_live[(size_t)g];
        return n > 0 ? n : 0;
    }
    bool can_reserve(const Request& r, long long n_new) const {
        if (r.length + r.reserved + n_new > (long long)max_pages * page_size) return false;
        std::vector<int> need((size_t)groups);
        pages_needed(r, n_new, need.data());
        for (int g = 0; g < groups; g++)
            if (need[(size_t)g] > pools[(size_t)g].n_free() + releasable(r, g)) return false;
        return true;
    }
    int release_behind_window(Request& r, int slot) {
        int n = 0;
        long long pos = r.length + r.reserved;
        for (int g = 0; g < groups; g++) {
            long long first = first_needed_page(g, pos), held_upto = ceil_pages(pos);
            if (held_upto < first) first = held_upto;
            int32_t* tab = row(g, slot);
            for (long long i = r.first_live[(size_t)g]; i < first; i++)
                if (tab[i] >= 0) {
                    pools[(size_t)g].give(tab[i]);
                    tab[i] = -1;
                    n++;
                }
            if (first > r.first_live[(size_t)g]) r.first_live[(size_t)g] = (int)first;
        }
        return n;
    }
};

}  // namespace

// ---- a pool on its own ------------------------------------------------------------------------------------
XRH_EXPORT void* xrh_pool_create(int n_pages) { return n_pages < 1 ? nullptr : new (std::nothrow) Pool(n_pages); }
XRH_EXPORT void xrh_pool_destroy(void* p) { delete (Pool*)p; }
XRH_EXPORT int xrh_pool_n_free(void* p) { return ((Pool*)p)->n_free(); }
XRH_EXPORT int xrh_pool_take(void* p) { return ((Pool*)p)->take(); }                           // -1: empty
XRH_EXPORT int xrh_pool_give(void* p, int page) { return ((Pool*)p)->give(page) ? XRH_OK : XRH_NOT_HELD; }

// ---- the cache manager -------------------------------------------------------------------------------------
// windows[g] < 0: group g keeps every key.  tables[g]: int32 [max_requests][max_pages], filled with -1 here.
XRH_EXPORT void* xrh_cache_create(int groups, const int* windows, int n_pages, int page_size, int max_requests, int max_pages,
                                  int32_t** tables) {
    if (groups < 0 || n_pages < 1 || page_size < 1 || max_requests < 1 || max_pages < 1) return nullptr;
    Cache* c = new (std::nothrow) Cache();
    if (!c) return nullptr;
    c->groups = groups; c->page_size = page_size; c->max_requests = max_requests; c->max_pages = max_pages;
    for (int g = 0; g < groups; g++) {
        c->window.push_back(windows[g]);
        c->pools.emplace_back(n_pages);
        c->tables.push_back(tables[g]);
        c->high_water.push_back(0);
        for (size_t i = 0; i < (size_t)max_requests * (size_t)max_pages; i++) tables[g][i] = -1;
    }
    c->reqs.resize((size_t)max_requests);
    for (int s = max_requests - 1; s >= 0; s--) c->free_slots.push_back(s);      // slot 0 is handed out first
    return c;
}
XRH_EXPORT void xrh_cache_destroy(void* h) { delete (Cache*)h; }

XRH_EXPORT int xrh_has_free_slot(void* h) { return ((Cache*)h)->free_slots.empty() ? 0 : 1; }
XRH_EXPORT int xrh_n_free(void* h, int g) { return ((Cache*)h)->pools[(size_t)g].n_free(); }
XRH_EXPORT int xrh_high_water(void* h, int g) { return ((Cache*)h)->high_water[(size_t)g]; }
XRH_EXPORT int xrh_pool_take_of(void* h, int g) { return ((Cache*)h)->pools[(size_t)g].take(); }
XRH_EXPORT int xrh_pool_give_of(void* h, int g, int page) { return ((Cache*)h)->pools[(size_t)g].give(page) ? XRH_OK : XRH_NOT_HELD; }

// A slot for a new request, or -1 when none is free.
XRH_EXPORT int xrh_open(void* h) {
    Cache* c = (Cache*)h;
    if (c->free_slots.empty()) return -1;
    int slot = c->free_slots.back();
    c->free_slots.pop_back();
    Request& r = c->reqs[(size_t)slot];
    r.open = true; r.length = 0; r.reserved = 0;
    r.first_live.assign((size_t)c->groups, 0);
    return slot;
}

// The request ended: all its pages and its slot go back.
XRH_EXPORT int xrh_close(void* h, int slot) {
    Cache* c = (Cache*)h;
    Request* r = c->req(slot);
    if (!r) return XRH_NOT_OPEN;
    long long upto = c->ceil_pages(r->length + r->reserved);
    for (int g = 0; g < c->groups; g++) {
        int32_t* tab = c->row(g, slot);
        for (long long i = r->first_live[(size_t)g]; i < upto; i++)
            if (tab[i] >= 0) c->pools[(size_t)g].give(tab[i]);
        for (int i = 0; i < c->max_pages; i++) tab[i] = -1;
    }
    r->open = false;
    c->free_slots.push_back(slot);
    return XRH_OK;
}

XRH_EXPORT long long xrh_length(void* h, int slot) { Request* r = ((Cache*)h)->req(slot); return r ? r->length : -1; }
XRH_EXPORT long long xrh_reserved(void* h, int slot) { Request* r = ((Cache*)h)->req(slot); return r ? r->reserved : -1; }

XRH_EXPORT int xrh_pages_needed(void* h, int slot, long long n_new, int* out) {
    Cache* c = (Cache*)h;
    Request* r = c->req(slot);
    if (!r) return XRH_NOT_OPEN;
    c->pages_needed(*r, n_new, out);
    return XRH_OK;
}

XRH_EXPORT int xrh_can_reserve(void* h, int slot, long long n_new) {
    Cache* c = (Cache*)h;
    Request* r = c->req(slot);
    return r && c->can_reserve(*r, n_new) ? 1 : 0;
}

// Take the pages that the request's next n_new tokens need, in every group, or none.
XRH_EXPORT int xrh_reserve(void* h, int slot, long long n_new) {
    Cache* c = (Cache*)h;
    Request* r = c->req(slot);
    if (!r) return XRH_NOT_OPEN;
    if (n_new < 1) return XRH_BAD_ARG;
    long long start = r->length + r->reserved;
    if (start + n_new > (long long)c->max_pages * c->page_size) return XRH_TOO_LONG;
    if (!c->can_reserve(*r, n_new)) return XRH_OUT_OF_PAGES;
    c->release_behind_window(*r, slot);
    long long end = start + n_new;
    for (int g = 0; g < c->groups; g++) {
        long long have_upto = c->ceil_pages(start), want_upto = c->ceil_pages(end);
        long long lo = have_upto > r->first_live[(size_t)g] ? have_upto : r->first_live[(size_t)g];
        int32_t* tab = c->row(g, slot);
        Pool& pool = c->pools[(size_t)g];
        for (long long i = lo; i < want_upto; i++) tab[i] = pool.take();
        int used = pool.n_pages - pool.n_free();
        if (used > c->high_water[(size_t)g]) c->high_water[(size_t)g] = used;
    }
    r->reserved += n_new;
    return XRH_OK;
}

// The step ran: reserved tokens now count as held.
XRH_EXPORT int xrh_commit(void* h, int slot) {
    Request* r = ((Cache*)h)->req(slot);
    if (!r) return XRH_NOT_OPEN;
    r->length += r->reserved;
    r->reserved = 0;
    return XRH_OK;
}

// The planned step did not run: give back pages that only the reservation needed.
XRH_EXPORT int xrh_cancel(void* h, int slot) {
    Cache* c = (Cache*)h;
    Request* r = c->req(slot);
    if (!r) return XRH_NOT_OPEN;
    if (r->reserved == 0) return XRH_OK;
    long long keep_upto = c->ceil_pages(r->length), had_upto = c->ceil_pages(r->length + r->reserved);
    for (int g = 0; g < c->groups; g++) {
        int32_t* tab = c->row(g, slot);
        long long lo = keep_upto > r->first_live[(size_t)g] ? keep_upto : r->first_live[(size_t)g];
        for (long long i = lo; i < had_upto; i++)
            if (tab[i] >= 0) {
                c->pools[(size_t)g].give(tab[i]);
                tab[i] = -1;
            }
    }
    r->reserved = 0;
    return XRH_OK;
}

// Give back the pages no query from the request's next position on can read.  Returns how many (or an error < 0).
XRH_EXPORT int xrh_release_behind_window(void* h, int slot) {
    Cache* c = (Cache*)h;
    Request* r = c->req(slot);
    if (!r) return XRH_NOT_OPEN;
    return c->release_behind_window(*r, slot);
}

// 0 if no page is lost, held twice or free twice and every table agrees with its request's length; else 1 and
// what is wrong in msg.
XRH_EXPORT int xrh_audit(void* h, char* msg, int cap) {
    Cache* c = (Cache*)h;
#define FAIL(...) do { snprintf(msg, (size_t)cap, __VA_ARGS__); return 1; } while (0)
    for (int g = 0; g < c->groups; g++) {
        Pool& pool = c->pools[(size_t)g];
        std::vector<int> seen((size_t)pool.n_pages, 0), fr((size_t)pool.n_pages, 0);
        for (int s = 0; s < c->max_requests; s++) {
            const Request& r = c->reqs[(size_t)s];
            int32_t* tab = c->row(g, s);
            if (!r.open) {
                for (int i = 0; i < c->max_pages; i++)
                    if (tab[i] >= 0) FAIL("group %d slot %d: a page at index %d of a slot that no request holds", g, s, i);
                continue;
            }
            long long upto = c->ceil_pages(r.length + r.reserved);
            for (int i = 0; i < c->max_pages; i++) {
                bool live = r.first_live[(size_t)g] <= i && i < upto;
                if (tab[i] >= 0) {
                    if (!live) FAIL("group %d slot %d: page at index %d outside its live range", g, s, i);
                    if (tab[i] >= pool.n_pages) FAIL("group %d slot %d: page number at index %d is outside the pool", g, s, i);
                    seen[(size_t)tab[i]]++;
                } else if (live) {
                    FAIL("group %d slot %d: hole at index %d", g, s, i);
                }
            }
        }
        for (int p : pool.free_) fr[(size_t)p]++;
        for (int p = 0; p < pool.n_pages; p++) {
            if (seen[(size_t)p] > 1) FAIL("group %d: page %d is in two tables", g, p);
            if (fr[(size_t)p] > 1) FAIL("group %d: page %d is free twice", g, p);
            if (seen[(size_t)p] + fr[(size_t)p] == 0) FAIL("group %d: page %d is lost", g, p);
            if (seen[(size_t)p] + fr[(size_t)p] > 1) FAIL("group %d: page %d is both free and held", g, p);
            if ((pool.held[(size_t)p] != 0) != (seen[(size_t)p] == 1)) FAIL("group %d: held flag of page %d disagrees with the tables", g, p);
        }
    }
    std::vector<int> used((size_t)c->max_requests, 0);
    int open = 0;
    for (int s = 0; s < c->max_requests; s++)
        if (c->reqs[(size_t)s].open) { used[(size_t)s]++; open++; }
    for (int s : c->free_slots) {
        if (s < 0 || s >= c->max_requests || used[(size_t)s]) FAIL("request slot %d is used twice", s);
        used[(size_t)s]++;
    }
    if (open + (int)c->free_slots.size() != c->max_requests) FAIL("a request slot is lost");
    return 0;
#undef FAIL
}

// ---- the step description -----------------------------------------------------------------------------------
// Flattens a batch of (request slot, its next tokens, wanted places) into the arrays that the kernels read:
// per token its id, position and segment; the rows whose logits are wanted; per segment its first row, length,
// first position and slot; per group the block-table rows of the segments.  `fill` more segments of one token
// at position 0 are appended, whose block-table rows hold `filler_page` at index 0 and -1 elsewhere (rows that
// bring a decode step to a size that repeats; every one of them is "wanted").  Positions come from the
// requests' lengths.  Returns the longest context (position + 1) among the real segments, or an error < 0.
XRH_EXPORT long long xrh_describe(void* h, int n_seg, const int* slots, const int* counts, const int* tokens, const int* want_counts,
                                  const int* wants, int fill, int filler_page, int32_t* tok, int32_t* pos, int32_t* seg, int32_t* rows,
                                  int32_t* s_start, int32_t* s_len, int32_t* s_pos0, int32_t* s_slot, int32_t** block_tables) {
    Cache* c = (Cache*)h;
    long long at = 0, ri = 0, wi = 0, max_kv = 0;
    for (int si = 0; si < n_seg; si++) {
        Request* r = c->req(slots[si]);
        if (!r) return XRH_NOT_OPEN;
        const int m = counts[si];
        const long long p0 = r->length;
        for (int j = 0; j < m; j++) {
            tok[at + j] = tokens[at + j];
            pos[at + j] = (int32_t)(p0 + j);
            seg[at + j] = si;
        }
        for (int j = 0; j < want_counts[si]; j++) rows[ri++] = (int32_t)(at + wants[wi++]);
        s_start[si] = (int32_t)at; s_len[si] = m; s_pos0[si] = (int32_t)p0; s_slot[si] = slots[si];
        if (p0 + m > max_kv) max_kv = p0 + m;
        at += m;
    }
    for (int si = n_seg; si < n_seg + fill; si++) {
        tok[at] = 0; pos[at] = 0; seg[at] = si; rows[ri++] = (int32_t)at;
        s_start[si] = (int32_t)at; s_len[si] = 1; s_pos0[si] = 0; s_slot[si] = n_seg > 0 ? slots[0] : 0;
        at++;
    }
    const size_t mp = (size_t)c->max_pages;
    for (int g = 0; g < c->groups; g++) {
        int32_t* bt = block_tables[g];
        for (int si = 0; si < n_seg; si++) memcpy(bt + (size_t)si * mp, c->row(g, slots[si]), mp * sizeof(int32_t));
        for (int si = n_seg; si < n_seg + fill; si++) {
            int32_t* row = bt + (size_t)si * mp;
            for (size_t i = 0; i < mp; i++) row[i] = -1;
            row[0] = filler_page;
        }
    }
    return max_kv;
}
