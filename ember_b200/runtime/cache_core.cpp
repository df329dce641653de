// Host-side bookkeeping of the paged cache, natively: page pools, block tables per request and group,
// window release, state slots, the audit.  No device memory is touched here; the ids it hands out index the
// tensors that ember_b200/cache/storage.py allocates.  ember_b200/cache/manager.py is the Python face.
// (The reference keeps the same books in C++ too: src/kvcache/block_manager.{hpp,cpp}; groups, windows and
// slots have no counterpart there.)
//
// Pages: ids 0..n-1; a fresh pool hands out low ids first, afterwards the most recently freed page first.
// Groups: kind 0 keeps all keys, kind 1 a window of them (pages wholly older than the window go back as soon
// as no later query can see them), kind 2 is fixed-size state (no pages).  Every admitted request holds one
// slot and one block table per group (-1 = page given back).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Pool {
    int n = 0;
    std::vector<int32_t> free_;
    std::vector<uint8_t> held;
    void init(int pages) {
        n = pages;
        free_.resize(pages);
        for (int i = 0; i < pages; i++) free_[i] = pages - 1 - i;      // pop from the back: 0, 1, 2, ...
        held.assign(pages, 0);
    }
    int allocate() {
        if (free_.empty()) return -1;
        const int p = free_.back();
        free_.pop_back();
        held[p] = 1;
        return p;
    }
    int release(int p) {                 // 0 ok, 1 outside the pool, 2 freed twice
        if (p < 0 || p >= n) return 1;
        if (!held[p]) return 2;
        held[p] = 0;
        free_.push_back(p);
        return 0;
    }
    std::string check() const {
        std::vector<uint8_t> seen(n, 0);
        char buf[128];
        for (int p : free_) {
            if (seen[p]) { snprintf(buf, sizeof buf, "page %d is on the free list twice", p); return buf; }
            seen[p] = 1;
            if (held[p]) { snprintf(buf, sizeof buf, "page %d is both free and held", p); return buf; }
        }
        int h = 0;
        for (int p = 0; p < n; p++) h += held[p];
        if (h + (int)free_.size() != n) {
            snprintf(buf, sizeof buf, "%d held + %d free != %d pages (a page is lost)", h, (int)free_.size(), n);
            return buf;
        }
        return "";
    }
};

struct Group {
    int kind = 0, window = 0;
    Pool pool;
    bool paged() const { return kind != 2; }
};

struct Request {
    bool live = false;
    int slot = -1;
    long long tokens = 0;
    std::vector<std::vector<int32_t>> tables;
    std::vector<int> first_live;
};

struct Core {
    int page = 16, max_requests = 0;
    std::vector<Group> groups;
    std::vector<int> free_slots;
    std::vector<Request> reqs;       // indexed by handle
    std::vector<int> free_handles;
    std::string message;
};

Request* get(Core* c, int h) {
    if (h < 0 || h >= (int)c->reqs.size() || !c->reqs[h].live) return nullptr;
    return &c->reqs[h];
}

void give_back(Core* c, Request& r) {    // pages in reverse order, as they were taken
    for (size_t g = 0; g < c->groups.size(); g++) {
        if (!c->groups[g].paged()) continue;
        auto& t = r.tables[g];
        for (size_t i = t.size(); i-- > 0;)
            if (t[i] >= 0) c->groups[g].pool.release(t[i]);
    }
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------- a pool alone
void* ember_pool_create(int pages) {
    if (pages < 0) return nullptr;
    Pool* p = new Pool();
    p->init(pages);
    return p;
}
void ember_pool_destroy(void* p) { delete (Pool*)p; }
int ember_pool_allocate(void* p) { return ((Pool*)p)->allocate(); }
int ember_pool_release(void* p, int page) { return ((Pool*)p)->release(page); }
int ember_pool_available(void* p) { return (int)((Pool*)p)->free_.size(); }
int ember_pool_is_held(void* p, int page) { Pool* q = (Pool*)p; return page >= 0 && page < q->n ? q->held[page] : 0; }
int ember_pool_check(void* p, char* msg, int cap) {
    const std::string s = ((Pool*)p)->check();
    snprintf(msg, cap, "%s", s.c_str());
    return s.empty() ? 0 : 1;
}

// --------------------------------------------------------------------------------- the manager
void* ember_cache_create(int n_groups, const int32_t* kinds, const int32_t* windows, const int32_t* pages,
                         int page_tokens, int max_requests) {
    if (n_groups < 0 || page_tokens <= 0 || max_requests < 0) return nullptr;
    Core* c = new Core();
    c->page = page_tokens;
    c->max_requests = max_requests;
    c->groups.resize(n_groups);
    for (int g = 0; g < n_groups; g++) {
        c->groups[g].kind = kinds[g];
        c->groups[g].window = windows[g];
        c->groups[g].pool.init(kinds[g] == 2 ? 0 : (pages[g] < 0 ? 0 : pages[g]));
    }
    for (int s = max_requests - 1; s >= 0; s--) c->free_slots.push_back(s);   // pop from the back: 0, 1, ...
    return c;
}
void ember_cache_destroy(void* c) { delete (Core*)c; }

// The pool of group g (for the queries above); null for a state group.
void* ember_cache_pool(void* cv, int g) {
    Core* c = (Core*)cv;
    return c->groups[g].paged() ? &c->groups[g].pool : nullptr;
}

// A slot and empty block tables; returns the request's handle, or -1 if no slot is free.
int ember_cache_admit(void* cv) {
    Core* c = (Core*)cv;
    if (c->free_slots.empty()) return -1;
    int h;
    if (!c->free_handles.empty()) {
        h = c->free_handles.back();
        c->free_handles.pop_back();
    } else {
        h = (int)c->reqs.size();
        c->reqs.emplace_back();
    }
    Request& r = c->reqs[h];
    r.live = true;
    r.slot = c->free_slots.back();
    c->free_slots.pop_back();
    r.tokens = 0;
    r.tables.assign(c->groups.size(), {});
    r.first_live.assign(c->groups.size(), 0);
    return h;
}

int ember_cache_slot(void* cv, int h) { Request* r = get((Core*)cv, h); return r ? r->slot : -1; }
long long ember_cache_tokens(void* cv, int h) { Request* r = get((Core*)cv, h); return r ? r->tokens : -1; }
int ember_cache_first_live(void* cv, int h, int g) { Request* r = get((Core*)cv, h); return r ? r->first_live[g] : -1; }

// The block table of (request, group): its length, and through `ptr` its entries (valid until the table grows).
int ember_cache_table(void* cv, int h, int g, const int32_t** ptr) {
    Request* r = get((Core*)cv, h);
    if (!r) return -1;
    if (ptr) *ptr = r->tables[g].data();
    return (int)r->tables[g].size();
}

// Pages for tokens [0, upto) in every paged group: all or nothing.  1 taken (or already there), 0 no room,
// -1 unknown request.
int ember_cache_ensure(void* cv, int h, long long upto) {
    Core* c = (Core*)cv;
    Request* r = get(c, h);
    if (!r) return -1;
    const long long want = (upto + c->page - 1) / c->page;
    for (size_t g = 0; g < c->groups.size(); g++) {
        if (!c->groups[g].paged()) continue;
        const long long need = want - (long long)r->tables[g].size();
        if (need > (long long)c->groups[g].pool.free_.size()) return 0;
    }
    for (size_t g = 0; g < c->groups.size(); g++) {
        if (!c->groups[g].paged()) continue;
        while ((long long)r->tables[g].size() < want) r->tables[g].push_back(c->groups[g].pool.allocate());
    }
    return 1;
}

// `tokens` tokens are now cached; window pages no later query can see go back.  Returns how many were freed.
int ember_cache_advance(void* cv, int h, long long tokens) {
    Core* c = (Core*)cv;
    Request* r = get(c, h);
    if (!r) return -1;
    r->tokens = tokens;
    int freed = 0;
    for (size_t g = 0; g < c->groups.size(); g++) {
        Group& grp = c->groups[g];
        if (grp.kind != 1) continue;
        // the next query is at position >= tokens and sees keys > position - window
        long long first_key = tokens - grp.window + 1;
        if (first_key < 0) first_key = 0;
        const long long dead = first_key / c->page;
        auto& t = r->tables[g];
        const long long stop = dead < (long long)t.size() ? dead : (long long)t.size();
        for (long long i = r->first_live[g]; i < stop; i++) {
            if (t[i] >= 0) {
                grp.pool.release(t[i]);
                t[i] = -1;
                freed++;
            }
        }
        if (stop > r->first_live[g]) r->first_live[g] = (int)stop;
    }
    return freed;
}

// Everything the request holds goes back (pages in reverse order, then its slot).  0 ok, -1 unknown request.
int ember_cache_release(void* cv, int h) {
    Core* c = (Core*)cv;
    Request* r = get(c, h);
    if (!r) return -1;
    give_back(c, *r);
    c->free_slots.push_back(r->slot);
    r->live = false;
    r->tables.clear();
    c->free_handles.push_back(h);
    return 0;
}

// Preemption: the pages go back, the slot stays.
int ember_cache_reset(void* cv, int h) {
    Core* c = (Core*)cv;
    Request* r = get(c, h);
    if (!r) return -1;
    give_back(c, *r);
    for (size_t g = 0; g < c->groups.size(); g++) {
        r->tables[g].clear();
        r->first_live[g] = 0;
    }
    r->tokens = 0;
    return 0;
}

int ember_cache_free_slots(void* cv) { return (int)((Core*)cv)->free_slots.size(); }

// What a step needs of n requests at once: cached tokens, slot, and per group the table's address and length
// (tables[g * n + i], lens[g * n + i]).  Returns the index of the first unknown request, or -1 if all are live.
int ember_cache_describe(void* cv, int n, const int32_t* handles, int64_t* tokens, int32_t* slots, uint64_t* tables,
                         int32_t* lens) {
    Core* c = (Core*)cv;
    const int G = (int)c->groups.size();
    for (int i = 0; i < n; i++) {
        Request* r = get(c, handles[i]);
        if (!r) return i;
        tokens[i] = r->tokens;
        slots[i] = r->slot;
        for (int g = 0; g < G; g++) {
            tables[(size_t)g * n + i] = (uint64_t)(uintptr_t)r->tables[g].data();
            lens[(size_t)g * n + i] = (int32_t)r->tables[g].size();
        }
    }
    return -1;
}

// Audit: every page is free or held by exactly one request; every slot likewise.  0 and "" if all is well.
int ember_cache_check(void* cv, char* msg, int cap) {
    Core* c = (Core*)cv;
    char buf[192];
    for (size_t g = 0; g < c->groups.size(); g++) {
        Group& grp = c->groups[g];
        if (!grp.paged()) continue;
        const std::string pm = grp.pool.check();
        if (!pm.empty()) { snprintf(msg, cap, "group %d: %s", (int)g, pm.c_str()); return 1; }
        std::vector<int> owner(grp.pool.n, -1);
        int owned = 0;
        for (size_t h = 0; h < c->reqs.size(); h++) {
            const Request& r = c->reqs[h];
            if (!r.live) continue;
            for (int32_t p : r.tables[g]) {
                if (p < 0) continue;
                if (p >= grp.pool.n) { snprintf(msg, cap, "group %d: page %d is outside the pool", (int)g, p); return 1; }
                if (owner[p] >= 0) {
                    snprintf(msg, cap, "group %d: page %d is held by two requests (handles %d and %d)", (int)g, p, owner[p], (int)h);
                    return 1;
                }
                owner[p] = (int)h;
                owned++;
                if (!grp.pool.held[p]) { snprintf(msg, cap, "group %d: page %d of handle %d is on the free list", (int)g, p, (int)h); return 1; }
            }
        }
        const int used = grp.pool.n - (int)grp.pool.free_.size();
        if (owned != used) { snprintf(msg, cap, "group %d: %d pages are out but requests hold %d", (int)g, used, owned); return 1; }
    }
    std::vector<uint8_t> slot_seen(c->max_requests, 0);
    int live = 0;
    for (const Request& r : c->reqs) {
        if (!r.live) continue;
        live++;
        if (r.slot < 0 || r.slot >= c->max_requests || slot_seen[r.slot]) { snprintf(msg, cap, "a state slot is held twice"); return 1; }
        slot_seen[r.slot] = 1;
    }
    for (int s : c->free_slots) {
        if (slot_seen[s]) { snprintf(msg, cap, "a state slot is both held and free"); return 1; }
        slot_seen[s] = 1;
    }
    if (live + (int)c->free_slots.size() != c->max_requests) { snprintf(msg, cap, "a state slot is lost"); return 1; }
    (void)buf;
    if (cap > 0) msg[0] = 0;
    return 0;
}

}  // extern "C"
