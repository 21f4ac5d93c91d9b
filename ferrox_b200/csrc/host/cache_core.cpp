// Host side of the cache manager: page pools, block tables, slots.  Plain C++ (no
// CUDA), compiled with the host compiler into libferrox_b200_host.so and driven from
// ferrox_b200/cache/manager.py, which owns the device tensors.
//
// A *group* is a set of layers that share one page-id space: its pool (LIFO free
// list: the page freed last is handed out first), one block table per request slot
// ([max_slots][width] int32, -1 = no page) and, for each slot, the range of logical
// pages still held [first_page, n_logical).  A group with a window gives back, at
// commit, the pages whose every position is older than new_len - window + 1.
// reserve() is all-or-nothing over all groups.
//
// Reference: crates/ferrox-core/src/cache.rs:331-405 (shared pages, LIFO free list),
// :427-488 (block table per sequence, exhaustion returned as a value, state
// unchanged).  Groups and window release have no counterpart there.
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

struct Group {
    int window;  // -1: every earlier position stays readable
    int n_pages;
    std::vector<int> free_list;      // back() is handed out next
    std::vector<uint8_t> held;
    std::vector<int32_t> table;      // [max_slots * width]
    std::vector<int> first_page, n_logical;
    std::vector<uint8_t> dirty;      // rows whose device copy is stale
    int peak = 0;
};

struct Cache {
    int page_size, max_slots, width, max_positions;
    std::vector<Group> groups;
    std::vector<int> free_slots;
    std::vector<uint8_t> live;
    std::vector<int> seq_len;
};

inline int pages_for(const Cache& c, int len) { return (len + c.page_size - 1) / c.page_size; }

}  // namespace

extern "C" {

// status codes
enum { FXH_OK = 0, FXH_NO = 1, FXH_BAD_SLOT = -1, FXH_TOO_LONG = -2, FXH_SHRINK = -3, FXH_CORRUPT = -4 };

void* fxh_cache_create(int n_groups, const int* windows, const int* n_pages, int page_size, int max_slots, int width,
                       int max_positions)
{
    if (n_groups < 0 || page_size <= 0 || max_slots <= 0 || width <= 0) return nullptr;
    Cache* c = new Cache();
    c->page_size = page_size; c->max_slots = max_slots; c->width = width; c->max_positions = max_positions;
    c->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        Group& G = c->groups[g];
        G.window = windows[g];
        G.n_pages = n_pages[g];
        G.free_list.reserve(G.n_pages);
        for (int p = G.n_pages - 1; p >= 0; --p) G.free_list.push_back(p);   // ascending ids come out first
        G.held.assign(G.n_pages, 0);
        G.table.assign((size_t)max_slots * width, -1);
        G.first_page.assign(max_slots, 0);
        G.n_logical.assign(max_slots, 0);
        G.dirty.assign(max_slots, 0);
    }
    for (int s = max_slots - 1; s >= 0; --s) c->free_slots.push_back(s);
    c->live.assign(max_slots, 0);
    c->seq_len.assign(max_slots, 0);
    return c;
}

void fxh_cache_destroy(void* h) { delete static_cast<Cache*>(h); }

int fxh_open(void* h)
{
    Cache* c = static_cast<Cache*>(h);
    if (c->free_slots.empty()) return -1;
    const int s = c->free_slots.back();
    c->free_slots.pop_back();
    c->live[s] = 1;
    c->seq_len[s] = 0;
    return s;
}

static int check_live(const Cache* c, int slot) { return slot >= 0 && slot < c->max_slots && c->live[slot]; }

int fxh_close(void* h, int slot)
{
    Cache* c = static_cast<Cache*>(h);
    if (!check_live(c, slot)) return FXH_BAD_SLOT;
    for (Group& G : c->groups) {
        int32_t* row = G.table.data() + (size_t)slot * c->width;
        for (int j = G.first_page[slot]; j < G.n_logical[slot]; ++j) {
            const int p = row[j];
            if (p < 0) continue;
            if (p >= G.n_pages || !G.held[p]) return FXH_CORRUPT;
            G.held[p] = 0;
            G.free_list.push_back(p);
        }
        if (G.n_logical[slot]) {
            for (int j = 0; j < G.n_logical[slot]; ++j) row[j] = -1;
            G.dirty[slot] = 1;
        }
        G.first_page[slot] = 0;
        G.n_logical[slot] = 0;
    }
    c->seq_len[slot] = 0;
    c->live[slot] = 0;
    c->free_slots.push_back(slot);
    return FXH_OK;
}

// out[g] = pages group g still has to get so that positions < new_len are mapped
int fxh_pages_needed(void* h, int slot, int new_len, int* out)
{
    Cache* c = static_cast<Cache*>(h);
    if (slot < 0 || slot >= c->max_slots) return FXH_BAD_SLOT;
    const int need = pages_for(*c, new_len);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        const int d = need - c->groups[g].n_logical[slot];
        out[g] = d > 0 ? d : 0;
    }
    return FXH_OK;
}

int fxh_reserve(void* h, int slot, int new_len)
{
    Cache* c = static_cast<Cache*>(h);
    if (!check_live(c, slot)) return FXH_BAD_SLOT;
    if (new_len > c->max_positions) return FXH_TOO_LONG;
    const int need = pages_for(*c, new_len);
    for (const Group& G : c->groups) {
        const int d = need - G.n_logical[slot];
        if (d > (int)G.free_list.size()) return FXH_NO;   // nothing has been changed
    }
    for (Group& G : c->groups) {
        const int d = need - G.n_logical[slot];
        if (d <= 0) continue;
        int32_t* row = G.table.data() + (size_t)slot * c->width;
        for (int i = 0; i < d; ++i) {
            const int p = G.free_list.back();
            G.free_list.pop_back();
            G.held[p] = 1;
            row[G.n_logical[slot] + i] = p;
        }
        G.n_logical[slot] += d;
        G.dirty[slot] = 1;
        const int in_use = G.n_pages - (int)G.free_list.size();
        if (in_use > G.peak) G.peak = in_use;
    }
    return FXH_OK;
}

int fxh_commit(void* h, int slot, int new_len)
{
    Cache* c = static_cast<Cache*>(h);
    if (!check_live(c, slot)) return FXH_BAD_SLOT;
    if (new_len < c->seq_len[slot]) return FXH_SHRINK;
    c->seq_len[slot] = new_len;
    for (Group& G : c->groups) {
        if (G.window < 0) continue;
        // the next query, at position new_len, reads from new_len - window + 1 on
        int first_needed = new_len - G.window + 1;
        if (first_needed < 0) first_needed = 0;
        int upto = first_needed / c->page_size;
        if (upto > G.n_logical[slot]) upto = G.n_logical[slot];
        int32_t* row = G.table.data() + (size_t)slot * c->width;
        if (upto > G.first_page[slot]) {
            for (int j = G.first_page[slot]; j < upto; ++j) {
                const int p = row[j];
                if (p < 0 || p >= G.n_pages || !G.held[p]) return FXH_CORRUPT;
                G.held[p] = 0;
                G.free_list.push_back(p);
                row[j] = -1;
            }
            G.first_page[slot] = upto;
            G.dirty[slot] = 1;
        }
    }
    return FXH_OK;
}

// One step's reservation in one call: request slots[i] grows by add[i] positions.  Pages are mapped for all of them or
// for none (FXH_NO: nothing has been changed); starts[i] receives the request's length before the step.  The slots
// must be distinct.
int fxh_reserve_step(void* h, int n, const int* slots, const int* add, int* starts)
{
    Cache* c = static_cast<Cache*>(h);
    for (int i = 0; i < n; ++i) {
        if (!check_live(c, slots[i]) || add[i] < 0) return FXH_BAD_SLOT;
        if (c->seq_len[slots[i]] + add[i] > c->max_positions) return FXH_TOO_LONG;
    }
    for (const Group& G : c->groups) {
        long need = 0;
        for (int i = 0; i < n; ++i) {
            const int d = pages_for(*c, c->seq_len[slots[i]] + add[i]) - G.n_logical[slots[i]];
            if (d > 0) need += d;
        }
        if (need > (long)G.free_list.size()) return FXH_NO;
    }
    for (int i = 0; i < n; ++i) {
        starts[i] = c->seq_len[slots[i]];
        const int rc = fxh_reserve(h, slots[i], starts[i] + add[i]);
        if (rc != FXH_OK) return rc < 0 ? rc : FXH_CORRUPT;   // cannot happen after the count above
    }
    return FXH_OK;
}

// The step has run: every request's length advances by add[i] (windowed groups give back what fell out).
int fxh_commit_step(void* h, int n, const int* slots, const int* add)
{
    Cache* c = static_cast<Cache*>(h);
    for (int i = 0; i < n; ++i) {
        if (!check_live(c, slots[i])) return FXH_BAD_SLOT;
        const int rc = fxh_commit(h, slots[i], c->seq_len[slots[i]] + add[i]);
        if (rc != FXH_OK) return rc;
    }
    return FXH_OK;
}

int32_t* fxh_table(void* h, int group) { return static_cast<Cache*>(h)->groups[group].table.data(); }
int fxh_free_pages(void* h, int group) { return (int)static_cast<Cache*>(h)->groups[group].free_list.size(); }
int fxh_peak_pages(void* h, int group) { return static_cast<Cache*>(h)->groups[group].peak; }
int fxh_free_slots(void* h) { return (int)static_cast<Cache*>(h)->free_slots.size(); }
int fxh_seq_len(void* h, int slot) { return static_cast<Cache*>(h)->seq_len[slot]; }
int fxh_first_page(void* h, int group, int slot) { return static_cast<Cache*>(h)->groups[group].first_page[slot]; }
int fxh_n_logical(void* h, int group, int slot) { return static_cast<Cache*>(h)->groups[group].n_logical[slot]; }
int fxh_is_live(void* h, int slot) { return check_live(static_cast<Cache*>(h), slot); }

// rows of group's table whose device copy is stale; clears the marks.  Returns the count.
int fxh_take_dirty(void* h, int group, int* rows, int cap)
{
    Group& G = static_cast<Cache*>(h)->groups[group];
    int n = 0;
    for (size_t s = 0; s < G.dirty.size() && n < cap; ++s)
        if (G.dirty[s]) { rows[n++] = (int)s; G.dirty[s] = 0; }
    return n;
}

// 0 when no page is lost, held twice or free while mapped; else a code that tells which rule broke.
int fxh_check(void* h)
{
    Cache* c = static_cast<Cache*>(h);
    for (Group& G : c->groups) {
        std::vector<int> seen(G.n_pages, 0);
        long mapped = 0;
        for (int s = 0; s < c->max_slots; ++s) {
            const int32_t* row = G.table.data() + (size_t)s * c->width;
            for (int j = 0; j < c->width; ++j) {
                const int p = row[j];
                const bool inside = c->live[s] && j >= G.first_page[s] && j < G.n_logical[s];
                if (p >= 0 && !inside) return 1;                 // a page mapped outside a live slot's held range
                if (p < 0 && inside) return 2;                   // a hole in the held range
                if (p >= 0) {
                    if (p >= G.n_pages || seen[p]++) return 3;   // a page held twice
                    if (!G.held[p]) return 4;                    // mapped but not marked held
                    ++mapped;
                }
            }
        }
        std::vector<int> on_free(G.n_pages, 0);
        for (int p : G.free_list) {
            if (p < 0 || p >= G.n_pages || on_free[p]++) return 5;   // on the free list twice
            if (seen[p]) return 6;                                   // mapped and free
        }
        if (mapped + (long)G.free_list.size() != G.n_pages) return 7;   // a page lost
    }
    return 0;
}

}  // extern "C"
