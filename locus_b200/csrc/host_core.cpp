// Host side of the cache, of the step and of the request loop: pools of ids with reference counts,
// the page tables of the live requests (one table per request and cache group), the assembly of a
// step's descriptors into one buffer that travels to the device in a single copy, and the scheduler's
// decisions (admission, portions under a token budget, preemption when pages run out).
//
// Plain C entry points over opaque pointers; no CUDA in here.  Every function reports misuse by a
// negative return code (the caller words the message); nothing throws across the boundary.
//
// The reference keeps the same bookkeeping in C++ (src/locus/kv/block_allocator.cpp:7-54,
// src/locus/kv/paged_cache.cpp:62-85) with one geometry for all layers; here a request holds one
// table per group of layers, and a group with a window gives pages back while the request lives.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

// Ids 0..n-1 with a count each.  A fresh pool hands out 0, 1, 2, ...; afterwards the most recently
// freed id goes out first.
struct Pool {
    std::vector<int> free_ids;
    std::vector<int> refs;

    explicit Pool(int n) : refs(static_cast<size_t>(n), 0) {
        free_ids.reserve(static_cast<size_t>(n));
        for (int i = n - 1; i >= 0; --i) free_ids.push_back(i);
    }
    int total() const { return static_cast<int>(refs.size()); }
    int n_free() const { return static_cast<int>(free_ids.size()); }
    bool in_range(int i) const { return i >= 0 && i < total(); }
    int allocate() {
        if (free_ids.empty()) return -1;
        const int i = free_ids.back();
        free_ids.pop_back();
        refs[static_cast<size_t>(i)] = 1;
        return i;
    }
    // 1: the id went back to the free list; 0: still held; -1 out of range; -2 freed twice
    int release(int i) {
        if (!in_range(i)) return -1;
        int& r = refs[static_cast<size_t>(i)];
        if (r == 0) return -2;
        if (--r == 0) {
            free_ids.push_back(i);
            return 1;
        }
        return 0;
    }
};

struct Seq {
    uint32_t generation = 0;
    bool open = false;
    int n_tokens = 0;
    int state_slot = -1;
    std::vector<std::vector<int>> tables;  // per group; -1 = page given back (window)
};

inline int pages_of(int tokens, int page_tokens) { return (tokens + page_tokens - 1) / page_tokens; }

struct Cache {
    int page_tokens, n_pages, max_seq_tokens, table_width;  // n_pages: of the largest group
    std::vector<int> window;  // per group, 0 = all keys
    std::vector<Pool> pools;
    Pool slots;
    std::vector<Seq> seqs;
    std::vector<int> spare;  // indices of closed entries of seqs
    std::vector<uint32_t> stamp;  // scratch of step assembly: which step saw a request last
    uint32_t step_no = 0;

    Cache(int n_groups, const int* windows, int page_tokens_, const int* group_pages, int n_slots, int max_seq)
        : page_tokens(page_tokens_), n_pages(0), max_seq_tokens(max_seq),
          table_width(pages_of(max_seq, page_tokens_) > 0 ? pages_of(max_seq, page_tokens_) : 1), slots(n_slots) {
        for (int g = 0; g < n_groups; ++g) {
            window.push_back(windows[g]);
            pools.emplace_back(group_pages[g]);
            n_pages = group_pages[g] > n_pages ? group_pages[g] : n_pages;
        }
    }
    int n_groups() const { return static_cast<int>(pools.size()); }
    // Pages that a request of n_tokens tokens holds in group g at most, when no step feeds it more than
    // step_tokens at once: all of them, or in a group with a window those that cover the window and the step.
    int pages_needed(int g, int n_tokens, int step_tokens) const {
        const int all = pages_of(n_tokens, page_tokens);
        const int w = window[static_cast<size_t>(g)];
        if (w <= 0 || step_tokens <= 0) return all;
        const int span = pages_of(w + step_tokens, page_tokens) + 1;
        return all < span ? all : span;
    }

    Seq* find(int64_t handle) {
        const uint32_t idx = static_cast<uint32_t>(handle & 0xffffffff);
        const uint32_t gen = static_cast<uint32_t>(static_cast<uint64_t>(handle) >> 32);
        if (idx >= seqs.size()) return nullptr;
        Seq& s = seqs[idx];
        return (s.open && s.generation == gen) ? &s : nullptr;
    }
    int capacity(const Seq& s) const {
        if (pools.empty()) return max_seq_tokens;
        size_t least = s.tables[0].size();
        for (const auto& t : s.tables) least = t.size() < least ? t.size() : least;
        return static_cast<int>(least) * page_tokens;
    }
};

Pool* as_pool(void* p) { return static_cast<Pool*>(p); }
Cache* as_cache(void* p) { return static_cast<Cache*>(p); }

// appends (group, page) to the caller's list of pages that became free
inline void note_freed(int* freed, int cap, int& n, int gid, int page) {
    if (2 * n + 1 < cap) {
        freed[2 * n] = gid;
        freed[2 * n + 1] = page;
    }
    ++n;
}

}  // namespace

extern "C" {

// ---- pools ---------------------------------------------------------------------------------
void* locus_pool_new(int n) { return n < 0 ? nullptr : new Pool(n); }
void locus_pool_delete(void* p) { delete as_pool(p); }
int locus_pool_total(void* p) { return as_pool(p)->total(); }
int locus_pool_free(void* p) { return as_pool(p)->n_free(); }
int locus_pool_refs(void* p, int i) { return as_pool(p)->in_range(i) ? as_pool(p)->refs[static_cast<size_t>(i)] : -1; }
int locus_pool_allocate(void* p) { return as_pool(p)->allocate(); }
int locus_pool_release(void* p, int i) { return as_pool(p)->release(i); }
// 0 ok; -1 out of range; -2 the id is free
int locus_pool_retain(void* p, int i) {
    Pool* pool = as_pool(p);
    if (!pool->in_range(i)) return -1;
    if (pool->refs[static_cast<size_t>(i)] == 0) return -2;
    ++pool->refs[static_cast<size_t>(i)];
    return 0;
}

// ---- cache ---------------------------------------------------------------------------------
// group_pages: pages of every group's pool (groups with a window may hold fewer than the others).
void* locus_cache_new(int n_groups, const int* windows, int page_tokens, const int* group_pages, int n_state_slots,
                      int max_seq_tokens) {
    if (n_groups < 0 || page_tokens <= 0 || n_state_slots <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (group_pages[g] < 0) return nullptr;
    return new Cache(n_groups, windows, page_tokens, group_pages, n_state_slots, max_seq_tokens);
}
int locus_cache_total_pages(void* c, int gid) { return as_cache(c)->pools[static_cast<size_t>(gid)].total(); }
int locus_cache_pages_needed(void* c, int gid, int n_tokens, int step_tokens) {
    return as_cache(c)->pages_needed(gid, n_tokens, step_tokens);
}
void locus_cache_delete(void* c) { delete as_cache(c); }
int locus_cache_table_width(void* c) { return as_cache(c)->table_width; }
int locus_cache_free_pages(void* c, int gid) { return as_cache(c)->pools[static_cast<size_t>(gid)].n_free(); }
int locus_cache_page_refs(void* c, int gid, int page) {
    Pool& p = as_cache(c)->pools[static_cast<size_t>(gid)];
    return p.in_range(page) ? p.refs[static_cast<size_t>(page)] : -1;
}
int locus_cache_slots_free(void* c) { return as_cache(c)->slots.n_free(); }
int locus_cache_slots_total(void* c) { return as_cache(c)->slots.total(); }

// A new request: takes a state slot.  Returns its handle, or -1 when no slot is free.
int64_t locus_cache_open(void* cv) {
    Cache* c = as_cache(cv);
    const int slot = c->slots.allocate();
    if (slot < 0) return -1;
    uint32_t idx;
    if (!c->spare.empty()) {
        idx = static_cast<uint32_t>(c->spare.back());
        c->spare.pop_back();
    } else {
        idx = static_cast<uint32_t>(c->seqs.size());
        c->seqs.emplace_back();
        c->stamp.push_back(0);
    }
    Seq& s = c->seqs[idx];
    s.generation = (s.generation + 1) & 0x7fffffffu;  // handles stay positive
    if (s.generation == 0) s.generation = 1;
    s.open = true;
    s.n_tokens = 0;
    s.state_slot = slot;
    s.tables.assign(static_cast<size_t>(c->n_groups()), std::vector<int>());
    return static_cast<int64_t>((static_cast<uint64_t>(s.generation) << 32) | idx);
}
int locus_cache_is_open(void* c, int64_t h) { return as_cache(c)->find(h) != nullptr; }
int locus_cache_n_tokens(void* c, int64_t h) {
    Seq* s = as_cache(c)->find(h);
    return s ? s->n_tokens : -1;
}
int locus_cache_state_slot(void* c, int64_t h) {
    Seq* s = as_cache(c)->find(h);
    return s ? s->state_slot : -1;
}
int locus_cache_capacity(void* c, int64_t h) {
    Seq* s = as_cache(c)->find(h);
    return s ? as_cache(c)->capacity(*s) : -1;
}
// Copies the request's table of group gid (at most cap entries); returns its length, -1 if not open.
int locus_cache_table(void* c, int64_t h, int gid, int* out, int cap) {
    Seq* s = as_cache(c)->find(h);
    if (!s) return -1;
    const auto& t = s->tables[static_cast<size_t>(gid)];
    const int n = static_cast<int>(t.size());
    if (n > 0 && cap > 0) std::memcpy(out, t.data(), sizeof(int) * static_cast<size_t>(n < cap ? n : cap));
    return n;
}

// Room for n_more tokens after the cached ones, in every group, all or nothing.
// 1 done; 0 some group is short of pages (nothing taken); -1 not open; -2 beyond max_seq_tokens.
int locus_cache_ensure(void* cv, int64_t h, int n_more) {
    Cache* c = as_cache(cv);
    Seq* s = c->find(h);
    if (!s) return -1;
    if (static_cast<int64_t>(s->n_tokens) + n_more > c->max_seq_tokens) return -2;
    const int want = pages_of(s->n_tokens + n_more, c->page_tokens);
    for (int g = 0; g < c->n_groups(); ++g) {
        const int missing = want - static_cast<int>(s->tables[static_cast<size_t>(g)].size());
        if (missing > c->pools[static_cast<size_t>(g)].n_free()) return 0;
    }
    for (int g = 0; g < c->n_groups(); ++g) {
        auto& t = s->tables[static_cast<size_t>(g)];
        while (static_cast<int>(t.size()) < want) t.push_back(c->pools[static_cast<size_t>(g)].allocate());
    }
    return 1;
}

// n tokens were written after the cached ones.  In a group with a window, pages that no later
// query can see go back: a query at position p sees keys t > p - window and the next query is at
// position n_tokens, so pages wholly below n_tokens - window + 1 are dead.  Writes the (group,
// page) pairs that became free to freed (cap ints) and returns their number; -1 not open; -3 the
// tokens do not fit the capacity.
int locus_cache_commit(void* cv, int64_t h, int n, int* freed, int cap) {
    Cache* c = as_cache(cv);
    Seq* s = c->find(h);
    if (!s) return -1;
    if (s->n_tokens + n > c->capacity(*s)) return -3;
    s->n_tokens += n;
    int n_freed = 0;
    for (int g = 0; g < c->n_groups(); ++g) {
        const int w = c->window[static_cast<size_t>(g)];
        if (w <= 0) continue;
        auto& t = s->tables[static_cast<size_t>(g)];
        int dead = (s->n_tokens - w + 1) / c->page_tokens;
        if (s->n_tokens - w + 1 < 0) dead = 0;
        if (dead > static_cast<int>(t.size())) dead = static_cast<int>(t.size());
        for (int i = 0; i < dead; ++i) {
            if (t[static_cast<size_t>(i)] >= 0) {
                if (c->pools[static_cast<size_t>(g)].release(t[static_cast<size_t>(i)]) == 1)
                    note_freed(freed, cap, n_freed, g, t[static_cast<size_t>(i)]);
                t[static_cast<size_t>(i)] = -1;
            }
        }
    }
    return n_freed;
}

// The request ends: everything it holds goes back.  Returns the number of (group, page) pairs
// written to freed; -1 not open.
int locus_cache_release(void* cv, int64_t h, int* freed, int cap) {
    Cache* c = as_cache(cv);
    Seq* s = c->find(h);
    if (!s) return -1;
    int n_freed = 0;
    for (int g = 0; g < c->n_groups(); ++g) {
        for (int page : s->tables[static_cast<size_t>(g)])
            if (page >= 0 && c->pools[static_cast<size_t>(g)].release(page) == 1) note_freed(freed, cap, n_freed, g, page);
        s->tables[static_cast<size_t>(g)].clear();
    }
    c->slots.release(s->state_slot);
    s->state_slot = -1;
    s->n_tokens = 0;
    s->open = false;
    c->spare.push_back(static_cast<int>(h & 0xffffffff));
    return n_freed;
}

// No page lost, held twice, or free while held; state slots likewise.  0 when all is well; else a
// code with detail[0..2]: 1 page (group, page) held detail[2] times; 2 page (group, page) held but
// its count is detail[2]; 3 group detail[0] lost detail[1] pages; 4 a state slot is held twice;
// 5 state slots lost.
int locus_cache_check(void* cv, int* detail) {
    Cache* c = as_cache(cv);
    for (int g = 0; g < c->n_groups(); ++g) {
        const int n_pages = c->pools[static_cast<size_t>(g)].total();
        std::vector<int> held(static_cast<size_t>(n_pages), 0);
        int distinct = 0;
        for (const Seq& s : c->seqs) {
            if (!s.open) continue;
            for (int page : s.tables[static_cast<size_t>(g)])
                if (page >= 0 && held[static_cast<size_t>(page)]++ == 0) ++distinct;
        }
        const Pool& pool = c->pools[static_cast<size_t>(g)];
        for (int page = 0; page < n_pages; ++page) {
            const int n = held[static_cast<size_t>(page)];
            if (n > 1) { detail[0] = g; detail[1] = page; detail[2] = n; return 1; }
            if (n == 1 && pool.refs[static_cast<size_t>(page)] != 1) {
                detail[0] = g; detail[1] = page; detail[2] = pool.refs[static_cast<size_t>(page)];
                return 2;
            }
        }
        if (distinct + pool.n_free() != pool.total()) {
            detail[0] = g; detail[1] = pool.total() - pool.n_free() - distinct; detail[2] = 0;
            return 3;
        }
    }
    std::vector<int> slot_held(static_cast<size_t>(c->slots.total()), 0);
    int n_open = 0;
    for (const Seq& s : c->seqs) {
        if (!s.open) continue;
        ++n_open;
        if (slot_held[static_cast<size_t>(s.state_slot)]++ != 0) return 4;
    }
    if (n_open + c->slots.n_free() != c->slots.total()) return 5;
    return 0;
}

// ---- step assembly -------------------------------------------------------------------------
//
// The descriptors of one step, written back to back into out (int32) in this order, with
// (offset, length) of each in layout:
//   0 tokens[T]  1 positions[T]  2 seg_q0[S]  3 seg_qn[S]  4 seg_ctx[S]  5 state_slots[S]
//   6 want_rows[n_want]  then per group g: 7 + 2g slots[T] (page * page_tokens + offset of each new
//   token), 8 + 2g block table [S, table_width] (-1 padded).
// Nothing here knows what a mixer's kernels want beyond that: work lists of tiles and the like are planned
// by the parts themselves (they may use the helpers at the end of this section) and ride behind these
// descriptors in the same buffer.
// info: T, n_want, longest context after the step, and on an error the offending entry [6] and a value
//       [7] (for codes 5 and 9 the index, within the entry, of the token or wanted place).
// Checks before anything is written that could be launched: 0 ok; 1 no entries; 2 more entries than
// max_segments; 3 a request twice; 4 an entry without tokens; 5 token outside the vocabulary;
// 6 beyond max_positions; 7 request not open; 8 capacity not ensured; 9 wanted place outside the
// entry; 10 more than max_tokens tokens; 11 more than max_wanted rows; 12 a position in a page
// already given back; 13 out too small.
int locus_step_build(void* cv, int n_entries, const int64_t* handles, const int* counts, const int64_t* tokens,
                     const int* want_counts, const int64_t* wants, int vocab, int max_positions, int max_tokens,
                     int max_segments, int max_wanted, int* out, int64_t out_cap, int* layout, int* info) {
    Cache* c = as_cache(cv);
    info[6] = info[7] = 0;
    if (n_entries <= 0) return 1;
    if (n_entries > max_segments) { info[7] = n_entries; return 2; }
    c->step_no += 1;
    if (c->step_no == 0) {  // wrapped: forget old stamps
        for (auto& s : c->stamp) s = 0;
        c->step_no = 1;
    }
    int64_t T = 0, n_want = 0;
    {
        const int64_t* tok = tokens;
        const int64_t* wnt = wants;
        for (int e = 0; e < n_entries; ++e) {
            info[6] = e;
            Seq* s = c->find(handles[e]);
            if (!s) return 7;
            const uint32_t idx = static_cast<uint32_t>(handles[e] & 0xffffffff);
            if (c->stamp[idx] == c->step_no) return 3;
            c->stamp[idx] = c->step_no;
            const int n = counts[e];
            if (n <= 0) return 4;
            for (int i = 0; i < n; ++i)
                if (tok[i] < 0 || tok[i] >= vocab) { info[7] = i; return 5; }
            if (static_cast<int64_t>(s->n_tokens) + n > max_positions) { info[7] = s->n_tokens + n; return 6; }
            if (s->n_tokens + n > c->capacity(*s)) { info[7] = n; return 8; }
            for (int i = 0; i < want_counts[e]; ++i)
                if (wnt[i] < 0 || wnt[i] >= n) { info[7] = i; return 9; }
            T += n;
            n_want += want_counts[e];
            tok += n;
            wnt += want_counts[e];
        }
    }
    if (T > max_tokens) { info[7] = static_cast<int>(T); return 10; }
    if (n_want > max_wanted) { info[7] = static_cast<int>(n_want); return 11; }
    const int S = n_entries, G = c->n_groups(), W = c->table_width;
    const int F = 7;
    const int64_t lens[F] = {T, T, S, S, S, S, n_want};
    int64_t off = 0;
    for (int f = 0; f < F; ++f) {
        layout[2 * f] = static_cast<int>(off);
        layout[2 * f + 1] = static_cast<int>(lens[f]);
        off += lens[f];
    }
    for (int g = 0; g < G; ++g) {
        layout[2 * (F + 2 * g)] = static_cast<int>(off);
        layout[2 * (F + 2 * g) + 1] = static_cast<int>(T);
        off += T;
        layout[2 * (F + 1 + 2 * g)] = static_cast<int>(off);
        layout[2 * (F + 1 + 2 * g) + 1] = S * W;
        off += static_cast<int64_t>(S) * W;
    }
    if (off > out_cap) return 13;
    int* o_tok = out + layout[0];
    int* o_pos = out + layout[2];
    int* o_q0 = out + layout[4];
    int* o_qn = out + layout[6];
    int* o_ctx = out + layout[8];
    int* o_slot = out + layout[10];
    int* o_want = out + layout[12];
    int row = 0, longest = 0;
    const int64_t* tok = tokens;
    const int64_t* wnt = wants;
    const int P = c->page_tokens;
    for (int e = 0; e < n_entries; ++e) {
        Seq* s = c->find(handles[e]);
        const int n = counts[e], ctx = s->n_tokens;
        o_q0[e] = row;
        o_qn[e] = n;
        o_ctx[e] = ctx;
        o_slot[e] = s->state_slot;
        for (int i = 0; i < want_counts[e]; ++i) *o_want++ = row + static_cast<int>(wnt[i]);
        for (int i = 0; i < n; ++i) {
            o_tok[row + i] = static_cast<int>(tok[i]);
            o_pos[row + i] = ctx + i;
        }
        if (ctx + n > longest) longest = ctx + n;
        for (int g = 0; g < G; ++g) {
            const auto& t = s->tables[static_cast<size_t>(g)];
            int* o_slots = out + layout[2 * (F + 2 * g)] + row;
            for (int i = 0; i < n; ++i) {
                const int pos = ctx + i;
                const int page = t[static_cast<size_t>(pos / P)];
                if (page < 0) { info[6] = e; info[7] = pos; return 12; }
                o_slots[i] = page * P + pos % P;
            }
            int* o_table = out + layout[2 * (F + 1 + 2 * g)] + static_cast<int64_t>(e) * W;
            const int len = static_cast<int>(t.size());
            if (len > 0) std::memcpy(o_table, t.data(), sizeof(int) * static_cast<size_t>(len));
            for (int i = len; i < W; ++i) o_table[i] = -1;
        }
        row += n;
        tok += n;
        wnt += want_counts[e];
    }
    info[0] = static_cast<int>(T);
    info[1] = static_cast<int>(n_want);
    info[2] = longest;
    return 0;
}

// Helpers for parts that plan work lists over the segments of a step.  seg_qn: new tokens per segment.
// Tiles of `tile` queries over every segment with at least min_new new tokens, as pairs (segment, first
// query of the tile) in segment order; returns the number of pairs, or -1 when out (cap ints) is too small.
int locus_plan_query_tiles(int n_seg, const int* seg_qn, int tile, int min_new, int* out, int64_t cap) {
    if (tile <= 0) return -1;
    int64_t n = 0;
    for (int s = 0; s < n_seg; ++s) {
        if (seg_qn[s] < min_new) continue;
        for (int q = 0; q < seg_qn[s]; q += tile) {
            if (2 * n + 1 >= cap) return -1;
            out[2 * n] = s;
            out[2 * n + 1] = q;
            ++n;
        }
    }
    return static_cast<int>(n);
}

// Orders n query tiles (segment, first query) by the position of their first query, seg_ctx[segment] + first
// query, ascending and stable: the attention kernels walk the list from its end, so the tiles that see the most
// keys go out first and the short ones fill the tail, whichever requests they belong to.
void locus_sort_tiles_by_position(int n, int* items, const int* seg_ctx) {
    if (n <= 1) return;
    std::vector<std::pair<int, int>> v(n);
    for (int i = 0; i < n; ++i) v[i] = {items[2 * i], items[2 * i + 1]};
    std::stable_sort(v.begin(), v.end(), [&](const std::pair<int, int>& a, const std::pair<int, int>& b) {
        return seg_ctx[a.first] + a.second < seg_ctx[b.first] + b.second;
    });
    for (int i = 0; i < n; ++i) {
        items[2 * i] = v[i].first;
        items[2 * i + 1] = v[i].second;
    }
}

// The segments with exactly `new_tokens` new tokens, in order; returns their number, or -1 when out is too small.
int locus_plan_segments_with(int n_seg, const int* seg_qn, int new_tokens, int* out, int64_t cap) {
    int64_t n = 0;
    for (int s = 0; s < n_seg; ++s) {
        if (seg_qn[s] != new_tokens) continue;
        if (n >= cap) return -1;
        out[n++] = s;
    }
    return static_cast<int>(n);
}

}  // extern "C"

// ---- scheduler -----------------------------------------------------------------------------
//
// The decisions of the request loop over the cache above: which waiting request is admitted, which
// tokens of which running request go into the next step, who gives way when pages run out.  The
// policy is the reference engine's (src/locus/engine/engine.cpp:503-634): admission first come first
// served while the pool has free pages for prompt + generated + headroom tokens (nothing is reserved,
// nobody overtakes the front of the queue); when a request cannot get its pages the newest admitted
// request is preempted (its pages go back, it returns to the FRONT of the queue and is recomputed
// later); a request that is itself the newest sits the step out, or fails if it runs alone; a request
// whose next token has no position left fails with a context overflow.  Unlike the reference, portions
// of prompts and decode tokens share one step and one token budget: decode tokens first, the rest to
// portions in admission order, each at most `chunk` tokens.
//
// The caller keeps the tokens and the records; this side keeps lengths and states, and reports what it
// decided as events (kind, request, argument) that the caller applies to its records.
namespace {

enum : int { ST_WAITING = 0, ST_RUNNING = 1, ST_DONE = 2, ST_FAILED = 3 };
enum : int { EV_ADMITTED = 1, EV_PREEMPTED = 2, EV_FAILED = 3, EV_DONE = 4 };
enum : int { WHY_OVERFLOW = 1, WHY_POOL_TOO_SMALL = 2 };

struct SReq {
    int stream_len = 0;  // prompt + generated tokens
    int n_fed = 0;       // of them, through the model
    int status = ST_WAITING;
    int64_t handle = -1;
    int preemptions = 0;
};

struct Sched {
    Cache* cache;
    int max_batch_tokens, chunk, headroom, max_running, max_positions;
    std::deque<int64_t> waiting;
    std::vector<int64_t> running;  // in admission order
    std::unordered_map<int64_t, SReq> reqs;
    std::vector<int64_t> events;   // triples (kind, request, argument)
    std::vector<int> freed;        // (group, page) pairs that became free since the caller last asked
    int n_preemptions = 0, n_admitted = 0;

    void event(int kind, int64_t rid, int64_t arg) {
        events.push_back(kind);
        events.push_back(rid);
        events.push_back(arg);
    }
    // whether every group has free pages for a request of n_tokens tokens (fed at most `chunk` at a time)
    bool room_for(int n_tokens) const {
        for (int g = 0; g < cache->n_groups(); ++g)
            if (cache->pages_needed(g, n_tokens, chunk) > cache->pools[static_cast<size_t>(g)].n_free()) return false;
        return true;
    }
    void give_back(SReq& r) {
        if (r.handle < 0) return;
        const size_t before = freed.size();
        freed.resize(before + 2 * static_cast<size_t>(cache->n_groups()) * static_cast<size_t>(cache->table_width));
        const int n = locus_cache_release(cache, r.handle, freed.data() + before,
                                          static_cast<int>(freed.size() - before));
        freed.resize(before + 2 * static_cast<size_t>(n > 0 ? n : 0));
        r.handle = -1;
    }
    void finish(int64_t rid, SReq& r, int status, int why) {
        give_back(r);
        running.erase(std::remove(running.begin(), running.end(), rid), running.end());
        r.status = status;
        event(status == ST_DONE ? EV_DONE : EV_FAILED, rid, why);
    }
    void preempt(int64_t rid, SReq& r) {
        give_back(r);
        r.n_fed = 0;
        r.status = ST_WAITING;
        r.preemptions += 1;
        running.erase(std::remove(running.begin(), running.end(), rid), running.end());
        waiting.push_front(rid);  // victims go to the front
        n_preemptions += 1;
        event(EV_PREEMPTED, rid, 0);
    }
};

Sched* as_sched(void* p) { return static_cast<Sched*>(p); }

}  // namespace

extern "C" {

void* locus_sched_new(void* cache, int max_batch_tokens, int chunk, int headroom, int max_running,
                      int max_positions) {
    if (cache == nullptr || max_batch_tokens <= 0 || chunk <= 0 || headroom < 0 || max_running <= 0) return nullptr;
    Sched* s = new Sched();
    s->cache = as_cache(cache);
    s->max_batch_tokens = max_batch_tokens;
    s->chunk = chunk;
    s->headroom = headroom;
    s->max_running = max_running;
    s->max_positions = max_positions;
    return s;
}
void locus_sched_delete(void* s) { delete as_sched(s); }

// A new request of prompt_len tokens joins the end of the queue.  0 ok; -1 the id is in use.
int locus_sched_add(void* sv, int64_t rid, int prompt_len) {
    Sched* s = as_sched(sv);
    if (s->reqs.count(rid)) return -1;
    SReq r;
    r.stream_len = prompt_len;
    s->reqs[rid] = r;
    s->waiting.push_back(rid);
    return 0;
}
// The record of a finished request is dropped.
void locus_sched_forget(void* sv, int64_t rid) {
    Sched* s = as_sched(sv);
    auto it = s->reqs.find(rid);
    if (it != s->reqs.end() && (it->second.status == ST_DONE || it->second.status == ST_FAILED)) s->reqs.erase(it);
}

// Admits from the front of the queue while there is room; returns how many were admitted.
int locus_sched_admit(void* sv) {
    Sched* s = as_sched(sv);
    int n = 0;
    while (!s->waiting.empty() && static_cast<int>(s->running.size()) < s->max_running) {
        const int64_t rid = s->waiting.front();
        SReq& r = s->reqs[rid];
        if (!s->room_for(r.stream_len + s->headroom) || s->cache->slots.n_free() == 0) break;  // nobody overtakes the front
        s->waiting.pop_front();
        r.handle = locus_cache_open(s->cache);
        r.status = ST_RUNNING;
        r.n_fed = 0;
        s->running.push_back(rid);
        s->n_admitted += 1;
        s->event(EV_ADMITTED, rid, r.handle);
        ++n;
    }
    return n;
}

// Chooses the next step's tokens and takes their pages.  Writes (request, first stream index, tokens,
// wants logits) per planned request to out (cap entries of 4), in admission order; returns their number.
int locus_sched_plan(void* sv, int64_t* out, int cap) {
    Sched* s = as_sched(sv);
    Cache* c = s->cache;
    // context overflow: the next token to feed has no position left
    {
        const std::vector<int64_t> snapshot = s->running;
        for (int64_t rid : snapshot) {
            SReq& r = s->reqs[rid];
            if (r.n_fed + 1 > s->max_positions || r.n_fed + 1 > c->max_seq_tokens) s->finish(rid, r, ST_FAILED, WHY_OVERFLOW);
        }
    }
    std::vector<int64_t> order;
    for (int64_t rid : s->running)
        if (s->reqs[rid].stream_len - s->reqs[rid].n_fed == 1) order.push_back(rid);
    for (int64_t rid : s->running)
        if (s->reqs[rid].stream_len - s->reqs[rid].n_fed > 1) order.push_back(rid);
    std::unordered_map<int64_t, std::pair<int, int>> planned;  // request -> (start, n)
    int budget = s->max_batch_tokens;
    for (int64_t rid : order) {
        auto it = s->reqs.find(rid);
        if (it == s->reqs.end() || it->second.status != ST_RUNNING || budget <= 0) continue;
        SReq& r = it->second;
        const int left = r.stream_len - r.n_fed;
        int n = std::min(std::min(left, budget), s->chunk);
        n = std::min(n, std::min(s->max_positions - r.n_fed, c->max_seq_tokens - r.n_fed));
        if (n <= 0) continue;
        bool ok = true;
        while (locus_cache_ensure(c, r.handle, n) != 1) {
            const int64_t victim = s->running.back();
            if (victim == rid) {
                if (s->running.size() == 1) s->finish(rid, r, ST_FAILED, WHY_POOL_TOO_SMALL);
                ok = false;  // the newest but not alone: it sits this step out
                break;
            }
            planned.erase(victim);
            s->preempt(victim, s->reqs[victim]);
        }
        if (!ok) continue;
        planned[rid] = std::make_pair(r.n_fed, n);
        budget -= n;
    }
    int n_out = 0;
    for (int64_t rid : s->running) {
        auto it = planned.find(rid);
        if (it == planned.end()) continue;
        if (n_out < cap) {
            const SReq& r = s->reqs[rid];
            out[4 * n_out] = rid;
            out[4 * n_out + 1] = it->second.first;
            out[4 * n_out + 2] = it->second.second;
            out[4 * n_out + 3] = (it->second.first + it->second.second == r.stream_len) ? 1 : 0;
        }
        ++n_out;
    }
    return n_out;
}

// n tokens of the request went through the model.
void locus_sched_fed(void* sv, int64_t rid, int n) {
    auto it = as_sched(sv)->reqs.find(rid);
    if (it != as_sched(sv)->reqs.end()) it->second.n_fed += n;
}
// A token was generated for the request; finished != 0: it ends here (everything it holds goes back).
void locus_sched_token(void* sv, int64_t rid, int finished) {
    Sched* s = as_sched(sv);
    auto it = s->reqs.find(rid);
    if (it == s->reqs.end()) return;
    it->second.stream_len += 1;
    if (finished) s->finish(rid, it->second, ST_DONE, 0);
}

// The events since the last call, as triples (kind, request, argument), at most cap triples; returns the
// number written and forgets them.  Kinds: 1 admitted (argument = cache handle), 2 preempted, 3 failed
// (argument: 1 context overflow, 2 pool too small for the request), 4 done.
int locus_sched_events(void* sv, int64_t* out, int cap) {
    Sched* s = as_sched(sv);
    const int n = std::min(cap, static_cast<int>(s->events.size() / 3));
    std::copy(s->events.begin(), s->events.begin() + 3 * n, out);
    s->events.erase(s->events.begin(), s->events.begin() + 3 * n);
    return n;
}
// The (group, page) pairs that became free through this scheduler since the last call (at most cap ints).
int locus_sched_freed(void* sv, int* out, int cap) {
    Sched* s = as_sched(sv);
    const int n = std::min(cap, static_cast<int>(s->freed.size()));
    std::copy(s->freed.begin(), s->freed.begin() + n, out);
    s->freed.erase(s->freed.begin(), s->freed.begin() + n);
    return n / 2;
}
// Queue contents: which = 0 waiting (front first), 1 running (admission order); returns the length.
int locus_sched_queue(void* sv, int which, int64_t* out, int cap) {
    Sched* s = as_sched(sv);
    int n = 0;
    if (which == 0) {
        for (int64_t rid : s->waiting) { if (n < cap) out[n] = rid; ++n; }
    } else {
        for (int64_t rid : s->running) { if (n < cap) out[n] = rid; ++n; }
    }
    return n;
}
int locus_sched_count(void* sv, int which) {
    Sched* s = as_sched(sv);
    return which == 0 ? static_cast<int>(s->waiting.size()) : static_cast<int>(s->running.size());
}

}  // extern "C"
