// The books of the cache manager in native code: pages, block tables, request slots, and
// the layout of a step's metadata.  Host logic only - no CUDA in this file; it is compiled with
// the host compiler and loaded through ctypes like the kernel libraries.
//
// Keys and values live in pages of `page_tokens` positions.  Layers with the same needs form a
// group with its own pool of pages and its own free list (a stack: the page given back last is
// handed out first); a page id is shared by all layers of the group.  The reference's device
// pool does the same with its "kinds" (model/KvPool.cajeta:11-17,170-210,
// model/KvFreeList.cajeta:4-60).  A request holds a slot: the row of its block table in every
// group.  Position p of a request lies in page table[slot][p / page_tokens] at p % page_tokens
// (model/KvPage.cajeta:15-19).
//
// Pages are given back when the request is released (model/PagedKvCache.cajeta:639-661,
// model/KvPool.cajeta:348-367) and, in a windowed group, as soon as every position of a page
// lies behind the window of the request's next token: with length L and window w the next token
// reads keys [L + 1 - w, L] (model/PagedKvCache.cajeta:382-388), so page j goes back when
// (j + 1) * page_tokens <= L + 1 - w.  A reservation is all or nothing across groups (and, for a
// whole step, across requests) and leaves the books unchanged when pages run out
// (model/PagedKvCache.cajeta:200-207, model/KvPool.cajeta:234-255).
//
// Every function returns a status: >= 0 as documented, CJ_BOOKS_ERROR (-1) for a misuse, whose
// text cj_books_error() gives.  Block tables, lengths and the live ranges are exposed as raw
// arrays (they never move), so that the Python side can view them without copies.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#define CJ_EXPORT extern "C" __attribute__((visibility("default")))
#define CJ_BOOKS_ERROR (-1)

namespace {

struct Allocator {
    int num_pages = 0;
    std::vector<int> free_list;          // a stack: back() is handed out next
    std::vector<uint8_t> held;
    std::string error;

    explicit Allocator(int n) : num_pages(n), held((size_t)(n > 0 ? n : 0), 0) {
        free_list.reserve((size_t)(n > 0 ? n : 0));
        for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
    }
    int free_count() const { return (int)free_list.size(); }

    // n pages into out, or false (nothing taken) when fewer are free
    bool take(int n, int* out) {
        if (n > free_count()) return false;
        for (int i = 0; i < n; ++i) {
            int p = free_list.back();
            free_list.pop_back();
            held[(size_t)p] = 1;
            out[i] = p;
        }
        return true;
    }
    bool give_back(const int* pages, int n) {
        for (int i = 0; i < n; ++i) {
            int p = pages[i];
            if (p < 0 || p >= num_pages) { error = "page " + std::to_string(p) + " does not exist"; return false; }
            if (!held[(size_t)p]) { error = "page " + std::to_string(p) + " freed twice"; return false; }
            held[(size_t)p] = 0;
            free_list.push_back(p);
        }
        return true;
    }
    // no page lost, held twice or free twice
    bool check() {
        std::vector<uint8_t> on_list((size_t)num_pages, 0);
        for (int p : free_list) {
            if (p < 0 || p >= num_pages) { error = "page " + std::to_string(p) + " on the free list does not exist"; return false; }
            if (on_list[(size_t)p]) { error = "a page is on the free list twice"; return false; }
            on_list[(size_t)p] = 1;
        }
        for (int p = 0; p < num_pages; ++p)
            if ((held[(size_t)p] != 0) == (on_list[(size_t)p] != 0)) {
                error = "page " + std::to_string(p) + (held[(size_t)p] ? " is both held and free" : " is neither held nor free");
                return false;
            }
        return true;
    }
};

struct Group {
    int window;
    Allocator alloc;
    std::vector<int32_t> table;          // [max_seqs, width], -1 where no page is held
    std::vector<int64_t> first_live;     // lowest logical page still held
    std::vector<int64_t> next_page;      // logical pages ever given (held: [first_live, next_page))
    Group(int window_, int pages, int max_seqs, int width)
        : window(window_), alloc(pages), table((size_t)max_seqs * width, -1), first_live((size_t)max_seqs, 0),
          next_page((size_t)max_seqs, 0) {}
};

struct Books {
    int page_tokens, max_seqs, max_tokens, width;
    std::vector<Group> groups;
    std::vector<int64_t> length;
    std::vector<uint8_t> live;
    std::vector<int> free_slots;         // a stack
    std::vector<int> scratch;
    std::string error;

    int64_t pages_for(int64_t length_) const { return (length_ + page_tokens - 1) / page_tokens; }
    bool is_live(int slot) const { return slot >= 0 && slot < max_seqs && live[(size_t)slot]; }
    bool need_live(int slot) {
        if (is_live(slot)) return true;
        error = "slot " + std::to_string(slot) + " holds no request";
        return false;
    }
    int64_t needed(const Group& g, int slot, int64_t L, int64_t n_new) const {
        int64_t n = pages_for(L + n_new) - g.next_page[(size_t)slot];
        return n > 0 ? n : 0;
    }
    bool grow(Group& g, int slot, int n) {
        int64_t start = g.next_page[(size_t)slot];
        if (start + n > width) {
            error = "request in slot " + std::to_string(slot) + " needs " + std::to_string(start + n) +
                    " pages; a table row holds " + std::to_string(width);
            return false;
        }
        if (n > 0) {
            scratch.resize((size_t)n);
            bool ok = g.alloc.take(n, scratch.data());
            if (!ok) { error = "pages ran out inside a reservation that was checked"; return false; }
            for (int i = 0; i < n; ++i) g.table[(size_t)slot * width + start + i] = scratch[(size_t)i];
            g.next_page[(size_t)slot] = start + n;
        }
        return true;
    }
    // gives back the pages that lie wholly behind the window of the next token
    bool trim_window(Group& g, int slot, int64_t L) {
        if (g.window <= 0) return true;
        int64_t dead_below = L + 1 - g.window;            // positions below are never read again
        if (dead_below <= 0) return true;
        int64_t last_dead = dead_below / page_tokens;
        if (last_dead > g.next_page[(size_t)slot]) last_dead = g.next_page[(size_t)slot];
        int64_t first = g.first_live[(size_t)slot];
        if (last_dead <= first) return true;
        int32_t* row = g.table.data() + (size_t)slot * width;
        scratch.assign(row + first, row + last_dead);
        if (!g.alloc.give_back(scratch.data(), (int)scratch.size())) { error = g.alloc.error; return false; }
        for (int64_t j = first; j < last_dead; ++j) row[j] = -1;
        g.first_live[(size_t)slot] = last_dead;
        return true;
    }
    bool release_group(Group& g, int slot) {
        int64_t first = g.first_live[(size_t)slot], nxt = g.next_page[(size_t)slot];
        int32_t* row = g.table.data() + (size_t)slot * width;
        scratch.assign(row + first, row + nxt);
        if (!g.alloc.give_back(scratch.data(), (int)scratch.size())) { error = g.alloc.error; return false; }
        for (int64_t j = 0; j < nxt; ++j) row[j] = -1;
        g.first_live[(size_t)slot] = 0;
        g.next_page[(size_t)slot] = 0;
        return true;
    }
};

Books* B(void* h) { return (Books*)h; }

}  // namespace

// ---- a free list on its own ------------------------------------------------------------------
CJ_EXPORT void* cj_pages_create(int num_pages) { return num_pages < 0 ? nullptr : new Allocator(num_pages); }
CJ_EXPORT void cj_pages_destroy(void* a) { delete (Allocator*)a; }
CJ_EXPORT const char* cj_pages_error(void* a) { return ((Allocator*)a)->error.c_str(); }
CJ_EXPORT int cj_pages_free_count(void* a) { return ((Allocator*)a)->free_count(); }
// 1 and n pages in out, or 0 and nothing taken
CJ_EXPORT int cj_pages_take(void* a, int n, int* out) {
    Allocator* al = (Allocator*)a;
    if (n < 0) { al->error = "cannot take " + std::to_string(n) + " pages"; return CJ_BOOKS_ERROR; }
    return al->take(n, out) ? 1 : 0;
}
CJ_EXPORT int cj_pages_give_back(void* a, const int* pages, int n) { return ((Allocator*)a)->give_back(pages, n) ? 0 : CJ_BOOKS_ERROR; }
CJ_EXPORT int cj_pages_check(void* a) { return ((Allocator*)a)->check() ? 0 : CJ_BOOKS_ERROR; }

// ---- the books ---------------------------------------------------------------------------------
CJ_EXPORT void* cj_books_create(int n_groups, const int* windows, const int* num_pages, int page_tokens, int max_seqs,
                                int max_tokens_per_seq) {
    if (n_groups < 0 || page_tokens < 1 || max_seqs < 0 || max_tokens_per_seq < 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (num_pages[g] < 0) return nullptr;
    Books* b = new Books();
    b->page_tokens = page_tokens;
    b->max_seqs = max_seqs;
    b->max_tokens = max_tokens_per_seq;
    b->width = (max_tokens_per_seq + page_tokens - 1) / page_tokens;
    b->groups.reserve((size_t)n_groups);
    for (int g = 0; g < n_groups; ++g) b->groups.emplace_back(windows[g], num_pages[g], max_seqs, b->width);
    b->length.assign((size_t)max_seqs, 0);
    b->live.assign((size_t)max_seqs, 0);
    for (int s = max_seqs - 1; s >= 0; --s) b->free_slots.push_back(s);
    return b;
}
CJ_EXPORT void cj_books_destroy(void* h) { delete B(h); }
CJ_EXPORT const char* cj_books_error(void* h) { return B(h)->error.c_str(); }

// raw views (the arrays never move while the books live)
CJ_EXPORT int64_t* cj_books_length(void* h) { return B(h)->length.data(); }
CJ_EXPORT uint8_t* cj_books_live(void* h) { return B(h)->live.data(); }
CJ_EXPORT int32_t* cj_books_table(void* h, int g) { return B(h)->groups[(size_t)g].table.data(); }
CJ_EXPORT int64_t* cj_books_first_live(void* h, int g) { return B(h)->groups[(size_t)g].first_live.data(); }
CJ_EXPORT int64_t* cj_books_next_page(void* h, int g) { return B(h)->groups[(size_t)g].next_page.data(); }
CJ_EXPORT int cj_books_width(void* h) { return B(h)->width; }
CJ_EXPORT int cj_books_free_slots(void* h) { return (int)B(h)->free_slots.size(); }
CJ_EXPORT int cj_books_free_count(void* h, int g) { return B(h)->groups[(size_t)g].alloc.free_count(); }

// a free slot for a new request (length 0), or -2 when all are taken
CJ_EXPORT int cj_books_admit(void* h) {
    Books* b = B(h);
    if (b->free_slots.empty()) return -2;
    int s = b->free_slots.back();
    b->free_slots.pop_back();
    b->live[(size_t)s] = 1;
    b->length[(size_t)s] = 0;
    return s;
}

// gives back everything the request holds; the slot is free again
CJ_EXPORT int cj_books_release(void* h, int slot) {
    Books* b = B(h);
    if (!b->need_live(slot)) return CJ_BOOKS_ERROR;
    for (Group& g : b->groups)
        if (!b->release_group(g, slot)) return CJ_BOOKS_ERROR;
    b->length[(size_t)slot] = 0;
    b->live[(size_t)slot] = 0;
    b->free_slots.push_back(slot);
    return 0;
}

// new pages per group that appending n_new tokens would draw
CJ_EXPORT int cj_books_pages_needed(void* h, int slot, int n_new, int* out) {
    Books* b = B(h);
    if (!b->need_live(slot)) return CJ_BOOKS_ERROR;
    for (size_t g = 0; g < b->groups.size(); ++g) out[g] = (int)b->needed(b->groups[g], slot, b->length[(size_t)slot], n_new);
    return 0;
}

// pages for positions [length, length + n_new): 1 reserved, 0 not enough pages (nothing changed)
CJ_EXPORT int cj_books_reserve(void* h, int slot, int n_new) {
    Books* b = B(h);
    if (!b->need_live(slot)) return CJ_BOOKS_ERROR;
    int64_t L = b->length[(size_t)slot];
    if (L + n_new > b->max_tokens) {
        b->error = "request in slot " + std::to_string(slot) + " would reach " + std::to_string(L + n_new) +
                   " tokens; the limit is " + std::to_string(b->max_tokens);
        return CJ_BOOKS_ERROR;
    }
    for (Group& g : b->groups)
        if (b->needed(g, slot, L, n_new) > g.alloc.free_count()) return 0;
    for (Group& g : b->groups)
        if (!b->grow(g, slot, (int)b->needed(g, slot, L, n_new))) return CJ_BOOKS_ERROR;
    return 1;
}

// the same for every request of a step at once, all or nothing over the whole step:
// 1 reserved, 0 not enough pages (nothing changed; needs[g] = pages the step wants of group g)
CJ_EXPORT int cj_books_reserve_step(void* h, const int* slots, const int* n_new, int n, int* needs) {
    Books* b = B(h);
    const size_t G = b->groups.size();
    for (size_t g = 0; g < G; ++g) needs[g] = 0;
    for (int i = 0; i < n; ++i) {
        if (!b->need_live(slots[i])) return CJ_BOOKS_ERROR;
        int64_t L = b->length[(size_t)slots[i]];
        if (n_new[i] < 0 || L + n_new[i] > b->max_tokens) {
            b->error = "request in slot " + std::to_string(slots[i]) + " would reach " + std::to_string(L + n_new[i]) +
                       " tokens; the limit is " + std::to_string(b->max_tokens);
            return CJ_BOOKS_ERROR;
        }
        for (size_t g = 0; g < G; ++g) needs[g] += (int)b->needed(b->groups[g], slots[i], L, n_new[i]);
    }
    for (size_t g = 0; g < G; ++g)
        if (needs[g] > b->groups[g].alloc.free_count()) return 0;
    for (int i = 0; i < n; ++i)
        for (Group& g : b->groups)
            if (!b->grow(g, slots[i], (int)b->needed(g, slots[i], b->length[(size_t)slots[i]], n_new[i]))) return CJ_BOOKS_ERROR;
    return 1;
}

// the step that wrote n_new tokens is launched: the length advances, pages behind a window go back
CJ_EXPORT int cj_books_commit(void* h, int slot, int n_new) {
    Books* b = B(h);
    if (!b->need_live(slot)) return CJ_BOOKS_ERROR;
    int64_t L = b->length[(size_t)slot] + n_new;
    for (Group& g : b->groups)
        if (b->pages_for(L) > g.next_page[(size_t)slot]) {
            b->error = "slot " + std::to_string(slot) + ": committed " + std::to_string(L) + " tokens without reserved pages";
            return CJ_BOOKS_ERROR;
        }
    b->length[(size_t)slot] = L;
    for (Group& g : b->groups)
        if (!b->trim_window(g, slot, L)) return CJ_BOOKS_ERROR;
    return 0;
}

// one token for each of several requests (a decode step): prior[i] = the length before the new
// token; 1 reserved, 0 not enough pages (nothing changed)
CJ_EXPORT int cj_books_reserve_one_each(void* h, const int* slots, int n, int64_t* prior) {
    Books* b = B(h);
    for (int i = 0; i < n; ++i) {
        if (!b->need_live(slots[i])) return CJ_BOOKS_ERROR;
        prior[i] = b->length[(size_t)slots[i]];
        if (prior[i] + 1 > b->max_tokens) {
            b->error = "request in slot " + std::to_string(slots[i]) + " would reach " + std::to_string(prior[i] + 1) +
                       " tokens; the limit is " + std::to_string(b->max_tokens);
            return CJ_BOOKS_ERROR;
        }
    }
    for (Group& g : b->groups) {
        int short_of = 0;
        for (int i = 0; i < n; ++i) short_of += b->pages_for(prior[i] + 1) > g.next_page[(size_t)slots[i]];
        if (short_of > g.alloc.free_count()) return 0;
    }
    for (Group& g : b->groups)
        for (int i = 0; i < n; ++i)
            if (b->pages_for(prior[i] + 1) > g.next_page[(size_t)slots[i]])
                if (!b->grow(g, slots[i], 1)) return CJ_BOOKS_ERROR;
    return 1;
}

CJ_EXPORT int cj_books_commit_one_each(void* h, const int* slots, int n) {
    Books* b = B(h);
    for (int i = 0; i < n; ++i) {
        if (!b->need_live(slots[i])) return CJ_BOOKS_ERROR;
        int64_t L = b->length[(size_t)slots[i]] + 1;
        for (Group& g : b->groups)
            if (b->pages_for(L) > g.next_page[(size_t)slots[i]]) {
                b->error = "a token was committed without reserved pages";
                return CJ_BOOKS_ERROR;
            }
    }
    for (int i = 0; i < n; ++i) {
        int64_t L = ++b->length[(size_t)slots[i]];
        for (Group& g : b->groups)
            if (!b->trim_window(g, slots[i], L)) return CJ_BOOKS_ERROR;
    }
    return 0;
}

// columns that cover every page the given slots have ever been given
CJ_EXPORT int cj_books_table_width(void* h, const int* slots, int n) {
    Books* b = B(h);
    int64_t w = 1;
    for (const Group& g : b->groups)
        for (int i = 0; i < n; ++i)
            if (slots[i] >= 0 && slots[i] < b->max_seqs && g.next_page[(size_t)slots[i]] > w) w = g.next_page[(size_t)slots[i]];
    return (int)w;
}

// The metadata of a step, laid into one int32 buffer:
//   tokens | positions | row -> request | request starts | prior lengths | slots | wanted rows |
//   one slab [requests, width] of block-table rows per group.
// n_tokens[i] tokens of request i follow one another in `tokens`; wants holds, request after
// request, n_want[i] indices into that request's tokens.  The caller has checked the tokens and
// the wanted indices and has reserved the step's pages.
// pad_requests > n lays the per-request arrays out for that many requests: the ones beyond n
// bring no rows (they start where the rows end, hold nothing, slot -1, a table row of -1), so
// that a step's buffer has the same shape whatever the number of its requests; pad_wanted > W
// fills the wanted rows up with row 0 (their logits are computed and thrown away).  Returns the
// int32 values written, or CJ_BOOKS_ERROR when `out` (capacity out_len) is too small or a slot
// holds nothing.
CJ_EXPORT long long cj_books_layout_step(void* h, int n, const int* slots, const int* n_tokens, const int* tokens,
                                         const int* n_want, const int* wants, int width, int pad_requests, int pad_wanted,
                                         int32_t* out, long long out_len) {
    Books* b = B(h);
    long long T = 0, W = 0;
    for (int i = 0; i < n; ++i) {
        if (!b->need_live(slots[i])) return CJ_BOOKS_ERROR;
        T += n_tokens[i];
        W += n_want[i];
    }
    if (width < 1 || width > b->width) { b->error = "block-table width " + std::to_string(width) + " is out of range"; return CJ_BOOKS_ERROR; }
    const long long R = pad_requests > n ? pad_requests : n;
    const long long Wp = pad_wanted > W ? pad_wanted : W;
    const long long G = (long long)b->groups.size();
    const long long total = 3 * T + (R + 1) + 2LL * R + Wp + G * R * width;
    if (total > out_len) { b->error = "the step's metadata needs " + std::to_string(total) + " values"; return CJ_BOOKS_ERROR; }
    int32_t* tok = out;
    int32_t* pos = tok + T;
    int32_t* row_req = pos + T;
    int32_t* req_start = row_req + T;
    int32_t* req_prior = req_start + R + 1;
    int32_t* req_slot = req_prior + R;
    int32_t* want_rows = req_slot + R;
    int32_t* tables = want_rows + Wp;
    long long row = 0, wi = 0;
    for (int i = 0; i < n; ++i) {
        const int64_t prior = b->length[(size_t)slots[i]];
        req_start[i] = (int32_t)row;
        req_prior[i] = (int32_t)prior;
        req_slot[i] = slots[i];
        for (int j = 0; j < n_tokens[i]; ++j) {
            tok[row + j] = tokens[row + j];
            pos[row + j] = (int32_t)(prior + j);
            row_req[row + j] = i;
        }
        for (int j = 0; j < n_want[i]; ++j) want_rows[wi + j] = (int32_t)(row + wants[wi + j]);
        wi += n_want[i];
        row += n_tokens[i];
    }
    for (long long i = n; i < R; ++i) {
        req_start[i] = (int32_t)row;
        req_prior[i] = 0;
        req_slot[i] = -1;
    }
    req_start[R] = (int32_t)row;
    for (long long j = W; j < Wp; ++j) want_rows[j] = 0;
    for (long long g = 0; g < G; ++g) {
        for (int i = 0; i < n; ++i)
            memcpy(tables + (g * R + i) * width, b->groups[(size_t)g].table.data() + (size_t)slots[i] * b->width,
                   (size_t)width * sizeof(int32_t));
        for (long long i = n; i < R; ++i)
            for (int j = 0; j < width; ++j) tables[(g * R + i) * width + j] = -1;
    }
    return total;
}

// invariants: no page lost, held twice or freed twice; tables agree with owners
CJ_EXPORT int cj_books_check(void* h) {
    Books* b = B(h);
    for (Group& g : b->groups) {
        if (!g.alloc.check()) { b->error = g.alloc.error; return CJ_BOOKS_ERROR; }
        std::vector<int> owner((size_t)g.alloc.num_pages, -1);
        int owned = 0;
        for (int s = 0; s < b->max_seqs; ++s) {
            const int32_t* row = g.table.data() + (size_t)s * b->width;
            const int64_t first = g.first_live[(size_t)s], nxt = g.next_page[(size_t)s];
            if (!b->live[(size_t)s] && nxt > first) { b->error = "free slot " + std::to_string(s) + " still holds pages"; return CJ_BOOKS_ERROR; }
            for (int64_t j = 0; j < b->width; ++j) {
                const bool in_range = j >= first && j < nxt;
                if ((row[j] >= 0) != in_range) {
                    b->error = "slot " + std::to_string(s) + ": table entry " + std::to_string(j) + " disagrees with the live range";
                    return CJ_BOOKS_ERROR;
                }
                if (!in_range) continue;
                const int p = row[j];
                if (p >= g.alloc.num_pages) { b->error = "slot " + std::to_string(s) + " names page " + std::to_string(p) + ", which does not exist"; return CJ_BOOKS_ERROR; }
                if (owner[(size_t)p] >= 0) {
                    b->error = "page " + std::to_string(p) + " is held by slots " + std::to_string(owner[(size_t)p]) + " and " + std::to_string(s);
                    return CJ_BOOKS_ERROR;
                }
                if (!g.alloc.held[(size_t)p]) { b->error = "page " + std::to_string(p) + " is in a table and on the free list"; return CJ_BOOKS_ERROR; }
                owner[(size_t)p] = s;
                ++owned;
            }
        }
        const int out = g.alloc.num_pages - g.alloc.free_count();
        if (owned != out) { b->error = std::to_string(out) + " pages are out, " + std::to_string(owned) + " are in tables"; return CJ_BOOKS_ERROR; }
    }
    return 0;
}
