// The cache manager's core, native: page pools, request state slots, block tables per
// request and cache group, the reservation ledger, and the table rows in the form that
// goes to the device.  `crucible_b200/cache/` wraps it; nothing here touches a device.
//
// What it mirrors in the reference: the page allocator, a stack of free ids with an
// in-use flag per page that rejects a double free or an id out of range
// (`engine/src/paged.rs:65-144`); growth that is all-or-nothing with rollback
// (`engine/src/paged.rs:199-217`); pages given back when a request ends
// (`engine/src/runtime.rs:896-898`); the logical reservation of a request's whole
// lifetime at admission (`engine/src/prefill.rs:160-206`); and the refusal of a batch
// whose tables are not sound before anything is written (`engine/src/gpu_model.rs:2809-2934`).
// Beyond the reference: several groups of layers with pools of their own, windowed groups
// that give pages back as the window passes them, and a second ledger (which request's
// table names a page) that is kept apart from the allocator's free stack, so that a fault
// of the allocator is seen before two requests write the same keys.
//
// A request is known here by its state slot (0 .. n_slots-1): live requests and slots
// correspond one to one.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#define CB_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

enum Code {
    OK = 0,
    PAGES_EXHAUSTED = 1,
    SLOTS_EXHAUSTED = 2,
    NOT_LIVE = 3,
    TOO_LONG = 4,
    ALIASED = 5,
    DOUBLE_FREE = 6,
    OUT_OF_RANGE = 7,
    BROKEN = 8,
    BAD_ARGUMENT = 9,
};

const int RELEASED = -1;

// Ids 0..n-1, each handed out once and taken back once.  The first id handed out is 0
// (`paged.rs:75-77`); an id given back is the next one handed out.
struct Stack {
    int n;
    std::vector<int> free_;
    std::vector<uint8_t> in_use;

    explicit Stack(int n_) : n(n_), free_(n_), in_use(n_, 0) {
        for (int i = 0; i < n_; ++i) free_[i] = n_ - 1 - i;
    }
    int n_free() const { return (int)free_.size(); }
    int take() {
        if (free_.empty()) return -1;
        const int id = free_.back();
        free_.pop_back();
        if (id >= 0 && id < n) in_use[id] = 1;
        return id;
    }
    int give(int id) {
        if (id < 0 || id >= n) return OUT_OF_RANGE;
        if (!in_use[id]) return DOUBLE_FREE;
        in_use[id] = 0;
        free_.push_back(id);
        return OK;
    }
    // Puts back an id that `take` just returned, whatever the flags say: a rollback
    // leaves the stack exactly as it found it, also when the stack itself is at fault.
    void untake(int id) {
        if (id >= 0 && id < n) in_use[id] = 0;
        free_.push_back(id);
    }
};

struct Group {
    int page_tokens;
    int window;          // < 0: every token is kept
    int stride;          // ints of a device table row; 0: no rows are kept
    int null_page;       // what a row holds in place of a page given back early
    long reserved;
    Stack pool;
    std::vector<int32_t> rows;    // n_slots * stride
    std::vector<int32_t> owner;   // per page: the slot whose table names it, or -1

    Group(int pt, int w, int n_pages, int st, int np, int n_slots)
        : page_tokens(pt), window(w), stride(st), null_page(np), reserved(0), pool(n_pages),
          rows((size_t)n_slots * st, 0), owner(n_pages, -1) {}
};

struct Request {
    bool live = false;
    long length = 0;
    std::vector<std::vector<int>> tables;   // per group: logical block -> page
    std::vector<int> first_live;            // per group: first block still held
    std::vector<long> reserved;             // per group: pages reserved logically
};

struct Cache {
    std::vector<Group> groups;
    Stack slots;
    std::vector<Request> requests;

    explicit Cache(int n_slots) : slots(n_slots), requests(n_slots) {}
};

inline long ceil_div(long a, long b) { return (a + b - 1) / b; }

void say(char* err, int err_len, const char* text) {
    if (err && err_len > 0) snprintf(err, err_len, "%s", text);
}

long pages_for(const Group& g, long n_tokens, long max_step) {
    const long full = ceil_div(n_tokens, g.page_tokens);
    if (g.window < 0) return full;
    long step = n_tokens;
    if (max_step >= 0) {
        step = max_step < n_tokens ? max_step : n_tokens;
        if (step < 1) step = 1;
    }
    // the window's keys before the step's first token, the step itself, and one page
    // for misalignment at either end
    const long live = ceil_div(g.window - 1 + step, g.page_tokens) + 1;
    return full < live ? full : live;
}

int32_t* row_of(Group& g, int slot) { return g.rows.data() + (size_t)slot * g.stride; }

// Gives back one held page of a table: to the pool, and out of the ledger.
int give_back(Group& g, int slot, int page) {
    const int code = g.pool.give(page);
    if (code == OK && g.owner[page] == slot) g.owner[page] = -1;
    return code;
}

int release_passed(Cache& c, int slot) {
    Request& r = c.requests[slot];
    int result = OK;
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group& g = c.groups[gi];
        if (g.window < 0) continue;
        // the next token sits at position `length` and reads keys from
        // length - window + 1 on; blocks wholly below that are done
        long first_needed = r.length - g.window + 1;
        if (first_needed < 0) first_needed = 0;
        long upto = first_needed / g.page_tokens;
        std::vector<int>& table = r.tables[gi];
        if (upto > (long)table.size()) upto = (long)table.size();
        for (long b = r.first_live[gi]; b < upto; ++b) {
            if (table[b] != RELEASED) {
                const int code = give_back(g, slot, table[b]);
                if (code != OK && result == OK) result = code;
            }
            table[b] = RELEASED;
            if (g.stride) row_of(g, slot)[b] = g.null_page;
        }
        if (upto > r.first_live[gi]) r.first_live[gi] = (int)upto;
    }
    return result;
}

int extend(Cache& c, int slot, long n_new, char* err, int err_len) {
    if (slot < 0 || slot >= c.slots.n || !c.requests[slot].live) {
        say(err, err_len, "the request is not live");
        return NOT_LIVE;
    }
    if (n_new <= 0) {
        say(err, err_len, "extend needs a positive token count");
        return BAD_ARGUMENT;
    }
    Request& r = c.requests[slot];
    int code = release_passed(c, slot);
    if (code != OK) {
        say(err, err_len, "a page that the window has passed could not be given back "
                          "(double free or out of range)");
        return code;
    }
    const long target = r.length + n_new;
    const size_t n_groups = c.groups.size();
    std::vector<size_t> before(n_groups);
    for (size_t gi = 0; gi < n_groups; ++gi) before[gi] = r.tables[gi].size();
    char text[200];
    bool page_at_fault = false;      // the last page on a table was taken but must not be kept
    for (size_t gi = 0; gi < n_groups && code == OK; ++gi) {
        Group& g = c.groups[gi];
        const long needed = ceil_div(target, g.page_tokens);
        if (g.stride && needed > g.stride) {
            snprintf(text, sizeof text, "%ld tokens need %ld table entries in cache group %d; "
                     "a table row has %d", target, needed, (int)gi, g.stride);
            say(err, err_len, text);
            code = TOO_LONG;
            break;
        }
        std::vector<int>& table = r.tables[gi];
        while ((long)table.size() < needed) {
            const int page = g.pool.take();
            if (page < 0) {
                snprintf(text, sizeof text, "kv page pool exhausted: all %d pages (%ld tokens) "
                         "of cache group %d are in use", g.pool.n, (long)g.pool.n * g.page_tokens,
                         (int)gi);
                say(err, err_len, text);
                code = PAGES_EXHAUSTED;
                break;
            }
            table.push_back(page);          // on the table first, so that the rollback finds it
            if (g.owner[page] != -1) {
                snprintf(text, sizeof text, "page %d of cache group %d is named by the table of "
                         "another live request (or twice): two requests would write the same "
                         "keys", page, (int)gi);
                say(err, err_len, text);
                code = ALIASED;
                page_at_fault = true;
                break;
            }
            g.owner[page] = slot;
        }
    }
    if (code != OK) {
        // Back to where the call began, last page first, so that the free stacks read as
        // before.  Groups are walked in reverse: the first page met is the one at fault, if
        // there is one, and that page never entered the ledger under this request.
        for (size_t gi = n_groups; gi-- > 0;) {
            Group& g = c.groups[gi];
            std::vector<int>& table = r.tables[gi];
            while (table.size() > before[gi]) {
                const int page = table.back();
                table.pop_back();
                if (page_at_fault)
                    page_at_fault = false;
                else if (g.owner[page] == slot)
                    g.owner[page] = -1;
                g.pool.untake(page);
            }
        }
        return code;
    }
    for (size_t gi = 0; gi < n_groups; ++gi) {
        Group& g = c.groups[gi];
        if (!g.stride) continue;
        int32_t* row = row_of(g, slot);
        const std::vector<int>& table = r.tables[gi];
        for (size_t b = before[gi]; b < table.size(); ++b) row[b] = table[b];
    }
    r.length = target;
    return OK;
}

int shrink(Cache& c, int slot, long n) {
    if (slot < 0 || slot >= c.slots.n || !c.requests[slot].live) return NOT_LIVE;
    Request& r = c.requests[slot];
    if (n < 0 || n > r.length) return BAD_ARGUMENT;
    r.length -= n;
    int result = OK;
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group& g = c.groups[gi];
        const long needed = ceil_div(r.length, g.page_tokens);
        std::vector<int>& table = r.tables[gi];
        while ((long)table.size() > needed) {
            const int page = table.back();
            table.pop_back();
            if (g.stride) row_of(g, slot)[table.size()] = 0;
            if (page == RELEASED) continue;
            const int code = give_back(g, slot, page);
            if (code != OK && result == OK) result = code;
        }
        if (r.first_live[gi] > (int)table.size()) r.first_live[gi] = (int)table.size();
    }
    return result;
}

int remove(Cache& c, int slot) {
    if (slot < 0 || slot >= c.slots.n || !c.requests[slot].live) return NOT_LIVE;
    Request& r = c.requests[slot];
    int result = OK;
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group& g = c.groups[gi];
        std::vector<int>& table = r.tables[gi];
        // last page first: the pool is a stack, so the next request takes these pages in
        // the order this one held them, and runs of consecutive pages (which the attention
        // kernels fetch with one copy per tile instead of one per page) survive reuse
        for (size_t b = table.size(); b-- > 0;) {
            if (table[b] == RELEASED) continue;
            const int code = give_back(g, slot, table[b]);
            if (code != OK && result == OK) result = code;
        }
        if (g.stride) memset(row_of(g, slot), 0, sizeof(int32_t) * (size_t)g.stride);
        g.reserved -= r.reserved[gi];
        table.clear();
    }
    const int code = c.slots.give(slot);
    if (code != OK && result == OK) result = code;
    r = Request();
    return result;
}

}  // namespace

// ---- a stack of ids by itself (the pools' own type, for use and tests alone) ----------------

CB_EXPORT void* cb_stack_create(int n) { return n > 0 ? new Stack(n) : nullptr; }
CB_EXPORT void cb_stack_destroy(void* s) { delete static_cast<Stack*>(s); }
CB_EXPORT int cb_stack_take(void* s) { return static_cast<Stack*>(s)->take(); }
CB_EXPORT int cb_stack_give(void* s, int id) { return static_cast<Stack*>(s)->give(id); }
CB_EXPORT int cb_stack_free(void* s) { return static_cast<Stack*>(s)->n_free(); }
CB_EXPORT int cb_stack_in_use(void* s, int id) {
    Stack* st = static_cast<Stack*>(s);
    return (id >= 0 && id < st->n) ? st->in_use[id] : -1;
}

// ---- the manager --------------------------------------------------------------------------------

// windows[g] < 0: the group keeps every token.  strides: ints of a device table row per
// group (null or 0: no rows kept); null_pages: what a row holds for a page given back early.
CB_EXPORT void* cb_cache_create(int n_groups, const int32_t* page_tokens, const int32_t* windows,
                                const int32_t* n_pages, int n_slots, const int32_t* strides,
                                const int32_t* null_pages) {
    if (n_groups < 0 || n_slots <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (page_tokens[g] <= 0 || n_pages[g] <= 0 || (strides && strides[g] < 0)) return nullptr;
    Cache* c = new Cache(n_slots);
    c->groups.reserve(n_groups);
    for (int g = 0; g < n_groups; ++g)
        c->groups.emplace_back(page_tokens[g], windows[g], n_pages[g], strides ? strides[g] : 0,
                               null_pages ? null_pages[g] : 0, n_slots);
    return c;
}

CB_EXPORT void cb_cache_destroy(void* h) { delete static_cast<Cache*>(h); }

// The pool of group g, or the slot pool for g < 0, as a stack for the cb_stack_* calls.
// It lives as long as the manager.
CB_EXPORT void* cb_cache_stack(void* h, int g) {
    Cache* c = static_cast<Cache*>(h);
    if (g < 0) return &c->slots;
    return g < (int)c->groups.size() ? &c->groups[g].pool : nullptr;
}

CB_EXPORT long cb_cache_pages_for(void* h, int g, long n_tokens, long max_step) {
    return pages_for(static_cast<Cache*>(h)->groups[g], n_tokens, max_step);
}

// Whether a request of `lifetime` tokens could be admitted now (a slot free, and its pages
// unreserved in every group); with `ignore_reservations`, whether it fits an empty cache.
CB_EXPORT int cb_cache_fits(void* h, long lifetime, long max_step, int ignore_reservations) {
    Cache* c = static_cast<Cache*>(h);
    if (!ignore_reservations && c->slots.n_free() == 0) return 0;
    for (const Group& g : c->groups) {
        const long room = g.pool.n - (ignore_reservations ? 0 : g.reserved);
        if (pages_for(g, lifetime, max_step) > room) return 0;
    }
    return 1;
}

// Registers a request: takes a slot and, with lifetime >= 0, reserves that many tokens'
// pages in every group.  A refusal changes nothing.
CB_EXPORT int cb_cache_add(void* h, long lifetime, long max_step, int32_t* slot_out, char* err,
                           int err_len) {
    Cache* c = static_cast<Cache*>(h);
    const size_t n_groups = c->groups.size();
    std::vector<long> reserved(n_groups, 0);
    if (lifetime >= 0) {
        for (size_t gi = 0; gi < n_groups; ++gi) {
            const Group& g = c->groups[gi];
            const long need = pages_for(g, lifetime, max_step);
            if (need > g.pool.n - g.reserved) {
                char text[200];
                snprintf(text, sizeof text, "needs %ld pages in cache group %d; %ld of %d are "
                         "unreserved", need, (int)gi, g.pool.n - g.reserved, g.pool.n);
                say(err, err_len, text);
                return PAGES_EXHAUSTED;
            }
            reserved[gi] = need;
        }
    }
    const int slot = c->slots.take();
    if (slot < 0) {
        char text[100];
        snprintf(text, sizeof text, "all %d request state slots are in use", c->slots.n);
        say(err, err_len, text);
        return SLOTS_EXHAUSTED;
    }
    Request& r = c->requests[slot];
    r = Request();
    r.live = true;
    r.tables.assign(n_groups, std::vector<int>());
    r.first_live.assign(n_groups, 0);
    r.reserved = reserved;
    for (size_t gi = 0; gi < n_groups; ++gi) c->groups[gi].reserved += reserved[gi];
    *slot_out = slot;
    return OK;
}

// Room for n_new more tokens of the request in every group, all or nothing.  Pages that a
// window has passed go back first (that part stays done when the growth is refused).
CB_EXPORT int cb_cache_extend(void* h, int slot, long n_new, char* err, int err_len) {
    return extend(*static_cast<Cache*>(h), slot, n_new, err, err_len);
}

// Takes the last n tokens of the request back, with the pages that only they needed.
CB_EXPORT int cb_cache_shrink(void* h, int slot, long n) {
    return shrink(*static_cast<Cache*>(h), slot, n);
}

CB_EXPORT int cb_cache_remove(void* h, int slot) { return remove(*static_cast<Cache*>(h), slot); }

// One step's growth: every request i (by slot) takes counts[i] more tokens, or none does.
// first_pos[i]: the tokens the request held before.  rows (may be null): n_groups * n_req
// addresses, group-major, of the requests' device table rows.  max_tokens: the most a
// request may hold (< 0: no limit).  On failure `bad` is the index of the request at fault.
CB_EXPORT int cb_cache_step(void* h, int n_req, const int32_t* slots, const int32_t* counts,
                            long max_tokens, int32_t* first_pos, const int32_t** rows,
                            int32_t* bad, char* err, int err_len) {
    Cache& c = *static_cast<Cache*>(h);
    int code = OK, done = 0;
    for (; done < n_req; ++done) {
        const int slot = slots[done];
        if (slot < 0 || slot >= c.slots.n || !c.requests[slot].live) {
            say(err, err_len, "the request is not live");
            code = NOT_LIVE;
            break;
        }
        const long held = c.requests[slot].length;
        if (max_tokens >= 0 && held + counts[done] > max_tokens) {
            char text[160];
            snprintf(text, sizeof text, "would hold %ld tokens; the model's context is %ld",
                     held + counts[done], max_tokens);
            say(err, err_len, text);
            code = TOO_LONG;
            break;
        }
        first_pos[done] = (int32_t)held;
        code = extend(c, slot, counts[done], err, err_len);
        if (code != OK) break;
    }
    if (code != OK) {
        *bad = done;
        while (done-- > 0) shrink(c, slots[done], counts[done]);
        return code;
    }
    if (rows) {
        const int n_groups = (int)c.groups.size();
        for (int g = 0; g < n_groups; ++g)
            for (int i = 0; i < n_req; ++i)
                rows[(size_t)g * n_req + i] = c.groups[g].stride ? row_of(c.groups[g], slots[i])
                                                                 : nullptr;
    }
    return OK;
}

// Undoes a step that cb_cache_step accepted (something after it failed).
CB_EXPORT int cb_cache_unstep(void* h, int n_req, const int32_t* slots, const int32_t* counts) {
    Cache& c = *static_cast<Cache*>(h);
    int result = OK;
    for (int i = n_req; i-- > 0;) {
        const int code = shrink(c, slots[i], counts[i]);
        if (code != OK && result == OK) result = code;
    }
    return result;
}

// ---- views ----------------------------------------------------------------------------------------

CB_EXPORT int cb_cache_is_live(void* h, int slot) {
    Cache* c = static_cast<Cache*>(h);
    return slot >= 0 && slot < c->slots.n && c->requests[slot].live;
}

CB_EXPORT long cb_cache_length(void* h, int slot) {
    return static_cast<Cache*>(h)->requests[slot].length;
}

CB_EXPORT int cb_cache_table_len(void* h, int slot, int g) {
    return (int)static_cast<Cache*>(h)->requests[slot].tables[g].size();
}

CB_EXPORT void cb_cache_table_copy(void* h, int slot, int g, int32_t* out) {
    const std::vector<int>& t = static_cast<Cache*>(h)->requests[slot].tables[g];
    for (size_t b = 0; b < t.size(); ++b) out[b] = t[b];
}

CB_EXPORT int cb_cache_held(void* h, int slot, int g) {
    int n = 0;
    for (int page : static_cast<Cache*>(h)->requests[slot].tables[g]) n += page != RELEASED;
    return n;
}

CB_EXPORT long cb_cache_reserved(void* h, int g) { return static_cast<Cache*>(h)->groups[g].reserved; }

CB_EXPORT const int32_t* cb_cache_row(void* h, int slot, int g) {
    Group& grp = static_cast<Cache*>(h)->groups[g];
    return grp.stride ? row_of(grp, slot) : nullptr;
}

// For tests of the checks below: writes a table entry behind the manager's back.
CB_EXPORT void cb_cache_poke(void* h, int slot, int g, int block, int page) {
    Cache* c = static_cast<Cache*>(h);
    c->requests[slot].tables[g][block] = page;
    if (c->groups[g].stride) row_of(c->groups[g], slot)[block] = page;
}

// The allocator against the tables: no page lost, held twice, or free while held.
// info: group, page, slot of the finding.
CB_EXPORT int cb_cache_check(void* h, int32_t* info, char* err, int err_len) {
    Cache& c = *static_cast<Cache*>(h);
    char text[200];
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        const Group& g = c.groups[gi];
        std::vector<uint8_t> seen(g.pool.n, 0);
        int n_seen = 0;
        for (int slot = 0; slot < c.slots.n; ++slot) {
            const Request& r = c.requests[slot];
            if (!r.live) continue;
            for (int page : r.tables[gi]) {
                if (page == RELEASED) continue;
                info[0] = (int)gi, info[1] = page, info[2] = slot;
                if (page < 0 || page >= g.pool.n) {
                    snprintf(text, sizeof text, "page %d of group %d is out of range", page, (int)gi);
                    say(err, err_len, text);
                    return OUT_OF_RANGE;
                }
                if (seen[page]) {
                    snprintf(text, sizeof text, "page %d of group %d is held twice", page, (int)gi);
                    say(err, err_len, text);
                    return BROKEN;
                }
                if (!g.pool.in_use[page]) {
                    snprintf(text, sizeof text, "page %d of group %d is held by a request but free",
                             page, (int)gi);
                    say(err, err_len, text);
                    return BROKEN;
                }
                seen[page] = 1;
                ++n_seen;
            }
        }
        const int used = g.pool.n - g.pool.n_free();
        if (n_seen != used) {
            info[0] = (int)gi, info[1] = -1, info[2] = -1;
            snprintf(text, sizeof text, "group %d: %d pages in use but %d held by requests",
                     (int)gi, used, n_seen);
            say(err, err_len, text);
            return BROKEN;
        }
    }
    return OK;
}

// The tables by themselves, all of them and not only the pages new to a step: every page
// in range, none named by two requests or twice by one, and the ledger agrees.
// info: group, page, the slot that names it, the slot that named it first.
CB_EXPORT int cb_cache_check_tables(void* h, int32_t* info, char* err, int err_len) {
    Cache& c = *static_cast<Cache*>(h);
    char text[200];
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        const Group& g = c.groups[gi];
        std::vector<int> first(g.pool.n, -1);
        for (int slot = 0; slot < c.slots.n; ++slot) {
            const Request& r = c.requests[slot];
            if (!r.live) continue;
            for (int page : r.tables[gi]) {
                if (page == RELEASED) continue;
                info[0] = (int)gi, info[1] = page, info[2] = slot, info[3] = -1;
                if (page < 0 || page >= g.pool.n) {
                    snprintf(text, sizeof text, "page %d of cache group %d is out of range", page,
                             (int)gi);
                    say(err, err_len, text);
                    return OUT_OF_RANGE;
                }
                if (first[page] != -1 || g.owner[page] != slot) {
                    info[3] = first[page] != -1 ? first[page] : g.owner[page];
                    snprintf(text, sizeof text, "page %d of cache group %d is named by the table "
                             "of another live request (or twice)", page, (int)gi);
                    say(err, err_len, text);
                    return ALIASED;
                }
                first[page] = slot;
            }
        }
    }
    return OK;
}
