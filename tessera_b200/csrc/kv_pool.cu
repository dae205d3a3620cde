// Host-side page pool behind the paged kept rows: tessera-kv's `Pool` restated
// (engine/ir/kv/src/pool.rs:71-449).  Holder counts per page (live and retained apart), lowest free
// page first, worst-case admission, copy-on-write of a shared partial page, oldest-retained-first
// eviction.  Every failing call leaves the pool untouched: checks come before any change.
#include <algorithm>
#include <optional>
#include <set>
#include <vector>

#include "tessera_b200_kv.h"
#include "ts_common.cuh"

namespace {

struct Run {
    uint64_t tag = 0;
    std::vector<uint32_t> pages;
    uint64_t rows = 0, worst = 0;
    uint64_t retired = 0;  // retirement number when retained, 0 when live
    bool retained() const { return retired != 0; }
};

struct Slot {
    uint32_t generation = 0;
    std::optional<Run> run;
};

}  // namespace

struct ts_kv_pool {
    uint64_t page = 1;
    std::vector<uint32_t> live, kept;  // holders per page
    std::set<uint32_t> free;
    std::vector<Slot> slots;
    uint64_t retirements = 0;
    uint64_t detail = 0;

    uint64_t span(uint64_t rows) const { return (rows + page - 1) / page; }
    uint32_t holders(uint32_t p) const { return live[p] + kept[p]; }

    // One if the next write lands in a shared page (pool.rs:345-349).
    uint64_t copies(uint64_t rows, const std::vector<uint32_t> &pages, size_t count) const {
        const bool partial = rows % page != 0;
        const bool shared = count > 0 && holders(pages[count - 1]) > 1;
        return partial && shared ? 1 : 0;
    }
    // Pages to reach the worst case, copies included (pool.rs:340-343).
    uint64_t need(const Run &r) const { return span(r.worst) - r.pages.size() + copies(r.rows, r.pages, r.pages.size()); }

    uint64_t spare() const {
        uint64_t reclaimable = 0;
        for (size_t p = 0; p < live.size(); p++) reclaimable += live[p] == 0 && kept[p] > 0;
        return free.size() + reclaimable;
    }
    uint64_t promised() const {
        uint64_t sum = 0;
        for (const Slot &s : slots)
            if (s.run && !s.run->retained()) sum += need(*s.run);
        return sum;
    }
    // Refuses unless every live run could still reach its worst case (pool.rs:351-357).
    bool fits(uint64_t want, uint64_t lost) {
        if (promised() + want + lost <= spare()) return true;
        detail = want;
        return false;
    }

    const Run *find(ts_kv_run id) const {
        if (id.at >= slots.size()) return nullptr;
        const Slot &s = slots[id.at];
        if (s.generation != id.generation || !s.run) return nullptr;
        return &*s.run;
    }
    Run &at(uint32_t i) { return *slots[i].run; }

    void unhold(uint32_t p, bool retained) {
        (retained ? kept[p] : live[p]) -= 1;
        if (holders(p) == 0) free.insert(p);
    }
    void end(uint32_t i) {
        Slot &s = slots[i];
        s.generation += 1;
        Run r = std::move(*s.run);
        s.run.reset();
        for (uint32_t p : r.pages) unhold(p, r.retained());
    }
    // The lowest free page, after evicting retained runs oldest first if needed (pool.rs:359-375).
    uint32_t take() {
        for (;;) {
            if (!free.empty()) {
                const uint32_t p = *free.begin();
                free.erase(free.begin());
                live[p] = 1;
                return p;
            }
            uint64_t oldest = ~0ull;
            uint32_t victim = 0;
            bool any = false;
            for (uint32_t i = 0; i < slots.size(); i++)
                if (slots[i].run && slots[i].run->retained() && slots[i].run->retired < oldest) {
                    oldest = slots[i].run->retired;
                    victim = i;
                    any = true;
                }
            if (!any) return 0xFFFFFFFFu;  // unreachable: the room check promised a page
            end(victim);
        }
    }
    ts_kv_run add(Run run) {
        uint32_t i = 0;
        while (i < slots.size() && slots[i].run) i++;
        if (i == slots.size()) slots.emplace_back();
        slots[i].run = std::move(run);
        return ts_kv_run{i, slots[i].generation};
    }

    bool consistent() const {
        std::vector<uint32_t> l(live.size(), 0), k(kept.size(), 0);
        for (const Slot &s : slots)
            if (s.run)
                for (uint32_t p : s.run->pages) (s.run->retained() ? k : l)[p] += 1;
        if (l != live || k != kept) return false;
        std::set<uint32_t> f;
        for (uint32_t p = 0; p < live.size(); p++)
            if (l[p] + k[p] == 0) f.insert(p);
        return f == free && promised() <= spare();
    }
};

#define KV_RUN(pool, id, name)                          \
    const Run *name = (pool)->find(id);                 \
    if (!name) return TS_KV_UNKNOWN

#define KV_LIVE(pool, id, name) \
    KV_RUN(pool, id, name);     \
    if (name->retained()) return TS_KV_RETAINED

#pragma GCC visibility push(default)
extern "C" {

ts_kv_pool *ts_kv_pool_new(uint32_t pages, uint32_t page_rows) {
    if (page_rows == 0) return nullptr;
    ts_kv_pool *p = new ts_kv_pool();
    p->page = page_rows;
    p->live.assign(pages, 0);
    p->kept.assign(pages, 0);
    for (uint32_t i = 0; i < pages; i++) p->free.insert(i);
    return p;
}

void ts_kv_pool_free(ts_kv_pool *pool) { delete pool; }
uint64_t ts_kv_last_detail(const ts_kv_pool *pool) { return pool ? pool->detail : 0; }

int ts_kv_reserve(ts_kv_pool *pool, uint64_t tag, uint64_t rows, uint64_t worst, ts_kv_run *out) {
    if (!pool || !out) return TS_KV_BAD_ARGUMENT;
    if (rows > worst) {
        pool->detail = worst;
        return TS_KV_PAST_WORST;
    }
    if (!pool->fits(pool->span(worst), 0)) return TS_KV_NO_ROOM;
    Run run;
    run.tag = tag;
    run.rows = rows;
    run.worst = worst;
    for (uint64_t i = 0; i < pool->span(rows); i++) run.pages.push_back(pool->take());
    *out = pool->add(std::move(run));
    return TS_KV_OK;
}

int ts_kv_fork(ts_kv_pool *pool, ts_kv_run source, uint64_t rows, uint64_t worst, ts_kv_run *out) {
    if (!pool || !out) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, source, src);
    if (rows > src->rows) {
        pool->detail = src->rows;
        return TS_KV_PAST_SOURCE;
    }
    if (rows > worst) {
        pool->detail = worst;
        return TS_KV_PAST_WORST;
    }
    const size_t shared = pool->span(rows);
    uint64_t lost = 0;
    for (size_t i = 0; i < shared; i++) lost += pool->live[src->pages[i]] == 0;
    // A shared partial page costs each live holder one copy (pool.rs:169-176).
    const bool mine = rows % pool->page != 0;
    const bool theirs = !src->retained() && src->rows % pool->page != 0 && shared == src->pages.size() && shared > 0 &&
                        pool->holders(src->pages[shared - 1]) == 1;
    const uint64_t want = pool->span(worst) - shared + (mine ? 1 : 0) + (theirs ? 1 : 0);
    if (!pool->fits(want, lost)) return TS_KV_NO_ROOM;
    Run run;
    run.tag = src->tag;
    run.pages.assign(src->pages.begin(), src->pages.begin() + shared);
    run.rows = rows;
    run.worst = worst;
    for (uint32_t p : run.pages) pool->live[p] += 1;
    *out = pool->add(std::move(run));
    return TS_KV_OK;
}

int ts_kv_grow(ts_kv_pool *pool, ts_kv_run id, uint64_t rows, ts_kv_copy *copies, uint32_t capacity,
               uint32_t *n_copies) {
    if (!pool || !n_copies) return TS_KV_BAD_ARGUMENT;
    KV_LIVE(pool, id, found);
    *n_copies = 0;
    if (rows > found->worst) {
        pool->detail = found->worst;
        return TS_KV_PAST_WORST;
    }
    if (rows <= found->rows) return TS_KV_OK;
    Run &r = pool->at(id.at);
    const uint64_t written = r.rows % pool->page;
    if (!r.pages.empty() && written > 0 && pool->holders(r.pages.back()) > 1) {
        if (capacity < 1 || !copies) return TS_KV_BAD_ARGUMENT;
        const uint32_t from = r.pages.back(), to = pool->take();
        pool->live[from] -= 1;
        r.pages.back() = to;
        copies[0] = ts_kv_copy{from, to, (uint32_t)written};
        *n_copies = 1;
    }
    while (r.pages.size() < pool->span(rows)) r.pages.push_back(pool->take());
    r.rows = rows;
    return TS_KV_OK;
}

int ts_kv_truncate(ts_kv_pool *pool, ts_kv_run id, uint64_t rows) {
    if (!pool) return TS_KV_BAD_ARGUMENT;
    KV_LIVE(pool, id, found);
    if (rows >= found->rows) return TS_KV_OK;
    const size_t keep = pool->span(rows);
    // The run may grow back; shared pages stay held (pool.rs:232-239).
    const uint64_t regrow = found->pages.size() - keep + pool->copies(rows, found->pages, keep);
    uint64_t freed = 0;
    for (size_t i = keep; i < found->pages.size(); i++) freed += pool->live[found->pages[i]] == 1;
    const uint64_t owed = freed + pool->copies(found->rows, found->pages, found->pages.size());
    if (!pool->fits(regrow > owed ? regrow - owed : 0, 0)) return TS_KV_NO_ROOM;
    Run &r = pool->at(id.at);
    std::vector<uint32_t> dropped(r.pages.begin() + keep, r.pages.end());
    r.pages.resize(keep);
    r.rows = rows;
    for (uint32_t p : dropped) pool->unhold(p, false);
    return TS_KV_OK;
}

int ts_kv_retain(ts_kv_pool *pool, ts_kv_run id) {
    if (!pool) return TS_KV_BAD_ARGUMENT;
    KV_LIVE(pool, id, found);
    (void)found;
    Run &r = pool->at(id.at);
    r.retired = ++pool->retirements;
    for (uint32_t p : r.pages) {
        pool->live[p] -= 1;
        pool->kept[p] += 1;
    }
    return TS_KV_OK;
}

int ts_kv_adopt(ts_kv_pool *pool, ts_kv_run id, uint64_t rows, uint64_t worst, ts_kv_run *out) {
    if (!pool || !out) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, id, found);
    if (!found->retained()) return TS_KV_LIVE;
    if (rows > found->rows) {
        pool->detail = found->rows;
        return TS_KV_PAST_SOURCE;
    }
    if (rows > worst) {
        pool->detail = worst;
        return TS_KV_PAST_WORST;
    }
    const size_t keep = pool->span(rows);
    uint64_t lost = 0;
    for (size_t i = 0; i < keep; i++) lost += pool->live[found->pages[i]] == 0;
    const uint64_t want = pool->span(worst) - keep + pool->copies(rows, found->pages, keep);
    if (!pool->fits(want, lost)) return TS_KV_NO_ROOM;
    Run &r = pool->at(id.at);
    std::vector<uint32_t> dropped(r.pages.begin() + keep, r.pages.end());
    r.pages.resize(keep);
    for (uint32_t p : dropped) pool->unhold(p, true);
    r.rows = rows;
    r.worst = worst;
    r.retired = 0;
    for (uint32_t p : r.pages) {
        pool->kept[p] -= 1;
        pool->live[p] += 1;
    }
    pool->slots[id.at].generation += 1;  // the retained id is now stale
    *out = ts_kv_run{id.at, pool->slots[id.at].generation};
    return TS_KV_OK;
}

int ts_kv_release(ts_kv_pool *pool, ts_kv_run id) {
    if (!pool) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, id, found);
    (void)found;
    pool->end(id.at);
    return TS_KV_OK;
}

int ts_kv_pages(const ts_kv_pool *pool, ts_kv_run id, uint32_t *out, uint32_t capacity, uint32_t *count) {
    if (!pool || !count) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, id, r);
    *count = (uint32_t)r->pages.size();
    for (uint32_t i = 0; i < *count && i < capacity && out; i++) out[i] = r->pages[i];
    return TS_KV_OK;
}

int ts_kv_rows(const ts_kv_pool *pool, ts_kv_run id, uint64_t *rows) {
    if (!pool || !rows) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, id, r);
    *rows = r->rows;
    return TS_KV_OK;
}

int ts_kv_tag(const ts_kv_pool *pool, ts_kv_run id, uint64_t *tag) {
    if (!pool || !tag) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, id, r);
    *tag = r->tag;
    return TS_KV_OK;
}

uint64_t ts_kv_spare(const ts_kv_pool *pool) { return pool ? pool->spare() : 0; }
uint64_t ts_kv_promised(const ts_kv_pool *pool) { return pool ? pool->promised() : 0; }

void ts_kv_get_stats(const ts_kv_pool *pool, ts_kv_stats *out) {
    if (!pool || !out) return;
    ts_kv_stats s = {};
    uint64_t held = 0;
    for (uint32_t l : pool->live) held += l > 0;
    s.size = pool->live.size() * pool->page;
    s.active = held * pool->page;
    for (const Slot &slot : pool->slots) {
        if (!slot.run) continue;
        if (slot.run->retained()) {
            s.kept_runs += 1;
        } else {
            s.live_runs += 1;
            s.worst += pool->span(slot.run->worst) * pool->page;
        }
    }
    *out = s;
}

// FNV-1a over each page's holders and each run (pool.rs:310-332).
uint64_t ts_kv_digest(const ts_kv_pool *pool) {
    if (!pool) return 0;
    uint64_t hash = 0xcbf29ce484222325ull;
    auto eat = [&](uint64_t x) {
        for (int b = 0; b < 8; b++) hash = (hash ^ ((x >> (8 * b)) & 0xFF)) * 0x100000001b3ull;
    };
    for (size_t p = 0; p < pool->live.size(); p++) eat(((uint64_t)pool->live[p] << 32) | pool->kept[p]);
    for (const Slot &slot : pool->slots) {
        eat(slot.generation);
        if (!slot.run) continue;
        eat(slot.run->tag);
        eat(slot.run->rows);
        eat(slot.run->worst);
        eat(slot.run->retired);
        for (uint32_t p : slot.run->pages) eat(p);
    }
    return hash;
}

int ts_kv_consistent(const ts_kv_pool *pool) { return pool && pool->consistent() ? 1 : 0; }

int ts_kv_fill_table(const ts_kv_pool *pool, ts_kv_run id, uint32_t *table, uint32_t slot, uint32_t kept_pages) {
    if (!pool || !table) return TS_KV_BAD_ARGUMENT;
    KV_RUN(pool, id, r);
    if (r->pages.size() > kept_pages) return TS_KV_BAD_ARGUMENT;
    for (size_t i = 0; i < r->pages.size(); i++) table[(size_t)slot * kept_pages + i] = r->pages[i];
    return TS_KV_OK;
}

int ts_kv_copy_pages(void *kept_rows, const ts_kv_copy *copies, uint32_t n_copies, uint32_t page_rows,
                     size_t row_bytes, void *stream) {
    if (!kept_rows || (!copies && n_copies)) return TS_KV_BAD_ARGUMENT;
    for (uint32_t i = 0; i < n_copies; i++) {
        char *base = (char *)kept_rows;
        cudaError_t e = cudaMemcpyAsync(base + (size_t)copies[i].to * page_rows * row_bytes,
                                        base + (size_t)copies[i].from * page_rows * row_bytes,
                                        (size_t)copies[i].rows * row_bytes, cudaMemcpyDeviceToDevice,
                                        (cudaStream_t)stream);
        if (e != cudaSuccess)
            return ts::fail(TS_ERR_CUDA, "page copy %u -> %u failed: %s", copies[i].from, copies[i].to,
                            cudaGetErrorString(e));
    }
    return TS_KV_OK;
}

// ---- prefix reuse (engine/ir/kv/src/reuse.rs, prefix.rs): host arithmetic on token ids ----
void ts_kv_begin_rows(const uint32_t *history, uint64_t history_len, uint64_t valid, const uint32_t *prompt,
                      uint64_t prompt_len, uint64_t limit, uint64_t grid, ts_kv_begin *out) {
    if (!out) return;
    uint64_t lcp = 0;
    const uint64_t both = history_len < prompt_len ? history_len : prompt_len;
    while (lcp < both && history[lcp] == prompt[lcp]) lcp++;
    uint64_t rows = lcp < valid ? lcp : valid;
    if (limit < rows) rows = limit;
    const uint64_t step = grid > 0 ? grid : 1;
    out->skip = rows / step * step;
    out->lcp = lcp;
    out->why = history_len == 0 ? TS_KV_WHY_FIRST : rows == 0 ? TS_KV_WHY_NO_LCP : out->skip == 0 ? TS_KV_WHY_GRID : TS_KV_WHY_HIT;
}

struct ts_kv_prefixes {
    struct Entry {
        ts_kv_run run;
        std::vector<uint32_t> history;
        uint64_t valid;
    };
    uint64_t grid;
    std::vector<Entry> kept;  // oldest first
};

ts_kv_prefixes *ts_kv_prefixes_new(uint64_t grid) {
    ts_kv_prefixes *p = new (std::nothrow) ts_kv_prefixes();
    if (p) p->grid = grid;
    return p;
}

void ts_kv_prefixes_free(ts_kv_prefixes *prefixes) { delete prefixes; }

int ts_kv_prefixes_keep(ts_kv_prefixes *prefixes, ts_kv_run run, const uint32_t *history, uint64_t history_len,
                        uint64_t valid) {
    if (!prefixes || (history_len > 0 && !history)) return TS_KV_BAD_ARGUMENT;
    ts_kv_prefixes::Entry e;
    e.run = run;
    e.history.assign(history, history + history_len);
    e.valid = valid;
    prefixes->kept.push_back(std::move(e));
    return TS_KV_OK;
}

int ts_kv_prefixes_find(ts_kv_prefixes *prefixes, const ts_kv_pool *pool, uint64_t tag, const uint32_t *prompt,
                        uint64_t prompt_len, uint64_t limit, ts_kv_run *run, uint64_t *skip, int *found) {
    if (!prefixes || !pool || !run || !skip || !found || (prompt_len > 0 && !prompt)) return TS_KV_BAD_ARGUMENT;
    // entries whose run is gone (released, reclaimed or adopted) leave first: prefix.rs:42
    std::vector<ts_kv_prefixes::Entry> alive;
    for (auto &e : prefixes->kept) {
        uint64_t rows;
        if (ts_kv_rows(pool, e.run, &rows) == TS_KV_OK) alive.push_back(std::move(e));
    }
    prefixes->kept.swap(alive);
    *found = 0;
    *skip = 0;
    for (const auto &e : prefixes->kept) {
        uint64_t its;
        if (ts_kv_tag(pool, e.run, &its) != TS_KV_OK || its != tag) continue;
        ts_kv_begin b;
        ts_kv_begin_rows(e.history.data(), e.history.size(), e.valid, prompt, prompt_len, limit, prefixes->grid, &b);
        if (b.skip > 0 && (!*found || b.skip >= *skip)) {  // a later entry wins a tie: the newest run
            *found = 1;
            *skip = b.skip;
            *run = e.run;
        }
    }
    return TS_KV_OK;
}

uint64_t ts_kv_prefixes_len(const ts_kv_prefixes *prefixes) { return prefixes ? prefixes->kept.size() : 0; }

// ---- slots over the pool (engine/engine/src/kept.rs:27-159) ----
struct ts_kept_slots {
    ts_kv_pool *pool = nullptr;
    ts_kv_prefixes *index = nullptr;
    uint64_t context = 0;
    std::vector<std::optional<ts_kv_run>> runs;  // each slot's live run
    bool paged = false;
    std::vector<uint32_t> free_slots;            // paged: the free slots, the next one last
    std::vector<size_t> laned;                   // paged: the pages each slot's lane names
    uint64_t hits = 0, misses = 0;
    ~ts_kept_slots() {
        ts_kv_prefixes_free(index);
        ts_kv_pool_free(pool);
    }
};

static const uint64_t kKeptTag = 0;  // kept.rs:6

ts_kept_slots *ts_kept_slots_dense(uint32_t slots, uint32_t context) {
    if (slots == 0 || context == 0) return nullptr;
    ts_kept_slots *k = new (std::nothrow) ts_kept_slots();
    if (!k) return nullptr;
    k->pool = ts_kv_pool_new(slots, context);
    k->index = ts_kv_prefixes_new(0);
    k->context = context;
    k->runs.assign(slots, std::nullopt);
    if (!k->pool || !k->index) {
        delete k;
        return nullptr;
    }
    return k;
}

ts_kept_slots *ts_kept_slots_paged(uint32_t slots, uint32_t context, uint32_t pages, uint32_t page) {
    if (slots == 0 || context == 0 || pages == 0 || page == 0) return nullptr;
    ts_kept_slots *k = new (std::nothrow) ts_kept_slots();
    if (!k) return nullptr;
    k->pool = ts_kv_pool_new(pages, page);
    k->index = ts_kv_prefixes_new(page);
    k->context = context;
    k->runs.assign(slots, std::nullopt);
    k->paged = true;
    for (uint32_t s = slots; s-- > 0;) k->free_slots.push_back(s);  // (0..slots).rev(): slot 0 goes first
    k->laned.assign(slots, 0);
    if (!k->pool || !k->index) {
        delete k;
        return nullptr;
    }
    return k;
}

void ts_kept_slots_free(ts_kept_slots *kept) { delete kept; }

int ts_kept_slots_admit(ts_kept_slots *k, const uint32_t *prompt, uint64_t prompt_len, uint64_t limit, uint32_t *slot,
                        uint64_t *skip, int *admitted) {
    if (!k || !slot || !skip || !admitted || (prompt_len > 0 && !prompt)) return TS_KV_BAD_ARGUMENT;
    *admitted = 0;
    *skip = 0;
    ts_kv_run hit_run = {};
    uint64_t hit_skip = 0;
    int found = 0;
    int rc = ts_kv_prefixes_find(k->index, k->pool, kKeptTag, prompt, prompt_len, limit, &hit_run, &hit_skip, &found);
    if (rc != TS_KV_OK) return rc;
    const uint64_t worst = k->context;
    ts_kv_run run = {};
    uint64_t got = 0;
    if (!k->paged) {
        bool have = found && ts_kv_adopt(k->pool, hit_run, hit_skip, worst, &run) == TS_KV_OK;
        if (have) got = hit_skip;
        else if (ts_kv_reserve(k->pool, kKeptTag, 1, worst, &run) != TS_KV_OK) return TS_KV_OK;  // no room: not admitted
        uint32_t page = 0, count = 0;
        if (ts_kv_pages(k->pool, run, &page, 1, &count) != TS_KV_OK || count == 0) return TS_KV_OK;
        *slot = page;  // dense: the slot is the run's one page
        k->runs[page] = run;
    } else {
        if (k->free_slots.empty()) return TS_KV_OK;
        const uint32_t s = k->free_slots.back();
        bool have = found && ts_kv_fork(k->pool, hit_run, hit_skip, worst, &run) == TS_KV_OK;
        if (have) got = hit_skip;
        else if (ts_kv_reserve(k->pool, kKeptTag, 0, worst, &run) != TS_KV_OK) return TS_KV_OK;
        k->free_slots.pop_back();
        k->runs[s] = run;
        k->laned[s] = 0;
        *slot = s;
    }
    *skip = got;
    *admitted = 1;
    (got == 0 ? k->misses : k->hits)++;
    return TS_KV_OK;
}

int ts_kept_slots_grow(ts_kept_slots *k, uint32_t slot, uint64_t rows, uint32_t *pages, uint32_t capacity,
                       uint32_t *count) {
    if (!k || !count || slot >= k->runs.size()) return TS_KV_BAD_ARGUMENT;
    *count = 0;
    if (!k->paged) return TS_KV_OK;
    if (!k->runs[slot]) return TS_KV_ROW_PLACE;
    const ts_kv_run run = *k->runs[slot];
    ts_kv_copy copies[2];
    uint32_t n = 0;
    int rc = ts_kv_grow(k->pool, run, rows, copies, 2, &n);
    if (rc != TS_KV_OK) return rc;
    if (n != 0) return TS_KV_SHARED_PAGE;  // runs share only whole pages, so no row moves
    uint32_t have = 0;
    rc = ts_kv_pages(k->pool, run, pages, pages ? capacity : 0, &have);
    if (rc != TS_KV_OK) return rc;
    const bool more = have != k->laned[slot];
    k->laned[slot] = have;
    *count = more ? have : 0;
    return TS_KV_OK;
}

int ts_kept_slots_finish(ts_kept_slots *k, uint32_t slot, const uint32_t *history, uint64_t history_len) {
    if (!k || slot >= k->runs.size() || (history_len > 0 && !history)) return TS_KV_BAD_ARGUMENT;
    if (!k->runs[slot]) return TS_KV_OK;
    const ts_kv_run run = *k->runs[slot];
    k->runs[slot].reset();
    if (k->paged) k->free_slots.push_back(slot);
    ts_kv_copy copies[2];
    uint32_t n = 0;
    const bool grown = history_len > 0 && ts_kv_grow(k->pool, run, history_len, copies, 2, &n) == TS_KV_OK;
    if (grown && ts_kv_retain(k->pool, run) == TS_KV_OK) ts_kv_prefixes_keep(k->index, run, history, history_len, history_len);
    else ts_kv_release(k->pool, run);
    return TS_KV_OK;
}

void ts_kept_slots_totals(const ts_kept_slots *k, ts_kept_totals *out) {
    if (!k || !out) return;
    ts_kv_get_stats(k->pool, &out->pool);
    out->hits = k->hits;
    out->misses = k->misses;
}

const ts_kv_pool *ts_kept_slots_pool(const ts_kept_slots *k) { return k ? k->pool : nullptr; }

}  // extern "C"
#pragma GCC visibility pop
