// The request loop over a stepper: host code only (no kernel, no CUDA call of its own).
// Restates the reference's scheduler with its Fair policy (engine/engine/src/schedule.rs:17-76 `Seq`,
// 122-153 `Fair`, 227-262 admission, 310-334 paging and retiring, 383-416 `turn`) over ts_kept_slots_*.
#include <deque>
#include <vector>

#include "tessera_b200_run.h"
#include "ts_common.cuh"

namespace {

// An answer in flight, in its slot.
struct Seq {
    uint32_t index;                // place in the caller's list
    uint32_t slot;
    std::deque<uint32_t> pending;  // tokens to feed: the prompt past the skip, then each token made
    uint64_t fed;                  // rows of this sequence in the kept rows
    std::vector<uint32_t> history; // the tokens behind those rows
    uint32_t made;
    bool prefilling() const { return pending.size() > 1; }
};

}  // namespace

struct ts_sessions {
    ts_stepper stepper = {};
    ts_kept_slots *kept = nullptr;
    bool reuse = true;
    uint32_t budget = 0, pages_per_slot = 0;
    std::vector<uint32_t> table;  // paged: the host copy of the page table (engine/engine/src/lanes.rs)
    bool stale = false;
    uint64_t steps = 0;
    ~ts_sessions() { ts_kept_slots_free(kept); }
};

#pragma GCC visibility push(default)
extern "C" {

ts_sessions *ts_sessions_new(const ts_stepper *st, int reuse, uint32_t budget) {
    if (!st || !st->step || st->slots == 0 || st->context == 0 || st->max_rows == 0) return nullptr;
    if (st->page != 0 && !st->set_table) return nullptr;
    ts_sessions *s = new (std::nothrow) ts_sessions();
    if (!s) return nullptr;
    s->stepper = *st;
    s->reuse = reuse != 0;
    s->budget = budget ? budget : st->max_rows;
    if (st->page) {
        s->pages_per_slot = (st->context + st->page - 1) / st->page;
        s->kept = ts_kept_slots_paged(st->slots, st->context, st->slots * s->pages_per_slot, st->page);
        s->table.resize((size_t)st->slots * s->pages_per_slot);
        for (size_t i = 0; i < s->table.size(); i++) s->table[i] = (uint32_t)i;  // each slot its own pages
        s->stale = true;
    } else {
        s->kept = ts_kept_slots_dense(st->slots, st->context);
    }
    if (!s->kept) {
        delete s;
        return nullptr;
    }
    return s;
}

static int decoder_step(void *self, const uint32_t *tokens, const uint32_t *slots, const uint32_t *positions, uint32_t rows,
                        const uint32_t *out_rows, uint32_t n_out, uint32_t *out_ids) {
    return ts_decoder_step((ts_decoder *)self, tokens, slots, positions, rows, out_rows, n_out, out_ids, nullptr);
}

static int decoder_table(void *self, const uint32_t *table, uint32_t entries) {
    return ts_decoder_set_table((ts_decoder *)self, table, entries);
}

ts_sessions *ts_sessions_on_decoder(ts_decoder *dec, int reuse, uint32_t budget) {
    ts_decoder_config c;
    if (!dec || ts_decoder_get_config(dec, &c) != TS_OK) return nullptr;
    ts_stepper st = {};
    st.self = dec;
    st.slots = c.slots;
    st.context = c.context;
    st.max_rows = c.max_rows;
    st.page = c.page;
    st.step = decoder_step;
    st.set_table = decoder_table;
    return ts_sessions_new(&st, reuse, budget);
}

void ts_sessions_free(ts_sessions *s) { delete s; }

int ts_sessions_generate(ts_sessions *s, const uint32_t *tokens, const uint64_t *offsets, uint32_t n_prompts,
                         uint32_t new_tokens, uint32_t *out) {
    TS_REQUIRE(s && offsets && out && (tokens || n_prompts == 0), "sessions: NULL argument");
    TS_REQUIRE(new_tokens >= 1, "sessions: an answer has at least one token");
    const ts_stepper &st = s->stepper;
    for (uint32_t i = 0; i < n_prompts; i++) {
        TS_REQUIRE(offsets[i + 1] > offsets[i], "sessions: prompt %u is empty", i);
        TS_REQUIRE(offsets[i + 1] - offsets[i] + new_tokens <= st.context,
                   "sessions: prompt %u: %llu tokens and %u new ones do not fit %u rows", i,
                   (unsigned long long)(offsets[i + 1] - offsets[i]), new_tokens, st.context);
    }
    uint32_t next = 0;  // the first prompt still waiting
    std::vector<Seq> active;
    // Every failing exit gives the active sequences' slots and pages back (finish with no history releases
    // instead of retaining), as the reference retires a sequence on every exit path (schedule.rs finish/retire):
    // the next generate on these sessions then starts from a clean pool.
    auto bail = [&](int rc) {
        for (Seq &q : active) ts_kept_slots_finish(s->kept, q.slot, nullptr, 0);
        active.clear();
        return rc;
    };
    std::vector<uint32_t> row_tokens, row_slots, row_positions, ends, ids, pages(s->pages_per_slot ? s->pages_per_slot : 1);
    std::vector<uint32_t> take;
    std::vector<size_t> owners;
    while (next < n_prompts || !active.empty()) {
        // ---- admit waiting prompts while slots are free (schedule.rs:227-262) ----
        while (next < n_prompts) {
            const uint32_t *prompt = tokens + offsets[next];
            const uint64_t len = offsets[next + 1] - offsets[next];
            uint32_t slot = 0;
            uint64_t skip = 0;
            int admitted = 0;
            // the last prompt row is always fed: its logits make the first token
            int rc = ts_kept_slots_admit(s->kept, prompt, len, s->reuse ? len - 1 : 0, &slot, &skip, &admitted);
            if (rc != TS_KV_OK) return bail(ts::fail(TS_ERR_PROTOCOL, "sessions: admission failed with pool status %d", rc));
            if (!admitted) break;
            Seq q;
            q.index = next;
            q.slot = slot;
            q.pending.assign(prompt + skip, prompt + len);
            q.fed = skip;
            q.history.assign(prompt, prompt + skip);
            q.made = 0;
            active.push_back(std::move(q));
            next++;
        }
        if (active.empty()) return bail(ts::fail(TS_ERR_PROTOCOL, "sessions: the pool has no room for one more sequence"));

        // ---- Fair: decodes first, then a prompt token each in turn within the budget (schedule.rs:127-153) ----
        take.assign(active.size(), 0);
        uint32_t rows = 0;
        for (size_t i = 0; i < active.size() && rows < st.max_rows; i++)
            if (!active[i].prefilling()) {
                take[i] = 1;
                rows++;
            }
        const uint32_t most = s->budget < st.max_rows ? s->budget : st.max_rows;
        for (bool more = true; more;) {
            more = false;
            for (size_t i = 0; i < active.size(); i++)
                if (active[i].prefilling() && take[i] < active[i].pending.size() && rows < most) {
                    take[i]++;
                    rows++;
                    more = true;
                }
        }

        // ---- the launch: a sequence's rows side by side, in position order; pages first (schedule.rs:311-322) ----
        row_tokens.clear();
        row_slots.clear();
        row_positions.clear();
        ends.clear();
        owners.clear();
        for (size_t i = 0; i < active.size(); i++) {
            const uint32_t n = take[i];
            if (n == 0) continue;
            Seq &q = active[i];
            for (uint32_t j = 0; j < n; j++) {
                row_tokens.push_back(q.pending[j]);
                row_slots.push_back(q.slot);
                row_positions.push_back((uint32_t)(q.fed + j));
            }
            uint32_t count = 0;
            int rc = ts_kept_slots_grow(s->kept, q.slot, q.fed + n, pages.data(), (uint32_t)pages.size(), &count);
            if (rc != TS_KV_OK)
                return bail(ts::fail(TS_ERR_PROTOCOL, "sessions: slot %u cannot grow to %llu rows (pool status %d)", q.slot,
                                     (unsigned long long)(q.fed + n), rc));
            if (count > 0) {
                for (uint32_t j = 0; j < count; j++) s->table[(size_t)q.slot * s->pages_per_slot + j] = pages[j];
                s->stale = true;
            }
            ends.push_back((uint32_t)row_tokens.size() - 1);
            owners.push_back(i);
        }
        if (s->stale) {
            int rc = st.set_table(st.self, s->table.data(), (uint32_t)s->table.size());
            if (rc != TS_OK) return bail(rc);
            s->stale = false;
        }
        ids.assign(ends.size(), 0);
        int rc = st.step(st.self, row_tokens.data(), row_slots.data(), row_positions.data(), (uint32_t)row_tokens.size(),
                         ends.data(), (uint32_t)ends.size(), ids.data());
        if (rc != TS_OK) return bail(rc);
        s->steps++;

        // ---- each answer takes its rows and its last id (Seq::advance, schedule.rs:52-76) ----
        std::vector<size_t> done;
        for (size_t k = 0; k < owners.size(); k++) {
            Seq &q = active[owners[k]];
            const uint32_t n = take[owners[k]];
            for (uint32_t j = 0; j < n; j++) {
                q.history.push_back(q.pending.front());
                q.pending.pop_front();
            }
            q.fed += n;
            if (!q.pending.empty()) continue;  // more of the prompt to feed: the id is not used
            out[(size_t)q.index * new_tokens + q.made] = ids[k];
            q.made++;
            if (q.made >= new_tokens) {
                ts_kept_slots_finish(s->kept, q.slot, q.history.data(), q.history.size());  // Sched::retire
                done.push_back(owners[k]);
            } else {
                q.pending.push_back(ids[k]);
            }
        }
        for (size_t k = done.size(); k-- > 0;) active.erase(active.begin() + (ptrdiff_t)done[k]);
    }
    return TS_OK;
}

uint64_t ts_sessions_steps(const ts_sessions *s) { return s ? s->steps : 0; }

void ts_sessions_totals(const ts_sessions *s, ts_kept_totals *out) {
    if (s && out) ts_kept_slots_totals(s->kept, out);
}

int ts_sessions_consistent(const ts_sessions *s) { return s ? ts_kv_consistent(ts_kept_slots_pool(s->kept)) : 0; }

}  // extern "C"
#pragma GCC visibility pop
