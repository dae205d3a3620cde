/*
 * tessera_b200 KV page pool — the host-side allocator that produces the page tables the paged
 * attention kernel walks.  It restates tessera-kv's `Pool` (engine/ir/kv/src/pool.rs:71-305): runs of
 * kept rows hold pages of `page` rows; forks share a source's pages (reference counts per page, live
 * and retained holders apart); a write into a shared partial page first copies it (`PageCopy`);
 * admission refuses anything that would keep some live run from reaching its worst case; retained
 * runs are reclaimed oldest first; pages are handed out lowest-free-first; every error leaves the
 * pool unchanged (pool.rs:25-40).  Pure host code: no CUDA call except ts_kv_copy_pages.
 */
#ifndef TESSERA_B200_KV_H
#define TESSERA_B200_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ts_kv_pool ts_kv_pool;

/* A run's place in the pool; stale ids fail (pool.rs:6-11). */
typedef struct {
    uint32_t at, generation;
} ts_kv_run;

/* Rows to copy between pages before the launch writes (pool.rs:17-23). */
typedef struct {
    uint32_t from, to, rows;
} ts_kv_copy;

/* pool.rs:25-40.  `detail` of the last failure: the page count of NO_ROOM, the bound of PAST_*. */
typedef enum {
    TS_KV_OK = 0,
    TS_KV_NO_ROOM = 1,
    TS_KV_PAST_WORST = 2,
    TS_KV_PAST_SOURCE = 3,
    TS_KV_LIVE = 4,
    TS_KV_RETAINED = 5,
    TS_KV_UNKNOWN = 6,
    TS_KV_BAD_ARGUMENT = 7,
    /* the engine's own two (engine/engine/src/lib.rs:101-102, 111-112) */
    TS_KV_ROW_PLACE = 8,   /* the slot holds no live run */
    TS_KV_SHARED_PAGE = 9  /* a slot's next row is in another run's page */
} ts_kv_status;

/* pool.rs:56-68. */
typedef struct {
    uint64_t size, active, worst, live_runs, kept_runs;
} ts_kv_stats;

ts_kv_pool *ts_kv_pool_new(uint32_t pages, uint32_t page_rows);
void ts_kv_pool_free(ts_kv_pool *pool);
uint64_t ts_kv_last_detail(const ts_kv_pool *pool);

/* pool.rs:139-156, 158-191, 193-222, 224-246, 248-262, 264-300, 302-308. */
int ts_kv_reserve(ts_kv_pool *pool, uint64_t tag, uint64_t rows, uint64_t worst, ts_kv_run *out);
int ts_kv_fork(ts_kv_pool *pool, ts_kv_run source, uint64_t rows, uint64_t worst, ts_kv_run *out);
int ts_kv_grow(ts_kv_pool *pool, ts_kv_run run, uint64_t rows, ts_kv_copy *copies, uint32_t capacity,
               uint32_t *n_copies);
int ts_kv_truncate(ts_kv_pool *pool, ts_kv_run run, uint64_t rows);
int ts_kv_retain(ts_kv_pool *pool, ts_kv_run run);
int ts_kv_adopt(ts_kv_pool *pool, ts_kv_run run, uint64_t rows, uint64_t worst, ts_kv_run *out);
int ts_kv_release(ts_kv_pool *pool, ts_kv_run run);

/* pool.rs:87-97: the run's pages in order (writes at most `capacity`, reports the count), rows, tag. */
int ts_kv_pages(const ts_kv_pool *pool, ts_kv_run run, uint32_t *out, uint32_t capacity, uint32_t *count);
int ts_kv_rows(const ts_kv_pool *pool, ts_kv_run run, uint64_t *rows);
int ts_kv_tag(const ts_kv_pool *pool, ts_kv_run run, uint64_t *tag);

/* pool.rs:99-137, 310-332, 433-449. */
uint64_t ts_kv_spare(const ts_kv_pool *pool);
uint64_t ts_kv_promised(const ts_kv_pool *pool);
void ts_kv_get_stats(const ts_kv_pool *pool, ts_kv_stats *out);
uint64_t ts_kv_digest(const ts_kv_pool *pool);
int ts_kv_consistent(const ts_kv_pool *pool);

/* Writes the run's pages into row `slot` of a page table of `kept_pages` entries per slot (the
 * layout ts_kept / ts_decoder_set_table take); entries past the run's pages keep their value. */
int ts_kv_fill_table(const ts_kv_pool *pool, ts_kv_run run, uint32_t *table, uint32_t slot, uint32_t kept_pages);

/* Performs page copies on the device before the launch that writes: for each copy, the first `rows`
 * rows of page `from` go to page `to` in a kept buffer of `row_bytes` bytes per row. */
int ts_kv_copy_pages(void *kept_rows, const ts_kv_copy *copies, uint32_t n_copies, uint32_t page_rows,
                     size_t row_bytes, void *stream);

/* ---------------------------------------------------------------------------
 * Prefix reuse: which rows of a prompt the kept rows of an earlier run spare.
 * Restates engine/ir/kv/src/reuse.rs:1-37 (`begin`) and engine/ir/kv/src/prefix.rs:1-55 (`Prefixes`).
 * ------------------------------------------------------------------------- */

/* reuse.rs:3-14: why a prompt skips the rows it does. */
typedef enum {
    TS_KV_WHY_FIRST = 0,   /* there is no history */
    TS_KV_WHY_NO_LCP = 1,  /* no common row is both valid and within the limit */
    TS_KV_WHY_GRID = 2,    /* the common rows end below one grid step */
    TS_KV_WHY_HIT = 3
} ts_kv_why;

/* reuse.rs:16-22. */
typedef struct {
    uint64_t skip, lcp;
    int why;
} ts_kv_begin;

/* reuse.rs:24-37: lcp = the common prefix of history and prompt; rows = min(lcp, valid, limit); skip = rows
 * rounded down to a whole number of `grid` steps (grid 0 counts as 1). */
void ts_kv_begin_rows(const uint32_t *history, uint64_t history_len, uint64_t valid, const uint32_t *prompt,
                      uint64_t prompt_len, uint64_t limit, uint64_t grid, ts_kv_begin *out);

/* prefix.rs:11-55: the tokens behind retained runs, oldest first. */
typedef struct ts_kv_prefixes ts_kv_prefixes;
ts_kv_prefixes *ts_kv_prefixes_new(uint64_t grid);
void ts_kv_prefixes_free(ts_kv_prefixes *prefixes);

/* Records the tokens behind a retained run's `valid` rows (the tokens are copied). */
int ts_kv_prefixes_keep(ts_kv_prefixes *prefixes, ts_kv_run run, const uint32_t *history, uint64_t history_len,
                        uint64_t valid);

/* The newest run of `tag` with the longest skip for `prompt`: first drops entries whose run the pool no longer
 * knows, then *found = 1 with the run and its skip, or *found = 0 when no entry spares a row. */
int ts_kv_prefixes_find(ts_kv_prefixes *prefixes, const ts_kv_pool *pool, uint64_t tag, const uint32_t *prompt,
                        uint64_t prompt_len, uint64_t limit, ts_kv_run *run, uint64_t *skip, int *found);

/* Entries held (after the last find's clean-up). */
uint64_t ts_kv_prefixes_len(const ts_kv_prefixes *prefixes);

/* ---------------------------------------------------------------------------
 * Slots over the pool: which slot a prompt gets and how many of its rows the kept rows spare.
 * Restates the engine's `Kept` (engine/engine/src/kept.rs:27-159), the caller of the pool and the prefix index.
 * Dense: each slot is one page of `context` rows, a hit adopts the retained run (and with it the slot).
 * Paged: slots share whole pages of `page` rows, a hit forks the retained run's pages into a free slot; skips come
 * in whole pages, so no row ever moves.
 * ------------------------------------------------------------------------- */
typedef struct ts_kept_slots ts_kept_slots;

typedef struct {
    ts_kv_stats pool;
    uint64_t hits, misses;
} ts_kept_totals;

ts_kept_slots *ts_kept_slots_dense(uint32_t slots, uint32_t context);                               /* kept.rs:43-55 */
ts_kept_slots *ts_kept_slots_paged(uint32_t slots, uint32_t context, uint32_t pages, uint32_t page); /* kept.rs:57-67 */
void ts_kept_slots_free(ts_kept_slots *kept);

/* kept.rs:69-106: a slot for `prompt` and the rows it may skip (at most `limit`).  *admitted = 0 when no slot or no
 * room is free (nothing changes then). */
int ts_kept_slots_admit(ts_kept_slots *kept, const uint32_t *prompt, uint64_t prompt_len, uint64_t limit, uint32_t *slot,
                        uint64_t *skip, int *admitted);

/* kept.rs:133-148: paged: grows the slot's run to `rows` rows; when its lane lacks pages, writes the run's pages
 * (at most `capacity`) and their count, else *count = 0.  Dense: *count = 0.  TS_KV_ROW_PLACE for a slot with no
 * run, TS_KV_SHARED_PAGE when the growth would have to copy a shared page, the pool's errors otherwise. */
int ts_kept_slots_grow(ts_kept_slots *kept, uint32_t slot, uint64_t rows, uint32_t *pages, uint32_t capacity,
                       uint32_t *count);

/* kept.rs:150-159: keeps the slot's rows under their tokens (the run is retained and indexed), or releases them when
 * there are none or the pool refuses; the slot is free again. */
int ts_kept_slots_finish(ts_kept_slots *kept, uint32_t slot, const uint32_t *history, uint64_t history_len);

void ts_kept_slots_totals(const ts_kept_slots *kept, ts_kept_totals *out);                          /* kept.rs:125-131 */
const ts_kv_pool *ts_kept_slots_pool(const ts_kept_slots *kept);

#ifdef __cplusplus
}
#endif
#endif
