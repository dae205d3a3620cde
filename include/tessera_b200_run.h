/*
 * tessera_b200 runner — the host side that replays a decoder's plan of launches on one GPU.
 *
 * It plays the part of tessera-run's CUDA backend for the Qwen3-shaped decoder graph
 * (engine/plan/run/src/run.rs:122-345: load, feed, submit, read; engine/plan/run/src/device.rs:
 * 128-242: bind arguments, launch, CUDA-graph replay keyed by the bound sizes) with the step list
 * of engine/models/src/decoder.rs:281-389 fixed at creation: gather, then per layer rms_norm,
 * fused q|k|v linear, per-head norm + rotation + kept-row append, ragged attention over kept rows,
 * o linear + residual, rms_norm, gate|up linear with SwiGLU, down linear + residual; final
 * rms_norm, tied unembedding, greedy top-1.
 *
 * Ownership follows the reference: the runner owns every plan buffer (allocated once at creation,
 * zeroed, freed at destroy), weights are uploaded once with ts_decoder_load, and nothing on the
 * step path allocates.  One runner per thread; calls take a CUDA stream.
 */
#ifndef TESSERA_B200_RUN_H
#define TESSERA_B200_RUN_H

#include <stddef.h>
#include <stdint.h>

#include "tessera_b200.h"
#include "tessera_b200_kv.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ts_decoder ts_decoder;

typedef struct {
    uint32_t layers, hidden, heads, kv_heads, head_dim, ffn, vocab;
    uint32_t slots;    /* sequences the kept store holds (engine `Seqs`) */
    uint32_t context;  /* positions per slot (engine `Context`) */
    uint32_t page;     /* 64 ("paged"), 16 ("paged16") or 0 (dense kept rows) */
    uint32_t max_rows; /* most rows one launch carries (engine `Rows`) */
    float eps, theta;
    int qk_norm;       /* per-head RMS norm on q and k (Qwen3) */
    int graphs;        /* replay steps as CUDA graphs (engine/plan/lower/src/recipe.rs:51-57 `launch.graphs`) */
    int pdl;           /* programmatic dependent launch between steps (`launch.pdl`) */
} ts_decoder_config;

/* Allocates the plan's buffers on the current device.  The page table starts as the identity
 * (engine/engine/src/lanes.rs:4-65). */
int ts_decoder_create(const ts_decoder_config *config, ts_decoder **out);
void ts_decoder_destroy(ts_decoder *dec);

/* Uploads one weight from host memory (tessera_run::Run::load_weight, run.rs:204-250).  Names follow the
 * declaration order of engine/models/src/decoder.rs:225-255: "embed", "layers.<i>.ln1", ".q", ".k", ".v",
 * ".q_norm", ".k_norm", ".o", ".ln2", ".mlp.gate", ".mlp.up", ".mlp.down", "norm".  Linears are bf16
 * [out, in]; norm gains are f32. */
int ts_decoder_load(ts_decoder *dec, const char *name, const void *host_data, size_t bytes);

/* Replaces the page table (slots * ceil(context / page) entries; every entry < that count).  Ordering: this call
 * and ts_decoder_load first wait for the stream of the decoder's most recent launches (a resident loop returns
 * without waiting), then copy; launches made after they return see the new contents. */
int ts_decoder_set_table(ts_decoder *dec, const uint32_t *host_table, uint32_t entries);

/* Applies the page copies a pool planned (ts_kv_grow: a write into a shared partial page first copies it,
 * engine/ir/kv/src/pool.rs:193-222) to the kept K and V rows of every layer, on `stream`, before the launch
 * that writes.  Pages are the table's units: copy {from, to, rows} moves the first `rows` rows of page `from`. */
int ts_decoder_copy_pages(ts_decoder *dec, const ts_kv_copy *copies, uint32_t n_copies, void *stream);

/* One launch: feeds `rows` (token, slot, position) triples from host memory, runs the step list and
 * returns the greedy token of each row listed in `out_rows` (n_out indices into the launch's rows;
 * NULL = every row) in `out_ids` (host).  Synchronises the stream before returning, like
 * Run::submit (run.rs:140-141).  Rows are validated on the host first: a slot, position or token
 * out of range returns TS_ERR_BAD_INPUT and launches nothing.  The launch itself carries the next power of two
 * of rows (copies of the last row, which rewrite that row's kept K and V with the same values), unless the rows
 * are whole prompts from position 0, which run at their exact size. */
int ts_decoder_step(ts_decoder *dec, const uint32_t *tokens, const uint32_t *slots, const uint32_t *positions,
                    uint32_t rows, const uint32_t *out_rows, uint32_t n_out, uint32_t *out_ids, void *stream);

/* Device-resident decode: after a ts_decoder_step that left one row per slot, runs `steps` further
 * launches in which each row's token is the id it just produced and its position moves on by one,
 * without host traffic.  ts_decoder_read_ids copies the latest ids (rows entries) to the host. */
int ts_decoder_run_resident(ts_decoder *dec, uint32_t steps, void *stream);
int ts_decoder_read_ids(ts_decoder *dec, uint32_t *out_ids, uint32_t rows, void *stream);

/* Final normed hidden rows of the last launch, bf16 [rows, hidden], to the host (for parity checks). */
int ts_decoder_read_hidden(ts_decoder *dec, void *out_bf16, uint32_t rows, void *stream);
/* Logits of the last launch, f32 [n_out, vocab], to the host. */
int ts_decoder_read_logits(ts_decoder *dec, float *out, uint32_t n_out, void *stream);

/* Kernel launches one step enqueues for `rows` rows at `keys` visible positions, and how many steps
 * have been replayed from a captured graph so far. */
uint32_t ts_decoder_launches_per_step(ts_decoder *dec, uint32_t rows, uint32_t keys);
uint64_t ts_decoder_graph_replays(ts_decoder *dec);
/* Graphs captured so far.  A launch's rows (and wanted rows) round up to a power of two, the last row filling out,
 * as the reference sizes a launch (engine/engine/src/lib.rs:166-200), so one graph serves a bucket of row counts. */
uint32_t ts_decoder_graphs(ts_decoder *dec);

/* Captures, without running them, the graphs of a decode step of `rows` rows (one per slot, one id out per row)
 * for every context bucket up to the plan's context, with and without on-device feedback: a serving loop then
 * never pays a capture in the middle of a generation.  The reference builds its plans before the first request
 * in the same way (engine/engine/src/lib.rs:401-468).  No-op without graphs. */
int ts_decoder_prepare(ts_decoder *dec, uint32_t rows, void *stream);

/* Per-kernel device time, the reference's Run::profiling / take_profile (engine/plan/run/src/run.rs:
 * 165-177; stamps behind a gate kernel so host launch gaps are excluded, device.rs:144-200).
 * ts_decoder_profile runs `steps` further device-resident decode launches without graphs, with a CUDA
 * event after every kernel of the step list; ts_decoder_take_profile writes the totals as JSON text
 * {"kernel name": [milliseconds, intervals], ...} into `out` and clears them. */
int ts_decoder_profile(ts_decoder *dec, uint32_t steps, void *stream);
int ts_decoder_take_profile(ts_decoder *dec, char *out, size_t capacity);

/* Decode steps of at most 64 rows, one row per slot, at head width 128 run their gather and whole layer stack as
 * one persistent kernel (every SM resident, phases separated by a bounded device-wide barrier, weights streamed
 * across the phases); `on` = 0 keeps one launch per product instead (the reference's plan of launches,
 * engine/models/src/decoder.rs:281-389, one kernel per step of it).  Returns 1 when the persistent kernel exists
 * for this decoder's shapes, 0 when it does not.  Captured graphs of the other form are dropped. */
int ts_decoder_use_step_kernel(ts_decoder *dec, int on);

/* The configuration the decoder was created with. */
int ts_decoder_get_config(const ts_decoder *dec, ts_decoder_config *out);

/* ---------------------------------------------------------------------------
 * The request loop over a decoder whose kept rows outlive the request that wrote them: the reference's
 * scheduler (engine/engine/src/schedule.rs:122-153, 227-345, 383-416) with its `Fair` policy, over
 * ts_kept_slots_*.  A waiting prompt is admitted to a slot and skips the rows an earlier answer left; every step
 * feeds each decoding sequence the token it made last, then the prompts a token each in turn while the step has
 * fewer than `budget` rows; before the launch each fed slot gets the pages its rows need; a finished sequence's
 * rows stay under the tokens that were fed.  The loop drives anything that steps rows: a ts_decoder, or a host's own
 * stepper (tests drive it with a stand-in that needs no GPU).
 * ------------------------------------------------------------------------- */
typedef struct {
    void *self;
    uint32_t slots, context, max_rows;
    uint32_t page;            /* rows per page, 0 = dense kept rows */
    /* rows in, the greedy id of each row listed in out_rows out; 0 = ok */
    int (*step)(void *self, const uint32_t *tokens, const uint32_t *slots, const uint32_t *positions, uint32_t rows,
                const uint32_t *out_rows, uint32_t n_out, uint32_t *out_ids);
    /* paged only: the whole table, slots * ceil(context / page) entries */
    int (*set_table)(void *self, const uint32_t *table, uint32_t entries);
} ts_stepper;

typedef struct ts_sessions ts_sessions;

/* reuse = 0: prompts never skip rows (the kept rows are still retained and reclaimed).  budget = 0: max_rows. */
ts_sessions *ts_sessions_new(const ts_stepper *stepper, int reuse, uint32_t budget);
ts_sessions *ts_sessions_on_decoder(ts_decoder *dec, int reuse, uint32_t budget);
void ts_sessions_free(ts_sessions *sessions);

/* `new_tokens` greedy tokens for each of `n_prompts` prompts (tokens packed, prompt i = tokens[offsets[i] ..
 * offsets[i + 1])); prompts wait while every slot is taken.  out [n_prompts, new_tokens].  TS_ERR_BAD_INPUT for an
 * empty prompt or one that does not fit the context with its answer; a failing step's status otherwise. */
int ts_sessions_generate(ts_sessions *sessions, const uint32_t *tokens, const uint64_t *offsets, uint32_t n_prompts,
                         uint32_t new_tokens, uint32_t *out);

uint64_t ts_sessions_steps(const ts_sessions *sessions);
void ts_sessions_totals(const ts_sessions *sessions, ts_kept_totals *out);
int ts_sessions_consistent(const ts_sessions *sessions);

#ifdef __cplusplus
}
#endif
#endif
