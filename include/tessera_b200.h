/*
 * tessera_b200 — C ABI of the B200 (sm_100a) kernels that stand in for tessera's
 * matmul and attention lowering rules.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the
 * given CUDA stream and returns without synchronising.  Nothing here allocates
 * device memory: scratch space is a caller-owned workspace whose size comes from
 * the matching *_workspace_bytes call, the way a tessera plan owns every buffer
 * its steps touch (engine/plan/run/src/device.rs:397-402).  Arguments are checked
 * on the host before any launch; a bad argument returns TS_ERR_BAD_INPUT and
 * launches nothing.  There is no CPU fallback: without a CUDA device the compute
 * calls return TS_ERR_CUDA.
 *
 * Data types: activations, weights and kept K/V rows are bf16 (little-endian u16,
 * engine/ir/mem/src/form.rs:220-231); sums are f32; the residual stream, norm
 * gains and router scores are f32; ids, slots, positions and page tables are u32.
 */
#ifndef TESSERA_B200_H
#define TESSERA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TS_ABI_VERSION 1

/* Status codes.  0..5 mirror the reference's device ABI
 * (engine/rules/device/include/tessera/core.h:104-111); 6 wraps a CUDA error the way
 * tessera_run::Error::Launch wraps a failed cuLaunchKernel
 * (engine/plan/run/src/device.rs:138-141). */
typedef enum {
    TS_OK = 0,
    TS_ERR_ABI = 1,
    TS_ERR_PEER = 2,
    TS_ERR_BAD_INPUT = 3,
    TS_ERR_TIMEOUT = 4,
    TS_ERR_PROTOCOL = 5,
    TS_ERR_CUDA = 6
} ts_status;

/* Message of the last failure on the calling thread (never NULL). */
const char *ts_last_error(void);
int ts_abi_version(void);

/* Element types of an output buffer. */
typedef enum { TS_BF16 = 0, TS_F32 = 1 } ts_dtype;

/* ---------------------------------------------------------------------------
 * Linear: out[m, n] = sum_k x[m, k] * w[n, k], then one fused epilogue stage.
 * Replaces the matmul rules `tiled*`, `parts_*` (engine/rules/linear/src/tiled.rs:295-304,
 * 577-591), `lanes` (engine/rules/linear/src/lanes.rs:20-65) and `thin`
 * (engine/rules/linear/src/thin.rs:31-55); the epilogue stands for the fused stage
 * chain of engine/plan/lower/src/sites/matmul.rs:148-176.
 *
 *   x   [m, k] bf16 row-major          w   [n, k] bf16 row-major ("[Out, In]")
 *   a0  epilogue operand or NULL       out [m, n] (or [m, n/2] for SWIGLU)
 *
 * x, w, out 16-byte aligned; the tensor-core kernels take k in multiples of 64, any other k runs on the plain kernel.
 * ------------------------------------------------------------------------- */
typedef enum {
    TS_EPI_NONE = 0,
    TS_EPI_ADD = 1,    /* out = acc + a0;  a0 f32 [m, n] (the residual add, Stage::Add) */
    TS_EPI_SWIGLU = 2, /* w holds gate rows [0, n/2) then up rows [n/2, n):
                          out[m, j] = silu(acc[m, j]) * acc[m, n/2 + j]  (Stage::Act + Stage::Mul) */
    TS_EPI_SCALE = 3,  /* out = acc * scale (Stage::Scale) */
    TS_EPI_GEGLU = 4   /* as SWIGLU with the tanh GELU (Act::GeluTanh) */
} ts_epilogue;

/* Which kernel family runs a linear.  AUTO picks by m. */
typedef enum {
    TS_LINEAR_AUTO = 0,
    TS_LINEAR_SKINNY = 1, /* decode-sized m: vector loads + warp MMA, split-K */
    TS_LINEAR_UMMA = 2,   /* tiled tcgen05 / TMEM accumulators fed by TMA (prefill-sized m) */
    TS_LINEAR_STREAM = 3, /* m <= 128: weight-streaming tcgen05, k split over a thread-block cluster and
                             reduced through distributed shared memory, epilogue fused */
    TS_LINEAR_PAIR = 4,   /* m >= 512: 256 x 256 tiles on pairs of SMs (tcgen05 cta_group::2), each block of
                             the pair loading half of both operands */
    TS_LINEAR_PLAIN = 5,  /* any m, n, k: a warp per output element; what AUTO falls back to when k is not a
                             multiple of 64 (the reference's tiled rule takes every size,
                             engine/rules/linear/tests/tiled_test.rs:61-67) */
    TS_LINEAR_ORDERED = 6 /* any m, n, k, no gated epilogue: every output summed over k in ascending order, one
                             multiply and one add at a time, the order of the reference's interpreter
                             (engine/ir/interp/src/cpu.rs, sequential f32 sums; numerics `Order::Fixed`,
                             engine/ir/graph/src/numerics.rs:26-35), so f32 outputs carry the interpreter's bits.
                             For outputs whose ranking matters: a MoE router's scores feed top-k, and an index
                             must not flip on a near tie.  Never picked by AUTO. */
} ts_linear_path;

/* Bytes of workspace ts_linear_bf16 needs for these sizes (0 when none). */
size_t ts_linear_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, int epilogue, int path);

int ts_linear_bf16(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n,
                   uint32_t k, int epilogue, float scale, int out_dtype, int path, void *workspace,
                   size_t workspace_bytes, void *stream);

/* A linear (decode-sized, m <= 128, or prefill-sized, m >= 512) with the RMS norms of the residual stream folded into its two
 * ends.  The reference runs `lane_norm` as a launch of its own between the residual add and the next
 * projection (engine/models/src/decoder.rs:327-389, engine/rules/kernels/src/lane_norm.rs:10-17); at
 * batch 64 that launch is pure latency.  Since rms_norm(row) * gain = (row * gain) / rms(row), the
 * 1/rms factor commutes with the projection:
 *   - out: a linear with the ADD epilogue and an f32 output can also leave xs_out = bf16(out * xs_gain),
 *     the next projection's input, and per output row the sum of squares over each 128-column tile in
 *     ss_out [m, ts_linear_sumsq_parts(...)];
 *   - in: the next linear takes x = that xs and row_ss = those sums, and multiplies its output rows by
 *     1 / sqrt(sum(row_ss[row, :]) / k + row_eps) before its epilogue.
 * The product differs from the unfolded one by where the bf16 rounding of the normed row falls (before
 * instead of after the 1/rms factor): same size of error, not the same bits.  Either half may be left
 * out (NULL pointers). */
typedef struct {
    const float *row_ss;
    uint32_t row_parts; /* partial sums per row in row_ss, 1..32 */
    float row_eps;
    float *ss_out;
    void *xs_out;        /* bf16 [m, n] */
    const float *xs_gain; /* f32 [n] */
} ts_linear_fused;

/* Embedding rows for a model whose first norm is folded into the projection after it: out f32 [rows, width]
 * as ts_gather_bf16 gives them, xs = bf16(row * gain) and ss [rows, parts] with the row's sum of squares in
 * part 0 and zeros in the others (`parts` = what the consuming linear will be told). */
int ts_gather_scaled_bf16(const void *table, const uint32_t *ids, float *out, void *xs, const float *gain, float *ss,
                          uint32_t parts, uint32_t rows, uint32_t table_rows, uint32_t width, void *stream);

/* Partial sums per row a linear of this shape writes to ss_out; 0 when it cannot (then run ts_rms_norm). */
uint32_t ts_linear_sumsq_parts(uint32_t m, uint32_t n, uint32_t k, int epilogue);

int ts_linear_fused_bf16(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n,
                         uint32_t k, int epilogue, float scale, int out_dtype, const ts_linear_fused *fused,
                         void *stream);

/* ---------------------------------------------------------------------------
 * Kept rows (paged KV).  Layouts follow engine/plan/codegen/src/kept.rs:135-194:
 *   dense        row = slot * kept_scalar + position          (kept_scalar = kept_stride)
 *   interleaved  row = position * kept_scalar + slot          (kept_scalar = kept_slots)
 *   paged(page)  entry = slot * kept_scalar + (position >> log2 page)   (kept_scalar = kept_pages)
 *                row = (table[entry] << log2 page) | (position & (page - 1))
 * K and V buffers are [rows, kv_heads, width] bf16.
 * ------------------------------------------------------------------------- */
typedef enum { TS_KEPT_DENSE = 0, TS_KEPT_INTERLEAVED = 1, TS_KEPT_PAGED = 2 } ts_kept_kind;

typedef struct {
    int kind;              /* ts_kept_kind */
    uint32_t page;         /* rows per page, a power of two (64 = "paged", 16 = "paged16") */
    uint32_t kept_scalar;  /* kept_stride | kept_slots | kept_pages: the layout's last scalar */
    const uint32_t *table; /* device, slots * kept_pages entries; NULL unless paged */
    uint32_t table_len;    /* entries in table */
    uint32_t rows;         /* rows the K/V buffers hold (bounds check) */
} ts_kept;

/* Ragged attention over kept rows, causal: row r (slot slots[r], position positions[r]) reads
 * keys [max(0, pos - back), min(pos + 1, keys)) of its slot.  Replaces `attend_rows`
 * (engine/rules/attention/src/attend.rs:124-167, arguments 182-201) and `flash_rows`
 * (engine/rules/attention/src/flash.rs:505-580).  The score scale, a separate `map` launch in
 * the reference (engine/rules/attention/src/lib.rs:22-31), is an argument here.
 *   q [rows, heads, width] bf16; out [rows, heads, width] bf16; width 16, 32, 64, 128 or 256 (the TMA-fed kernels take 128). */
size_t ts_attend_rows_workspace_bytes(uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads,
                                      uint32_t width);

int ts_attend_rows_bf16(const void *q, const void *k, const void *v, void *out, const uint32_t *slots,
                        const uint32_t *positions, const ts_kept *kept, uint32_t rows, uint32_t keys,
                        uint32_t heads, uint32_t kv_heads, uint32_t width, uint32_t back, float scale,
                        void *workspace, size_t workspace_bytes, void *stream);

/* A decode step's ts_qk_norm_rope_append_bf16 and causal ts_attend_rows_bf16 in one launch: the attention
 * kernel norms and rotates the row's q heads and its new key itself, appends the key and value at
 * kept_row(slot, position) and attends over positions [0, position].  Same arithmetic, same bits as the
 * two launches.  Preconditions: no two rows of the call share a slot (a row must not read a key that
 * another row of the same call appends: that is a prefill, use the two launches); head width 128; a dense
 * layout or pages of >= 32 rows, with kept->rows set.  Workspace: ts_attend_rows_workspace_bytes.
 *   qkv [rows, (heads + 2 kv_heads) * width] bf16 (q heads, k heads, v heads); k_rows, v_rows are written. */
int ts_attend_rows_append_bf16(const void *qkv, const float *q_norm, const float *k_norm, const float *inv_freq,
                               void *k_rows, void *v_rows, void *out, const uint32_t *slots,
                               const uint32_t *positions, const ts_kept *kept, uint32_t rows, uint32_t keys,
                               uint32_t heads, uint32_t kv_heads, uint32_t width, float eps, float scale,
                               void *workspace, size_t workspace_bytes, void *stream);

/* Writes rows of x at kept_row(slot, position).  Replaces `scatter`
 * (engine/plan/lower/src/kernels/scatter.rs:11-83).  x [rows, width] bf16, out [kept rows, width]. */
int ts_scatter_bf16(const void *x, const uint32_t *slots, const uint32_t *positions, void *out,
                    const ts_kept *kept, uint32_t rows, uint32_t width, void *stream);

/* The decoder's per-head step between the projections and attention, fused: per-head RMS norm of
 * q and k (gains q_norm, k_norm [width] f32, or NULL for none), half-pair rotation at the row's
 * position (angle = position * inv_freq[j] for the pair (j, j + width/2); inv_freq is a device
 * array of width/2 f32 that ts_rope_inv_freq fills on the host, the reference's `angles` table,
 * engine/rules/kernels/src/rope.rs:38-45), then q -> q_out and k, v -> kept rows.  Stands for the reference's lane_norm + rope +
 * scatter K + scatter V launches (engine/models/src/decoder.rs:354-389;
 * engine/rules/kernels/src/{lane_norm,rope}.rs).
 *   qkv [rows, (heads + 2 kv_heads) * width] bf16 (q heads, then k heads, then v heads). */
int ts_qk_norm_rope_append_bf16(const void *qkv, const float *q_norm, const float *k_norm,
                                const float *inv_freq, const uint32_t *slots, const uint32_t *positions,
                                void *q_out, void *k_rows, void *v_rows, const ts_kept *kept,
                                uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t width,
                                float eps, void *stream);

/* The reference's two rotary launches on their own (engine/rules/kernels/src/rope.rs:10-60), for a host that replays
 * its step list launch by launch.  `angles`: out[p, 2j] = cos(a), out[p, 2j + 1] = sin(a), a = positions[p] *
 * theta^(-2j / width) for pair j < turned, else 0; out f32 [count, width], width even and at most 512; the powers
 * are taken on the host in f32 (cpu.rs:31-34) and ride in the launch.  `rope` (adjacent = 0: pair j is (j, j +
 * width/2); adjacent = 1, `rope_adjacent`: (2j, 2j + 1)) rotates x [positions, heads, width] in place, f32 as in
 * the reference or bf16; products and sums are separate roundings, so f32 rows equal the CPU interpreter's bit
 * for bit given the same angles. */
int ts_rope_angles(const uint32_t *positions, float *out, uint32_t count, uint32_t width, float theta, uint32_t turned,
                   void *stream);

int ts_rope(void *x, ts_dtype dtype, const float *freqs, uint32_t positions, uint32_t heads, uint32_t width, int adjacent,
            void *stream);

/* out[j] = theta^(-2j / width) for j < width/2, in f32 on the host (engine/ir/interp/src/cpu.rs:31-34). */
void ts_rope_inv_freq(float theta, uint32_t width, float *out);

/* Whole-sequence attention.  Replaces `flash*` (engine/rules/attention/src/flash.rs:415-502,
 * arguments 648-668) and `attend` (engine/rules/attention/src/attend.rs:80-123).  Query t of a
 * sequence sits at position past + t with past = keys - queries (0 when keys < queries under a
 * two-sided mask) and sees keys [max(0, pos - back), min(keys, pos + ahead + 1))
 * (engine/ir/graph/src/node.rs:162-187); causal: back = UINT32_MAX, ahead = 0; bidirectional: both
 * UINT32_MAX; Within(n): both n; Back(n): back = n, ahead = 0.  The score scale (> 0) is applied to
 * the dot products, where the reference runs a separate `map` launch on q.
 *   q [seqs, queries, heads, width], k/v [seqs, keys, kv_heads, width], out like q; all bf16.
 * With cu_seqlens (device u32 [seqs + 1], widths 128 and 256) the sequences are packed back to back:
 * q/k/v/out are [total, heads|kv_heads, width], sequence s owns rows [cu[s], cu[s+1]) as both its
 * queries and its keys, `queries` bounds the longest sequence and `keys` is the total row count.
 * Widths 128 and 256 run on tcgen05 (no workspace); width 64 takes the ragged-rows kernel and needs
 * the workspace ts_attend_workspace_bytes reports. */
size_t ts_attend_workspace_bytes(uint32_t seqs, uint32_t queries, uint32_t keys, uint32_t heads,
                                 uint32_t kv_heads, uint32_t width);

int ts_attend_bf16(const void *q, const void *k, const void *v, void *out, const uint32_t *cu_seqlens,
                   uint32_t seqs, uint32_t queries, uint32_t keys, uint32_t heads, uint32_t kv_heads,
                   uint32_t width, uint32_t back, uint32_t ahead, float scale, void *workspace,
                   size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------
 * Row kernels the decode loop needs around the two hot rules.
 * ------------------------------------------------------------------------- */

/* out = rms_norm(x) * w.  Replaces `lane_norm` / `rms_norm` (engine/rules/kernels/src/lane_norm.rs:10-17).
 * x f32 or bf16 [rows, width]; w f32 [width] or NULL (Stage::Rms); out bf16 or f32. */
int ts_rms_norm(const void *x, int x_dtype, const float *w, void *out, int out_dtype, uint32_t rows,
                uint32_t width, float eps, void *stream);

/* out[r] = table[ids[r]] widened to out_dtype; rows outside [first, first + table_rows) read zero.
 * Replaces `gather` (engine/ir/interp/src/cpu.rs:510-525). table bf16 [table_rows, width]. */
int ts_gather_bf16(const void *table, const uint32_t *ids, void *out, int out_dtype, uint32_t rows,
                   uint32_t table_rows, uint32_t width, uint32_t first, void *stream);

/* ids[r, 0..k) = indices of the k largest entries of x[r, :], best first; ties keep the lower
 * index, -inf and NaN are never picked, spare slots hold `width`.  Replaces `top_k`
 * (engine/rules/kernels/src/argmax.rs:38-70); k = 1 is `peaks` + `argmax` (argmax.rs:72-114).
 * x f32 or bf16 [rows, width]; k <= 32; workspace from ts_top_k_workspace_bytes. */
size_t ts_top_k_workspace_bytes(uint32_t rows, uint32_t width, uint32_t k);
int ts_top_k(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, uint32_t k,
             void *workspace, size_t workspace_bytes, void *stream);

/* Greedy top-1 (ts_top_k with k = 1) for callers that have no scratch memory to give.  It has no
 * counterpart in the reference.  A host runtime that fixed all of its device buffers when it planned,
 * or a process whose memory budget is already spent, cannot supply the workspace ts_top_k asks for and
 * cannot allocate one; this entry point needs none from them: its scratch is a 512 KiB device array
 * built into the library (so every GPU that loads the library holds those 512 KiB until exit), and it
 * calls no allocator of any kind.
 *   x f32 or bf16 [rows, width]; ids u32 [rows]; same ordering rules and same results as ts_top_k.
 *   rows must not exceed 1024 (the size of the built-in scratch): more returns TS_ERR_BAD_INPUT.
 * The first call on each device looks up the array's device address (with that device current); make
 * that first call before starting any stream capture.  All calls share the one array - nothing in it
 * has to be cleared, each call overwrites what it reads - so two calls that overlap on the GPU (two
 * streams, two threads) race: serialise them. */
int ts_top_1_static(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, void *stream);

/* out[s, :] = mean over the rows [cu_seqlens[s], cu_seqlens[s + 1]) of x (the graph's `.mean(1)`,
 * engine/models/src/eg2.rs:249; sums x / count in row order as engine/ir/interp/src/cpu.rs:449-473), then
 * with normalize != 0 scaled to unit length (frontend/tasks/src/embed.rs:47-52).  x, out f32. */
int ts_mean_pool(const float *x, const uint32_t *cu_seqlens, float *out, uint32_t seqs, uint32_t width,
                 int normalize, void *stream);

/* gates[r, :] = softmax(x[r, ids[r, :]]) — the router's `take` + `softmax`
 * (engine/models/src/decoder.rs:73-75).  x f32 [rows, width], ids u32 [rows, k], gates f32. */
int ts_take_softmax(const float *x, const uint32_t *ids, float *gates, uint32_t rows, uint32_t width,
                    uint32_t k, void *stream);

/* ---------------------------------------------------------------------------
 * Routed experts.  Replaces the `picked` matmuls (engine/rules/linear/src/picked.rs:28-60, arguments
 * `x, w, ids, out, rows, n, k, count, stride, offset, repeat, first`; engine/ir/interp/src/cpu.rs:89-105)
 * and the `mix` (cpu.rs:449-473) of the reference's MoE block (engine/models/src/decoder.rs:70-84):
 *     expert_e(x) = (silu(x W_gate[e]^T) * (x W_up[e]^T)) W_down[e]^T
 *   w_in  [experts, 2 * ffn, hidden] bf16: each expert's gate rows, then its up rows
 *   w_out [experts, hidden, ffn] bf16
 * `experts` is the number of experts in these tables and `first` the global id of the first one: a
 * pick whose id falls outside [first, first + experts) contributes zeros, the reference's rule for
 * experts another rank holds (picked.rs:49-59).  The inner rows pass through bf16.
 * ------------------------------------------------------------------------- */
size_t ts_moe_workspace_bytes(uint32_t picks, uint32_t experts, uint32_t hidden, uint32_t ffn);

/* out[i, :] = expert_{ids[i]}(x[i / repeat, :]) for i < picks; x bf16 [picks / repeat, hidden], out f32. */
int ts_moe_experts_bf16(const void *x, const uint32_t *ids, const void *w_in, const void *w_out, float *out,
                        uint32_t picks, uint32_t repeat, uint32_t experts, uint32_t first, uint32_t hidden,
                        uint32_t ffn, void *workspace, size_t workspace_bytes, void *stream);

/* y[r, :] = sum_p gates[r, p] * expert_{ids[r, p]}(h[r, :]) in pick order p = 0..top-1, plus add[r, :]
 * when add is not NULL (the shared expert's output, engine/models/src/mla.rs:466-467).
 *   h bf16 [rows, hidden]; ids u32 [rows, top]; gates f32 [rows, top]; add, y f32 [rows, hidden]. */
int ts_moe_bf16(const void *h, const uint32_t *ids, const float *gates, const float *add, const void *w_in,
                const void *w_out, float *y, uint32_t rows, uint32_t top, uint32_t experts, uint32_t first,
                uint32_t hidden, uint32_t ffn, void *workspace, size_t workspace_bytes, void *stream);

/* One `picked` launch on its own, with the reference's argument list (engine/rules/linear/src/picked.rs:28-60):
 *     out[i, col] = sum_j x[i / repeat, j] * w[(ids[i] - first) * stride + offset + col, j]      col < n, j < k
 * and zeros where ids[i] falls outside [first, first + count).  x bf16 [rows / repeat, k]; w bf16, `count`
 * matrices `stride` rows apart, of which this launch reads rows [offset, offset + n) (the gate or the up half of a
 * fused table, say); ids u32 [rows]; out f32 [rows, n].  With n a multiple of 128 and k of 64, rows are grouped by matrix
 * (stable counting sort, integer work) so that each matrix streams once per 32 rows that picked it; any other
 * size runs a warp per output element (the reference's own case is 4 matrices of 64 x 32). */
size_t ts_picked_workspace_bytes(uint32_t rows, uint32_t n, uint32_t k, uint32_t count);

int ts_picked_bf16(const void *x, const void *w, const uint32_t *ids, float *out, uint32_t rows, uint32_t n, uint32_t k,
                   uint32_t count, uint32_t stride, uint32_t offset, uint32_t repeat, uint32_t first, void *workspace,
                   size_t workspace_bytes, void *stream);

/* The `mix` alone (engine/ir/interp/src/cpu.rs:449-473): out[r, :] = sum_p gates[r, p] * y_picks[r * top + p, :]
 * in pick order, plus add[r, :] when add is not NULL.  For expert-parallel runs, where the per-pick outputs
 * come back from the ranks that hold the experts.  All f32. */
int ts_moe_mix(const float *y_picks, const float *gates, const float *add, float *out, uint32_t rows, uint32_t top,
               uint32_t hidden, void *stream);

/* The token permutation alone (integer work, the same bits on every run): order[j] = index of the
 * j-th pick when picks are sorted by expert, stable in pick index; place[i] = j with order[j] = i, or
 * UINT32_MAX for a pick of an expert outside [first, first + experts); offsets[e] = first j of expert e
 * (experts + 1 entries); batch_tiles[e] = prefix sum of ceil(count_e / 32) (experts + 1 entries). */
int ts_moe_permutation(const uint32_t *ids, uint32_t *order, uint32_t *place, uint32_t *offsets,
                       uint32_t *batch_tiles, uint32_t picks, uint32_t experts, uint32_t first, void *stream);

/* Programmatic dependent launch on every kernel of this library (off by default): a kernel's
 * weight prefetch then overlaps the tail of the kernel before it, as the reference's `pdl` launch
 * setting does (engine/gpu/gpukit/src/cuda/context.rs:126-148). Process-wide. */
int ts_set_pdl(int enabled);

/* Reads and clears the device-side status word: TS_OK, or TS_ERR_TIMEOUT when a bounded wait
 * inside a tcgen05 kernel gave up (engine/rules/device/include/tessera/status.h:9-39 keeps the same
 * kind of record).  Synchronises the device. */
int ts_device_status(void);

/* ---------------------------------------------------------------------------
 * Narrow weights, first form: Q8_0 (engine/ir/mem/src/block.rs:259-260; the matmul rules accept it through
 * engine/plan/codegen/src/block.rs:209-215).  A matrix [n, k] (k a multiple of 32) is its elements in row-major
 * order cut into blocks of 32: an f16 scale (little endian), then 32 signed bytes; 34 bytes a block, a row is
 * k / 32 blocks.  ts_q8_0_pack / ts_q8_0_unpack are the form's host-side pack and unpack (block.rs:223-258:
 * scale = max |x| / 127 as stored in f16, codes rounded ties-to-even and clamped); ts_q8_0_bytes the packed size.
 *
 * ts_linear_q8_0: out[m, n] = sum_k x[m, k] * w[n, k] (+ epilogue as ts_linear_bf16) for decode-sized launches:
 * 1 <= m <= 64, n a multiple of 64, k a multiple of 256; x bf16, w packed Q8_0 on the device, f32 sums by the
 * form's dot product (block.rs:204-221: per block the sum of x times code, times the scale).  Other sizes return
 * TS_ERR_BAD_INPUT: dequantise (ts_q8_0_unpack) and use ts_linear_bf16.
 * ------------------------------------------------------------------------- */
size_t ts_q8_0_bytes(size_t elements);
int ts_q8_0_pack(const float *data, size_t elements, void *out);
int ts_q8_0_unpack(const void *bytes, size_t elements, float *out);
size_t ts_linear_q8_0_workspace_bytes(uint32_t m, uint32_t n, uint32_t k);
int ts_linear_q8_0(const void *x, const void *w_q8_0, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                   int epilogue, float scale, int out_dtype, void *workspace, size_t workspace_bytes, void *stream);

/* The B200 entry of the reference's platform table plus what the current device reports, as JSON text:
 *   {"row": <the table row: matches "cuda sm_100", tile = bf16_tile = [128, 256, 16] (tcgen05.mma, M x N x K with
 *            N up to 256), pdl, check ["sm_100a"], and under "b200" what the reference's `Needs` has no field for
 *            yet: the paired-SM tile, TMEM columns, cluster size, shared memory per block, the library and ABI>,
 *    "asked": <backend, arch, name, driver, units, memory, bandwidth, limits as the reference's `Asked`
 *              (engine/gpu/platform/src/platform.rs:72-84), "fits": whether this library's kernels run there;
 *              null without a device>}
 * The row is the content of tessera_b200/platforms/cuda-b200.json, which refines
 * engine/gpu/platform/platforms/cuda-blackwell.json:1-21 (that row still names the mma.sync tiles) the way
 * engine/gpu/platform/src/platform.rs:11-29 `Row` is read.  Needs no device. */
int ts_platform_info(char *out, size_t capacity);

/* Runs a one-block kernel whose only act is a bounded wait on a barrier nothing arrives at, with `wait_ns`
 * as the bound, and waits for it.  The wait gives up, and the next ts_device_status() reads TS_ERR_TIMEOUT: the
 * give-up path every waiting kernel of this library shares (bounded poll -> flag -> status word), made
 * observable without a fault or a hang.  The reference tests its bounded spins the same way, against a
 * flag nothing sets (engine/rules/device/include/tessera/status.h:9-39). */
int ts_wait_runs_out(uint64_t wait_ns, void *stream);

/* ---------------------------------------------------------------------------
 * Launch by the reference's kernel names.  `args` is the list the reference's runner builds for a planned
 * launch, in the kernel's parameter order: read buffers, the output buffer, the page table if the kept layout
 * has one, then the u32 / f32 scalars, the layout's own scalar last (engine/plan/lower/src/abi.rs:11-18, 148-153;
 * engine/plan/lower/src/rule.rs:62-109).  Names (ts_kernel_info_at lists them with their signatures):
 *   lanes_bf16, thin_bf16, tiled_bf16, parts_bf16      x, w, out, [m,] n, k  (m from shape->down when left out)
 *   attend_rows_<layout>, flash_rows_<layout>           q, k, v, out, slots, positions, [table], queries, keys,
 *                                                       heads, kv_heads, width, back, <kept scalar>
 *   scatter_<layout>                                    x, slots, positions, out, [table], rows, width, <kept scalar>
 *   top_k                                               x (f32), out (u32), rows, width, k
 *   lane_norm (f32 out), lane_norm_bf16                 x (f32), w, out, rows, width, eps
 *   flash_128, flash_256 (one sequence per launch)      q, k, v, out, queries, keys, past, heads, kv_heads, back, ahead
 * <layout> = dense | interleaved | paged | paged16, as in the reference's `plan_attend_rows_<layout>`.  Queries
 * arrive already scaled, as the reference scales them in a launch of its own.  The list is checked against the
 * kernel's signature before anything is launched; a mismatch is TS_ERR_BAD_INPUT.  `shape` is advisory (the
 * kernels size their own grids) except for the rows of a five-argument linear. */
typedef enum { TS_ARG_PTR = 0, TS_ARG_U32 = 1, TS_ARG_F32 = 2 } ts_arg_kind;

typedef struct {
    int kind; /* ts_arg_kind */
    union {
        void *ptr;
        uint32_t u32;
        float f32;
    } v;
} ts_arg;

typedef struct {
    uint32_t across, down, threads; /* Shape::Grid of the reference (engine/plan/lower/src/abi.rs:119-123) */
} ts_shape;

typedef struct {
    const char *name;
    const char *signature; /* one letter per argument: p = device pointer, u = u32, f = f32 */
    int order;             /* 0: same bits in any batch (Order::Fixed); 1: deterministic per configuration */
} ts_kernel_info;

int ts_kernel_count(void);
int ts_kernel_info_at(int index, ts_kernel_info *out);
size_t ts_launch_workspace_bytes(const char *kernel, const ts_arg *args, int nargs, const ts_shape *shape);
int ts_launch(const char *kernel, const ts_arg *args, int nargs, const ts_shape *shape, void *workspace,
              size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif
