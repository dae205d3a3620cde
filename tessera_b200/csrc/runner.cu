// The host side of the decoder: owns the plan's buffers, binds arguments, enqueues the step
// list and replays it as a CUDA graph keyed by the bound sizes - the part tessera-run's CUDA
// backend plays for a lowered plan (engine/plan/run/src/device.rs:128-242, 348-419;
// engine/plan/run/src/run.rs:122-345).  The step list is the Qwen3-shaped decoder of
// engine/models/src/decoder.rs:281-389.
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "tessera_b200_run.h"
#include "ts_kernels.cuh"

using namespace ts;

struct ts_decoder {
    ts_decoder_config c;
    uint32_t qkv_n, page_rows, kept_pages, kept_total_rows;
    // weights
    uint16_t *embed = nullptr;
    float *norm = nullptr;
    struct Layer {
        uint16_t *wqkv, *wo, *wgu, *wdown;
        float *ln1, *ln2, *q_norm, *k_norm;
        uint16_t *k_rows, *v_rows;
    };
    std::vector<Layer> layers;
    // plan buffers
    float *x = nullptr;          // residual rows [max_rows, hidden] f32
    uint16_t *h = nullptr;       // normed rows [max_rows, hidden]
    uint16_t *qkv = nullptr;     // [max_rows, qkv_n]
    uint16_t *q = nullptr;       // [max_rows, heads * head_dim]
    uint16_t *attn = nullptr;    // [max_rows, heads * head_dim]
    uint16_t *act = nullptr;     // [max_rows, ffn]
    uint16_t *h_out = nullptr;   // final normed rows of the wanted rows [max_rows, hidden]
    float *sumsq = nullptr;      // per-tile sums of squares of the residual rows [max_rows, 32]
    bool last_distinct = false;  // the rows of the last launch sat in slots of their own
    uint16_t *k_dense = nullptr, *v_dense = nullptr;  // packed k, v of a fresh-prompt launch [max_rows, kv_heads, head_dim]
    uint32_t *cu = nullptr;      // device: row offsets of the prompts of such a launch [slots + 1]
    uint32_t fresh_seqs = 0, fresh_longest = 0;  // set by ts_decoder_step for the launch it is about to submit
    float *logits = nullptr;     // [max_out, vocab]
    uint32_t max_out = 0;
    uint32_t *tokens = nullptr, *slots = nullptr, *positions = nullptr, *out_rows = nullptr, *ids = nullptr;
    uint32_t *table = nullptr;
    float *inv_freq = nullptr;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    // pinned staging for feeds and reads
    uint32_t *stage = nullptr;   // 5 * max_rows u32
    // graphs keyed by (rows, keys, n_out, resident)
    std::map<uint64_t, cudaGraphExec_t> graphs;
    uint64_t replays = 0;
    uint32_t last_rows = 0, last_out = 0, last_keys = 0;
    std::vector<uint32_t> host_positions;  // of the last launch, to follow the resident loop
    std::vector<void *> owned;
    // per-kernel device time (tessera_run::Run::profiling / take_profile, run.rs:165-177)
    bool profiling = false;
    std::vector<cudaEvent_t> events;
    size_t events_used = 0;
    std::vector<const char *> event_names;
    std::map<std::string, std::pair<double, uint64_t>> profile;  // name -> (ms, intervals)
    StepKernel *step = nullptr;  // the persistent layer-stack kernel, when the shapes allow it
    bool use_step = false;       // off until ts_decoder_use_step_kernel(dec, 1): slower than the launches it replaces so far
    uint32_t step_keys = 1024;   // decode steps that see more positions than this keep the per-product launches
    cudaStream_t own_stream = nullptr;  // used when the caller passes the NULL stream, which cannot capture
    cudaStream_t last_stream = nullptr; // the stream of the most recent launches
    volatile uint32_t *gate_flag = nullptr;  // pinned; the gate kernel holds the stream until it is set
};

namespace {

template <typename T>
int dev_alloc(ts_decoder *d, T **out, size_t count) {
    void *p = nullptr;
    size_t bytes = count * sizeof(T);
    if (bytes == 0) bytes = 16;
    TS_CUDA(cudaMalloc(&p, bytes));
    TS_CUDA(cudaMemset(p, 0, bytes));  // plan buffers start zeroed (device.rs:397-402)
    d->owned.push_back(p);
    *out = (T *)p;
    return TS_OK;
}

ts_kept kept_of(const ts_decoder *d) {
    ts_kept k = {};
    if (d->c.page == 0) {
        k.kind = TS_KEPT_DENSE;
        k.page = 1;
        k.kept_scalar = d->c.context;
    } else {
        k.kind = TS_KEPT_PAGED;
        k.page = d->c.page;
        k.kept_scalar = d->kept_pages;
        k.table = d->table;
        k.table_len = d->c.slots * d->kept_pages;
    }
    k.rows = d->kept_total_rows;
    return k;
}

size_t max_size(size_t a, size_t b) { return a > b ? a : b; }

// One linear through the kernel family the sizes pick.
int linear_any(ts_decoder *d, const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n,
               uint32_t k, int epi, int out_dtype, cudaStream_t s) {
    const int path = pick_linear_path(m, n, k, epi, TS_LINEAR_AUTO);
    if (path == TS_LINEAR_SKINNY)
        return linear_skinny(x, w, a0, out, m, n, k, epi, 1.0f, out_dtype, d->workspace, d->workspace_bytes, s);
    if (path == TS_LINEAR_STREAM) return linear_stream(x, w, a0, out, m, n, k, epi, 1.0f, out_dtype, s);
    if (path == TS_LINEAR_PAIR) return linear_pair(x, w, a0, out, m, n, k, epi, 1.0f, out_dtype, s);
    if (path == TS_LINEAR_UMMA)
        return linear_umma(x, w, a0, out, m, n, k, epi, 1.0f, out_dtype, d->workspace, d->workspace_bytes, s);
    return fail(TS_ERR_BAD_INPUT, "decoder: no linear kernel takes m=%u n=%u k=%u", m, n, k);
}

size_t linear_workspace(uint32_t m, uint32_t n, uint32_t k, int epi) {
    const int path = pick_linear_path(m, n, k, epi, TS_LINEAR_AUTO);
    if (path == TS_LINEAR_SKINNY) return skinny_workspace_bytes(m, n, k, epi == TS_EPI_SWIGLU || epi == TS_EPI_GEGLU);
    if (path == TS_LINEAR_UMMA) return umma_workspace_bytes(m, n, k, epi);
    return 0;
}

// Partial sums per row when the layer norms can fold into the projections around them (every
// projection of the layer takes the weight-streaming kernel and the two that feed the residual
// split their k), else 0.
uint32_t fold_parts(const ts_decoder *d, uint32_t rows) {
    // TS_FOLD_NORMS=0 keeps every norm a launch of its own (for A/B timing).
    static const bool off = [] {
        const char *v = getenv("TS_FOLD_NORMS");
        return v && v[0] == '0';
    }();
    if (off) return 0;
    const ts_decoder_config &c = d->c;
    const uint32_t H = c.hidden, QW = c.heads * c.head_dim;
    const uint32_t parts = stream_sumsq_parts(rows, H, QW, TS_EPI_ADD);
    const bool ok = parts != 0 && parts <= 32 && stream_sumsq_parts(rows, H, c.ffn, TS_EPI_ADD) == parts &&
                    pick_linear_path(rows, H, QW, TS_EPI_ADD, TS_LINEAR_AUTO) == TS_LINEAR_STREAM &&
                    pick_linear_path(rows, H, c.ffn, TS_EPI_ADD, TS_LINEAR_AUTO) == TS_LINEAR_STREAM &&
                    pick_linear_path(rows, d->qkv_n, H, TS_EPI_NONE, TS_LINEAR_AUTO) == TS_LINEAR_STREAM &&
                    pick_linear_path(rows, 2 * c.ffn, H, TS_EPI_SWIGLU, TS_LINEAR_AUTO) == TS_LINEAR_STREAM;
    return ok ? parts : 0;
}

// TS_FRESH_PROMPTS=0 sends whole prompts through the kept-row attention like any other launch (for A/B).
bool early_keys_enabled() {
    static const bool on = [] {
        const char *e = getenv("TS_EARLY_KEYS");
        return !(e && e[0] == '0');
    }();
    return on;
}

bool fresh_prompts_enabled() {
    static const bool off = [] {
        const char *v = getenv("TS_FRESH_PROMPTS");
        return v && v[0] == '0';
    }();
    return !off;
}

// Whether the attention launch also does the per-head norm, the rotation and the append: only when no
// two rows of the launch share a slot (a row must not read a key that another row of the same launch
// appends), at head width 128 over a layout the TMA-fed kernel takes.  TS_FUSE_APPEND=0 turns it off.
bool append_in_attention(const ts_decoder *d, bool distinct) {
    static const bool off = [] {
        const char *v = getenv("TS_FUSE_APPEND");
        return v && v[0] == '0';
    }();
    const bool contiguous = d->c.page == 0 || d->c.page >= 32;
    return !off && distinct && attend_rows_fused_supports(contiguous, d->c.head_dim, d->kept_total_rows);
}

// Whether this launch's gather and layers run as the one persistent kernel: a decode step (every row in a slot of
// its own) of at most 64 rows within the context limit.
bool takes_step_kernel(const ts_decoder *d, uint32_t rows, uint32_t keys, bool distinct) {
    return d->step && d->use_step && distinct && d->fresh_seqs == 0 && rows <= step_kernel_max_rows() &&
           keys <= d->step_keys;
}

// The step list for `rows` rows that see at most `keys` positions; logits for n_out rows.
int enqueue(ts_decoder *d, uint32_t rows, uint32_t keys, uint32_t n_out, bool feedback, bool distinct, cudaStream_t s,
            uint32_t *count) {
    const ts_decoder_config &c = d->c;
    const uint32_t H = c.hidden, D = c.head_dim, QW = c.heads * D;
    uint32_t launches = 0;
    int rc;
    ts_kept kept = kept_of(d);
    KeptDev kd;
    if ((rc = kept_to_dev(&kept, &kd)) != TS_OK) return rc;
    const bool contiguous = kept.kind == TS_KEPT_DENSE || kept.page >= 32;
    const float scale = 1.0f / sqrtf((float)D);
    auto mark = [&](const char *name) -> int {
        if (!d->profiling) return TS_OK;
        if (d->events_used == d->events.size()) {
            cudaEvent_t e;
            TS_CUDA(cudaEventCreate(&e));
            d->events.push_back(e);
        }
        TS_CUDA(cudaEventRecord(d->events[d->events_used++], s));
        d->event_names.push_back(name);
        return TS_OK;
    };
#define STEP(name, expr)                       \
    do {                                       \
        if ((rc = (expr)) != TS_OK) return rc; \
        if ((rc = mark(name)) != TS_OK) return rc; \
        launches++;                            \
    } while (0)
    auto linear = [&](const void *xin, const void *w, const void *a0, void *out, uint32_t n, uint32_t k, int epi,
                      int out_dtype) -> int {
        return linear_any(d, xin, w, a0, out, rows, n, k, epi, out_dtype, s);
    };
    // Decode-sized steps fold the layer norms into the projections on either side: the embedding gather
    // and the o and down projections leave bf16(row * gain) in d->h and the rows' sums of squares in
    // d->sumsq; the q,k,v and gate/up projections multiply their output rows by 1/rms.  Only the final
    // norm (over the wanted rows) stays a launch.
    const uint32_t ss_parts = fold_parts(d, rows);
    const bool fold = ss_parts != 0;
    // x_in: bf16(residual * gain) as the upstream step left it in d->h; next_gain: the gain of the norm
    // that follows this linear's output (NULL: none follows inside the layer stack).
    auto folded = [&](bool scaled_in, const void *xin, const void *w, const void *a0, void *out, uint32_t n, uint32_t k,
                      int epi, int out_dtype, const float *next_gain) -> int {
        StreamFused f;
        if (scaled_in) {
            f.row_ss = d->sumsq;
            f.row_parts = ss_parts;
            f.row_eps = c.eps;
        }
        if (next_gain) {
            f.ss_out = d->sumsq;
            f.xs_out = d->h;
            f.xs_gain = next_gain;
        }
        return linear_stream(xin, w, a0, out, rows, n, k, epi, 1.0f, out_dtype, s, &f);
    };
    if ((rc = mark("")) != TS_OK) return rc;  // interval origin
    if (feedback) STEP("advance_rows", advance_rows(d->ids, d->tokens, d->positions, rows, s));
    const bool one_kernel = takes_step_kernel(d, rows, keys, distinct);
    if (one_kernel) {
        STEP("decode_layers", step_kernel_launch(d->step, rows, keys, kd, s));
    } else if (fold) {
        STEP("gather", gather_scaled(d->embed, d->tokens, d->x, d->h, d->layers[0].ln1, d->sumsq, ss_parts, rows, c.vocab, H, s));
    } else {
        STEP("gather", gather_rows(d->embed, d->tokens, d->x, TS_F32, rows, c.vocab, H, 0, s));
    }
    for (uint32_t l = 0; l < c.layers && !one_kernel; l++) {
        ts_decoder::Layer &L = d->layers[l];
        if (fold) {
            STEP("linear_qkv", folded(true, d->h, L.wqkv, nullptr, d->qkv, d->qkv_n, H, TS_EPI_NONE, TS_BF16, nullptr));
        } else {
            STEP("rms_norm", rms_norm(d->x, TS_F32, L.ln1, d->h, TS_BF16, rows, H, c.eps, nullptr, s));
            STEP("linear_qkv", linear(d->h, L.wqkv, nullptr, d->qkv, d->qkv_n, H, TS_EPI_NONE, TS_BF16));
        }
        if (d->fresh_seqs > 0) {
            // Whole prompts from position 0: every key a row may see was made in this launch, so attention runs
            // over the packed q, k, v with the tensor-core kernel; the kept rows are still written for later steps.
            STEP("qk_norm_rope_append", qk_norm_rope_append(d->qkv, c.qk_norm ? L.q_norm : nullptr, c.qk_norm ? L.k_norm : nullptr, d->inv_freq,
                                     d->slots, d->positions, d->q, L.k_rows, L.v_rows, kd, rows, c.heads, c.kv_heads, D,
                                     c.eps, s, d->k_dense, d->v_dense));
            STEP("attend_flash", attend_flash(d->q, d->k_dense, d->v_dense, d->attn, d->cu, d->fresh_seqs, d->fresh_longest, rows, rows,
                              rows, c.heads, c.kv_heads, D, 0xFFFFFFFFu, 0, scale, s));
        } else if (append_in_attention(d, distinct)) {
            // One row per slot (a decode step): the attention kernel norms, rotates and appends itself.
            RowsFused f;
            f.qkv = d->qkv;
            f.q_norm = c.qk_norm ? L.q_norm : nullptr;
            f.k_norm = c.qk_norm ? L.k_norm : nullptr;
            f.inv_freq = d->inv_freq;
            f.eps = c.eps;
            // This layer's kept rows were last written a whole step ago, the slots and positions before the
            // step's first launch, and the upstream launch is this layer's q,k,v projection.
            f.early_keys = early_keys_enabled();
            STEP("attend_rows", attend_rows(nullptr, L.k_rows, L.v_rows, d->attn, d->slots, d->positions, kd, contiguous, rows, keys,
                             c.heads, c.kv_heads, D, 0xFFFFFFFFu, scale, d->workspace, d->workspace_bytes, s, 0, nullptr,
                             d->kept_total_rows, &f));
        } else {
            STEP("qk_norm_rope_append", qk_norm_rope_append(d->qkv, c.qk_norm ? L.q_norm : nullptr, c.qk_norm ? L.k_norm : nullptr, d->inv_freq,
                                     d->slots, d->positions, d->q, L.k_rows, L.v_rows, kd, rows, c.heads, c.kv_heads, D,
                                     c.eps, s));
            STEP("attend_rows", attend_rows(d->q, L.k_rows, L.v_rows, d->attn, d->slots, d->positions, kd, contiguous, rows, keys, c.heads,
                             c.kv_heads, D, 0xFFFFFFFFu, scale, d->workspace, d->workspace_bytes, s, 0, nullptr,
                             d->kept_total_rows));
        }
        if (attend_rows_workspace_bytes(rows, keys, c.heads, c.kv_heads, D) > 0) launches++;
        if (fold) {
            STEP("linear_o", folded(false, d->attn, L.wo, d->x, d->x, H, QW, TS_EPI_ADD, TS_F32, L.ln2));
            STEP("linear_gate_up", folded(true, d->h, L.wgu, nullptr, d->act, 2 * c.ffn, H, TS_EPI_SWIGLU, TS_BF16, nullptr));
            STEP("linear_down", folded(false, d->act, L.wdown, d->x, d->x, H, c.ffn, TS_EPI_ADD, TS_F32,
                                       l + 1 < c.layers ? d->layers[l + 1].ln1 : nullptr));
        } else {
            STEP("linear_o", linear(d->attn, L.wo, d->x, d->x, H, QW, TS_EPI_ADD, TS_F32));
            STEP("rms_norm", rms_norm(d->x, TS_F32, L.ln2, d->h, TS_BF16, rows, H, c.eps, nullptr, s));
            STEP("linear_gate_up", linear(d->h, L.wgu, nullptr, d->act, 2 * c.ffn, H, TS_EPI_SWIGLU, TS_BF16));
            STEP("linear_down", linear(d->act, L.wdown, d->x, d->x, H, c.ffn, TS_EPI_ADD, TS_F32));
        }
    }
    // Only the wanted rows go through the final norm and the unembedding.
    STEP("rms_norm", rms_norm(d->x, TS_F32, d->norm, d->h_out, TS_BF16, n_out, H, c.eps, n_out == rows ? nullptr : d->out_rows, s));
    STEP("linear_unembed", linear_any(d, d->h_out, d->embed, nullptr, d->logits, n_out, c.vocab, H, TS_EPI_NONE, TS_F32, s));
    STEP("top_1", top_k(d->logits, TS_F32, d->ids, n_out, c.vocab, 1, d->workspace, d->workspace_bytes, s));
    launches++;  // top-1 over the vocabulary is two launches
#undef STEP
    if (count) *count = launches;
    return TS_OK;
}

// Replays the captured graph for these sizes, capturing it on first sight.
int submit(ts_decoder *d, uint32_t rows, uint32_t keys, uint32_t n_out, bool feedback, bool distinct, cudaStream_t s,
           bool capture_only = false) {
    set_pdl(d->c.pdl != 0);
    if (!d->c.graphs) return capture_only ? TS_OK : enqueue(d, rows, keys, n_out, feedback, distinct, s, nullptr);
    const uint64_t key = ((uint64_t)(distinct ? 1 : 0) << 63) | ((uint64_t)rows << 40) | ((uint64_t)keys << 16) |
                         ((uint64_t)(n_out & 0x7FFF) << 1) | (feedback ? 1 : 0);
    auto it = d->graphs.find(key);
    if (it == d->graphs.end()) {
        cudaGraph_t graph = nullptr;
        TS_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed));
        int rc = enqueue(d, rows, keys, n_out, feedback, distinct, s, nullptr);
        cudaError_t e = cudaStreamEndCapture(s, &graph);
        if (rc != TS_OK) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        if (e != cudaSuccess) return fail(TS_ERR_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return fail(TS_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
        it = d->graphs.emplace(key, exec).first;
    }
    if (capture_only) return TS_OK;
    TS_CUDA(cudaGraphLaunch(it->second, s));
    d->replays++;
    return TS_OK;
}

// The legacy NULL stream cannot be captured into a graph: fall back to the runner's own stream
// (a blocking stream, so it still orders against work on the NULL stream).
cudaStream_t stream_of(ts_decoder *d, void *stream) {
    cudaStream_t s = stream ? (cudaStream_t)stream : d->own_stream;
    d->last_stream = s;  // what a later table or weight update has to wait for
    return s;
}

// Before the host overwrites something launches read (the page table, a weight): everything this decoder
// launched last, on whatever stream, must be over.  A resident loop returns without waiting, and its launches
// read the table without any dependency on the legacy stream the blocking copies below run on.
int settle(ts_decoder *d) {
    if (d->last_stream) TS_CUDA(cudaStreamSynchronize(d->last_stream));
    return TS_OK;
}

uint32_t keys_bucket(const ts_decoder *d, uint32_t furthest) {
    uint32_t k = (furthest + 127) / 128 * 128;
    return k > d->c.context ? d->c.context : k;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int ts_decoder_create(const ts_decoder_config *config, ts_decoder **out) {
    TS_REQUIRE(config && out, "decoder: config and out must not be NULL");
    const ts_decoder_config &c = *config;
    TS_REQUIRE(c.layers && c.hidden && c.heads && c.kv_heads && c.head_dim && c.ffn && c.vocab && c.slots &&
                   c.context && c.max_rows,
               "decoder: every size must be positive");
    TS_REQUIRE(c.heads % c.kv_heads == 0, "decoder: %u heads do not split over %u kv heads", c.heads, c.kv_heads);
    TS_REQUIRE(c.head_dim == 64 || c.head_dim == 128 || c.head_dim == 256, "decoder: head_dim %u is not 64, 128 or 256",
               c.head_dim);
    TS_REQUIRE(c.page == 0 || c.page == 16 || c.page == 64, "decoder: page %u is not 0, 16 or 64", c.page);
    TS_REQUIRE(c.hidden % 256 == 0 && c.ffn % 256 == 0 && (c.heads * c.head_dim) % 256 == 0,
               "decoder: hidden, ffn and heads * head_dim must be multiples of 256");
    int dev_count = 0;
    if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0)
        return fail(TS_ERR_CUDA, "decoder: no CUDA device (there is no CPU path)");
    ts_decoder *d = new ts_decoder();
    d->c = c;
    d->qkv_n = (c.heads + 2 * c.kv_heads) * c.head_dim;
    d->page_rows = c.page ? c.page : 1;
    d->kept_pages = c.page ? (c.context + c.page - 1) / c.page : c.context;
    d->kept_total_rows = c.page ? c.slots * d->kept_pages * c.page : c.slots * c.context;
    d->max_out = c.max_rows < 256 ? c.max_rows : 256;
    int rc = TS_OK;
    auto A = [&](int r) { if (rc == TS_OK) rc = r; };
    const size_t H = c.hidden, QW = (size_t)c.heads * c.head_dim, KW = (size_t)c.kv_heads * c.head_dim;
    A(dev_alloc(d, &d->embed, (size_t)c.vocab * H));
    A(dev_alloc(d, &d->norm, H));
    d->layers.resize(c.layers);
    {
        // Every layer's copy of a weight (and of the kept K and V rows) sits in one slab, layer after layer: one
        // tensor map then covers all layers of that weight, which the persistent decode kernel relies on.
        const size_t n_qkv = (size_t)d->qkv_n * H, n_o = H * QW, n_gu = (size_t)2 * c.ffn * H, n_down = H * c.ffn;
        const size_t n_kept = (size_t)d->kept_total_rows * KW;
        uint16_t *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wdown = nullptr, *k_rows = nullptr, *v_rows = nullptr;
        A(dev_alloc(d, &wqkv, c.layers * n_qkv));
        A(dev_alloc(d, &wo, c.layers * n_o));
        A(dev_alloc(d, &wgu, c.layers * n_gu));
        A(dev_alloc(d, &wdown, c.layers * n_down));
        A(dev_alloc(d, &k_rows, c.layers * n_kept));
        A(dev_alloc(d, &v_rows, c.layers * n_kept));
        for (uint32_t l = 0; l < c.layers && rc == TS_OK; l++) {
            ts_decoder::Layer &L = d->layers[l];
            L.wqkv = wqkv + l * n_qkv;
            L.wo = wo + l * n_o;
            L.wgu = wgu + l * n_gu;
            L.wdown = wdown + l * n_down;
            L.k_rows = k_rows + l * n_kept;
            L.v_rows = v_rows + l * n_kept;
            A(dev_alloc(d, &L.ln1, H));
            A(dev_alloc(d, &L.ln2, H));
            A(dev_alloc(d, &L.q_norm, c.head_dim));
            A(dev_alloc(d, &L.k_norm, c.head_dim));
        }
    }
    const size_t R = c.max_rows;
    A(dev_alloc(d, &d->x, R * H));
    A(dev_alloc(d, &d->h, R * H));
    A(dev_alloc(d, &d->qkv, R * d->qkv_n));
    A(dev_alloc(d, &d->q, R * QW));
    A(dev_alloc(d, &d->attn, R * QW));
    A(dev_alloc(d, &d->act, R * c.ffn));
    A(dev_alloc(d, &d->h_out, R * H));
    A(dev_alloc(d, &d->sumsq, R * 32));
    A(dev_alloc(d, &d->k_dense, R * KW));
    A(dev_alloc(d, &d->v_dense, R * KW));
    A(dev_alloc(d, &d->cu, (size_t)c.slots + 1));
    A(dev_alloc(d, &d->logits, (size_t)d->max_out * c.vocab));
    A(dev_alloc(d, &d->tokens, R));
    A(dev_alloc(d, &d->slots, R));
    A(dev_alloc(d, &d->positions, R));
    A(dev_alloc(d, &d->out_rows, R));
    A(dev_alloc(d, &d->ids, R));
    A(dev_alloc(d, &d->table, (size_t)c.slots * d->kept_pages));
    A(dev_alloc(d, &d->inv_freq, c.head_dim / 2));
    // One workspace for every step: the largest any of them asks for at max_rows.
    size_t ws = 0;
    std::vector<uint32_t> row_counts = {1u, 8u, 16u, 32u, 64u, 128u, c.max_rows, d->max_out};
    for (uint32_t rows = 129; rows < 512 && rows <= c.max_rows; rows++) row_counts.push_back(rows);  // tiled kernel, k split by tile count
    for (uint32_t rows : row_counts) {
        if (rows > c.max_rows) continue;
        auto need = [&](uint32_t n, uint32_t k, int epi) { return linear_workspace(rows, n, k, epi); };
        ws = max_size(ws, need(d->qkv_n, c.hidden, TS_EPI_NONE));
        ws = max_size(ws, need(c.hidden, c.heads * c.head_dim, TS_EPI_ADD));
        ws = max_size(ws, need(2 * c.ffn, c.hidden, TS_EPI_SWIGLU));
        ws = max_size(ws, need(c.hidden, c.ffn, TS_EPI_ADD));
        if (rows <= d->max_out) ws = max_size(ws, need(c.vocab, c.hidden, TS_EPI_NONE));
        ws = max_size(ws, attend_rows_workspace_bytes(rows, c.context, c.heads, c.kv_heads, c.head_dim));
        ws = max_size(ws, top_k_workspace_bytes(rows, c.vocab, 1));
    }
    d->workspace_bytes = ws + 256;
    if (rc == TS_OK) {
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, d->workspace_bytes);
        if (e != cudaSuccess) rc = fail(TS_ERR_CUDA, "cudaMalloc of the workspace failed: %s", cudaGetErrorString(e));
        else { d->workspace = p; d->owned.push_back(p); }
    }
    if (rc == TS_OK) {
        cudaError_t e = cudaMallocHost((void **)&d->stage, 6 * R * sizeof(uint32_t));
        if (e != cudaSuccess) rc = fail(TS_ERR_CUDA, "cudaMallocHost failed: %s", cudaGetErrorString(e));
    }
    if (rc == TS_OK) {
        cudaError_t e = cudaStreamCreate(&d->own_stream);
        if (e != cudaSuccess) rc = fail(TS_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(e));
    }
    if (rc == TS_OK) {
        std::vector<float> f(c.head_dim / 2);
        for (uint32_t j = 0; j < c.head_dim / 2; j++) f[j] = powf(c.theta, -((float)(2 * j)) / (float)c.head_dim);
        cudaError_t e = cudaMemcpy(d->inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice);
        std::vector<uint32_t> t((size_t)c.slots * d->kept_pages);
        for (size_t i = 0; i < t.size(); i++) t[i] = (uint32_t)i;  // identity: lanes.rs:4-65
        if (e == cudaSuccess) e = cudaMemcpy(d->table, t.data(), t.size() * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) rc = fail(TS_ERR_CUDA, "initial uploads failed: %s", cudaGetErrorString(e));
    }
    if (rc == TS_OK) {
        StepKernelShape shape = {c.layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.ffn, c.vocab, c.page,
                                 d->kept_total_rows, c.max_rows, c.eps, c.qk_norm};
        if (step_kernel_supports(shape)) {
            std::vector<StepKernelLayer> layers(c.layers);
            for (uint32_t l = 0; l < c.layers; l++) {
                const ts_decoder::Layer &L = d->layers[l];
                layers[l] = {L.wqkv, L.wo, L.wgu, L.wdown, L.ln1, L.ln2, L.q_norm, L.k_norm, L.k_rows, L.v_rows};
            }
            StepKernelBuffers buffers = {layers.data(), d->embed, d->x, d->h, d->attn, d->act, d->qkv,
                                         d->tokens, d->slots, d->positions, d->inv_freq};
            rc = step_kernel_create(shape, buffers, &d->step);
            if (const char *v = getenv("TS_STEP_KERNEL_KEYS")) d->step_keys = std::min<uint32_t>((uint32_t)atoi(v), 1024u);
        }
    }
    if (rc != TS_OK) {
        ts_decoder_destroy(d);
        return rc;
    }
    *out = d;
    return TS_OK;
}

int ts_decoder_use_step_kernel(ts_decoder *d, int on) {
    if (!d) return 0;
    const bool want = on != 0;
    if (want != d->use_step) {
        // captured graphs hold the other form of the step
        for (auto &g : d->graphs) cudaGraphExecDestroy(g.second);
        d->graphs.clear();
        d->use_step = want;
    }
    return d->step != nullptr ? 1 : 0;
}

void ts_decoder_destroy(ts_decoder *d) {
    if (!d) return;
    for (auto &g : d->graphs) cudaGraphExecDestroy(g.second);
    step_kernel_destroy(d->step);
    for (void *p : d->owned) cudaFree(p);
    if (d->stage) cudaFreeHost(d->stage);
    if (d->gate_flag) cudaFreeHost((void *)d->gate_flag);
    if (d->own_stream) cudaStreamDestroy(d->own_stream);
    for (cudaEvent_t e : d->events) cudaEventDestroy(e);
    delete d;
}

int ts_decoder_load(ts_decoder *d, const char *name, const void *host, size_t bytes) {
    TS_REQUIRE(d && name && host, "decoder load: NULL argument");
    const ts_decoder_config &c = d->c;
    const size_t H = c.hidden, D = c.head_dim, QW = (size_t)c.heads * D, KW = (size_t)c.kv_heads * D, F = c.ffn;
    void *dst = nullptr;
    size_t want = 0;
    std::string n(name);
    if (n == "embed") { dst = d->embed; want = (size_t)c.vocab * H * 2; }
    else if (n == "norm") { dst = d->norm; want = H * 4; }
    else if (n.rfind("layers.", 0) == 0) {
        size_t dot = n.find('.', 7);
        TS_REQUIRE(dot != std::string::npos, "decoder load: weight name '%s' is malformed", name);
        const uint32_t l = (uint32_t)atoi(n.substr(7, dot - 7).c_str());
        TS_REQUIRE(l < c.layers, "decoder load: layer %u is past the %u layers", l, c.layers);
        ts_decoder::Layer &L = d->layers[l];
        const std::string f = n.substr(dot + 1);
        if (f == "ln1") { dst = L.ln1; want = H * 4; }
        else if (f == "ln2") { dst = L.ln2; want = H * 4; }
        else if (f == "q_norm") { dst = L.q_norm; want = D * 4; }
        else if (f == "k_norm") { dst = L.k_norm; want = D * 4; }
        else if (f == "q") { dst = L.wqkv; want = QW * H * 2; }
        else if (f == "k") { dst = L.wqkv + QW * H; want = KW * H * 2; }
        else if (f == "v") { dst = L.wqkv + (QW + KW) * H; want = KW * H * 2; }
        else if (f == "o") { dst = L.wo; want = H * QW * 2; }
        else if (f == "mlp.gate") { dst = L.wgu; want = F * H * 2; }
        else if (f == "mlp.up") { dst = L.wgu + F * H; want = F * H * 2; }
        else if (f == "mlp.down") { dst = L.wdown; want = H * F * 2; }
    }
    TS_REQUIRE(dst != nullptr, "decoder load: no weight is called '%s'", name);
    TS_REQUIRE(bytes == want, "decoder load: '%s' wants %zu bytes, got %zu", name, want, bytes);
    int settled = settle(d);
    if (settled != TS_OK) return settled;
    TS_CUDA(cudaMemcpy(dst, host, bytes, cudaMemcpyHostToDevice));
    return TS_OK;
}

int ts_decoder_set_table(ts_decoder *d, const uint32_t *host_table, uint32_t entries) {
    TS_REQUIRE(d && host_table, "decoder table: NULL argument");
    TS_REQUIRE(d->c.page != 0, "decoder table: the kept rows are dense, there is no table");
    const uint32_t want = d->c.slots * d->kept_pages;
    TS_REQUIRE(entries == want, "decoder table: wants %u entries, got %u", want, entries);
    for (uint32_t i = 0; i < entries; i++)
        TS_REQUIRE(host_table[i] < want, "decoder table: entry %u names page %u of %u", i, host_table[i], want);
    int rc = settle(d);
    if (rc != TS_OK) return rc;
    TS_CUDA(cudaMemcpy(d->table, host_table, (size_t)entries * 4, cudaMemcpyHostToDevice));
    return TS_OK;
}

int ts_decoder_copy_pages(ts_decoder *d, const ts_kv_copy *copies, uint32_t n_copies, void *stream) {
    TS_REQUIRE(d && (copies || n_copies == 0), "decoder page copies: NULL argument");
    TS_REQUIRE(d->c.page != 0, "decoder page copies: the kept rows are dense, there are no pages");
    const uint32_t pages = d->c.slots * d->kept_pages;
    for (uint32_t i = 0; i < n_copies; i++)
        TS_REQUIRE(copies[i].from < pages && copies[i].to < pages && copies[i].rows <= d->c.page,
                   "decoder page copies: copy %u (%u -> %u, %u rows) is outside %u pages of %u rows", i, copies[i].from,
                   copies[i].to, copies[i].rows, pages, d->c.page);
    const size_t row_bytes = (size_t)d->c.kv_heads * d->c.head_dim * 2;
    cudaStream_t s = stream_of(d, stream);
    for (auto &L : d->layers) {
        int rc = ts_kv_copy_pages(L.k_rows, copies, n_copies, d->c.page, row_bytes, s);
        if (rc != TS_OK) return rc;
        rc = ts_kv_copy_pages(L.v_rows, copies, n_copies, d->c.page, row_bytes, s);
        if (rc != TS_OK) return rc;
    }
    return TS_OK;
}

int ts_decoder_step(ts_decoder *d, const uint32_t *tokens, const uint32_t *slots, const uint32_t *positions,
                    uint32_t rows, const uint32_t *out_rows, uint32_t n_out, uint32_t *out_ids, void *stream) {
    TS_REQUIRE(d && tokens && slots && positions, "decoder step: NULL argument");
    const ts_decoder_config &c = d->c;
    TS_REQUIRE(rows >= 1 && rows <= c.max_rows, "decoder step: %u rows, the plan takes 1..%u", rows, c.max_rows);
    if (!out_rows) n_out = rows;
    TS_REQUIRE(n_out >= 1 && n_out <= d->max_out, "decoder step: %u output rows, the plan takes 1..%u", n_out, d->max_out);
    uint32_t furthest = 0;
    for (uint32_t r = 0; r < rows; r++) {
        TS_REQUIRE(slots[r] < c.slots, "decoder step: row %u at slot %u is outside the %u slots", r, slots[r], c.slots);
        TS_REQUIRE(positions[r] < c.context, "decoder step: row %u at position %u is past the context of %u", r,
                   positions[r], c.context);
        TS_REQUIRE(tokens[r] < c.vocab, "decoder step: row %u holds token %u of a %u vocabulary", r, tokens[r], c.vocab);
        if (positions[r] + 1 > furthest) furthest = positions[r] + 1;
    }
    for (uint32_t i = 0; out_rows && i < n_out; i++)
        TS_REQUIRE(out_rows[i] < rows, "decoder step: output row %u is past the %u rows", out_rows[i], rows);
    cudaStream_t s = stream_of(d, stream);
    const size_t R = c.max_rows;
    uint32_t *st = d->stage;
    const uint32_t given_rows = rows, given_out = n_out;
    memcpy(st, tokens, rows * 4);
    memcpy(st + R, slots, rows * 4);
    memcpy(st + 2 * R, positions, rows * 4);
    if (out_rows) memcpy(st + 3 * R, out_rows, n_out * 4);
    // Do all rows sit in slots of their own (a decode step), or does a slot take several (a prefill)?
    bool distinct = true;
    {
        std::vector<bool> seen(c.slots, false);
        for (uint32_t r = 0; r < rows && distinct; r++) {
            distinct = !seen[slots[r]];
            seen[slots[r]] = true;
        }
    }
    // A launch of whole prompts: the rows of every slot are consecutive and hold positions 0, 1, 2, ... (a fresh
    // sequence, nothing kept before).  Then attention needs no kept rows and takes the prefill kernel.
    d->fresh_seqs = 0;
    std::vector<uint32_t> cu;
    if (!distinct && flash_supports(c.head_dim) && fresh_prompts_enabled()) {
        bool fresh = true;
        cu.push_back(0);
        uint32_t longest = 0;
        for (uint32_t r = 0; r < rows && fresh; r++) {
            const bool starts = r == 0 || slots[r] != slots[r - 1];
            if (starts) {
                fresh = positions[r] == 0;
                if (r > 0) {
                    longest = std::max(longest, r - cu.back());
                    cu.push_back(r);
                }
            } else {
                fresh = positions[r] == positions[r - 1] + 1;
            }
        }
        if (fresh) {
            // no slot may come back after another one started
            std::vector<bool> seen(c.slots, false);
            for (size_t i = 0; i < cu.size() && fresh; i++) {
                fresh = !seen[slots[cu[i]]];
                seen[slots[cu[i]]] = true;
            }
        }
        if (fresh) {
            longest = std::max(longest, rows - cu.back());
            cu.push_back(rows);
            TS_CUDA(cudaMemcpyAsync(d->cu, cu.data(), cu.size() * 4, cudaMemcpyHostToDevice, s));
            TS_CUDA(cudaStreamSynchronize(s));  // cu is a local: the copy must have read it before it goes away
            d->fresh_seqs = (uint32_t)cu.size() - 1;
            d->fresh_longest = longest;
        }
    }
    const uint32_t keys = keys_bucket(d, furthest);
    // Rows and wanted rows round up to a power of two, the last row (and the last wanted row) filling out, as the
    // reference sizes a launch (engine/engine/src/lib.rs:166-200): a plan, and here a captured graph, then exists per
    // bucket instead of per row count.  The copies rewrite their row's kept K and V with the same values.  Whole
    // prompts (the prefill kernel over packed rows) keep their exact size.
    if (d->fresh_seqs == 0) {
        auto pow2 = [](uint32_t v) {
            uint32_t p = 1;
            while (p < v) p <<= 1;
            return p;
        };
        const uint32_t filled = pow2(rows), wanted = out_rows ? pow2(n_out) : filled;
        if (filled <= c.max_rows && wanted <= d->max_out) {
            for (uint32_t r = rows; r < filled; r++) {
                st[r] = st[rows - 1];
                st[R + r] = st[R + rows - 1];
                st[2 * R + r] = st[2 * R + rows - 1];
            }
            if (out_rows)
                for (uint32_t i = n_out; i < wanted; i++) st[3 * R + i] = st[3 * R + n_out - 1];
            rows = filled;
            n_out = wanted;
        }
    }
    TS_CUDA(cudaMemcpyAsync(d->tokens, st, rows * 4, cudaMemcpyHostToDevice, s));
    TS_CUDA(cudaMemcpyAsync(d->slots, st + R, rows * 4, cudaMemcpyHostToDevice, s));
    TS_CUDA(cudaMemcpyAsync(d->positions, st + 2 * R, rows * 4, cudaMemcpyHostToDevice, s));
    if (out_rows) TS_CUDA(cudaMemcpyAsync(d->out_rows, st + 3 * R, n_out * 4, cudaMemcpyHostToDevice, s));
    int rc;
    if (d->fresh_seqs > 0) {
        // one-off shapes: not worth a captured graph
        set_pdl(d->c.pdl != 0);
        rc = enqueue(d, rows, keys, n_out, false, false, s, nullptr);
        d->fresh_seqs = 0;
    } else {
        rc = submit(d, rows, keys, n_out, false, distinct, s);
    }
    if (rc != TS_OK) return rc;
    d->last_distinct = distinct;
    d->last_rows = rows;
    d->last_out = n_out;
    d->last_keys = furthest;
    d->host_positions.assign(st + 2 * R, st + 2 * R + rows);
    (void)given_rows;
    if (out_ids) {
        TS_CUDA(cudaMemcpyAsync(st + 4 * R, d->ids, given_out * 4, cudaMemcpyDeviceToHost, s));
        TS_CUDA(cudaStreamSynchronize(s));
        memcpy(out_ids, st + 4 * R, given_out * 4);
    } else {
        TS_CUDA(cudaStreamSynchronize(s));
    }
    return TS_OK;
}

int ts_decoder_run_resident(ts_decoder *d, uint32_t steps, void *stream) {
    TS_REQUIRE(d, "decoder: NULL");
    TS_REQUIRE(d->last_rows > 0 && d->last_out == d->last_rows,
               "decoder resident loop: the last launch must have produced one id per row");
    cudaStream_t s = stream_of(d, stream);
    for (uint32_t i = 0; i < steps; i++) {
        const uint32_t furthest = d->last_keys + 1;
        TS_REQUIRE(furthest <= d->c.context, "decoder resident loop: position %u is past the context of %u",
                   furthest - 1, d->c.context);
        int rc = submit(d, d->last_rows, keys_bucket(d, furthest), d->last_rows, true, d->last_distinct, s);
        if (rc != TS_OK) return rc;
        d->last_keys = furthest;
        for (auto &p : d->host_positions) p++;
    }
    return TS_OK;
}

int ts_decoder_read_ids(ts_decoder *d, uint32_t *out_ids, uint32_t rows, void *stream) {
    TS_REQUIRE(d && out_ids && rows <= d->c.max_rows, "decoder read: bad argument");
    cudaStream_t s = stream_of(d, stream);
    TS_CUDA(cudaMemcpyAsync(d->stage + 4 * (size_t)d->c.max_rows, d->ids, rows * 4, cudaMemcpyDeviceToHost, s));
    TS_CUDA(cudaStreamSynchronize(s));
    memcpy(out_ids, d->stage + 4 * (size_t)d->c.max_rows, rows * 4);
    return TS_OK;
}

int ts_decoder_read_hidden(ts_decoder *d, void *out_bf16, uint32_t rows, void *stream) {
    TS_REQUIRE(d && out_bf16 && rows <= d->c.max_rows, "decoder read: bad argument");
    cudaStream_t s = stream_of(d, stream);
    TS_CUDA(cudaMemcpyAsync(out_bf16, d->h_out, (size_t)rows * d->c.hidden * 2, cudaMemcpyDeviceToHost, s));
    TS_CUDA(cudaStreamSynchronize(s));
    return TS_OK;
}

int ts_decoder_read_logits(ts_decoder *d, float *out, uint32_t n_out, void *stream) {
    TS_REQUIRE(d && out && n_out <= d->max_out, "decoder read: bad argument");
    cudaStream_t s = stream_of(d, stream);
    TS_CUDA(cudaMemcpyAsync(out, d->logits, (size_t)n_out * d->c.vocab * 4, cudaMemcpyDeviceToHost, s));
    TS_CUDA(cudaStreamSynchronize(s));
    return TS_OK;
}

uint32_t ts_decoder_launches_per_step(ts_decoder *d, uint32_t rows, uint32_t keys) {
    if (!d) return 0;
    // Count by walking the same decisions enqueue makes, without launching.
    const ts_decoder_config &c = d->c;
    auto lin = [&](uint32_t m, uint32_t n, uint32_t k, int epi) -> uint32_t {
        return linear_workspace(m, n, k, epi) > 0 ? 2 : 1;
    };
    if (takes_step_kernel(d, rows, keys, d->last_distinct))
        return 1 /*gather and every layer*/ + 1 /*final norm*/ + lin(rows, c.vocab, c.hidden, TS_EPI_NONE) + 2 /*top-1*/;
    const bool fold = fold_parts(d, rows) != 0;
    uint32_t per_layer = (fold ? 0 : 2) /*norms*/ + (append_in_attention(d, d->last_distinct) ? 0 : 1) /*append*/ +
                         1 /*attention*/ +
                         (attend_rows_workspace_bytes(rows, keys, c.heads, c.kv_heads, c.head_dim) > 0 ? 1 : 0) +
                         lin(rows, d->qkv_n, c.hidden, TS_EPI_NONE) + lin(rows, c.hidden, c.heads * c.head_dim, TS_EPI_ADD) +
                         lin(rows, 2 * c.ffn, c.hidden, TS_EPI_SWIGLU) + lin(rows, c.hidden, c.ffn, TS_EPI_ADD);
    return 1 /*gather*/ + c.layers * per_layer + 1 /*final norm*/ + lin(rows, c.vocab, c.hidden, TS_EPI_NONE) + 2 /*top-1*/;
}

uint64_t ts_decoder_graph_replays(ts_decoder *d) { return d ? d->replays : 0; }

uint32_t ts_decoder_graphs(ts_decoder *d) { return d ? (uint32_t)d->graphs.size() : 0; }

int ts_decoder_get_config(const ts_decoder *d, ts_decoder_config *out) {
    TS_REQUIRE(d && out, "decoder config: NULL argument");
    *out = d->c;
    return TS_OK;
}

int ts_decoder_prepare(ts_decoder *d, uint32_t rows, void *stream) {
    TS_REQUIRE(d, "decoder: NULL");
    TS_REQUIRE(rows >= 1 && rows <= d->c.max_rows && rows <= d->max_out, "decoder prepare: %u rows, the plan takes 1..%u",
               rows, d->c.max_rows < d->max_out ? d->c.max_rows : d->max_out);
    cudaStream_t s = stream_of(d, stream);
    {   // the bucket a launch of `rows` rows runs in (see ts_decoder_step)
        uint32_t p = 1;
        while (p < rows) p <<= 1;
        if (p <= d->c.max_rows && p <= d->max_out) rows = p;
    }
    for (uint32_t keys = 128;; keys += 128) {
        const uint32_t k = keys > d->c.context ? d->c.context : keys;
        for (int feedback = 0; feedback < 2; feedback++) {
            int rc = submit(d, rows, k, rows, feedback != 0, true, s, true);
            if (rc != TS_OK) return rc;
        }
        if (k == d->c.context) break;
    }
    return TS_OK;
}

int ts_decoder_profile(ts_decoder *d, uint32_t steps, void *stream) {
    TS_REQUIRE(d, "decoder: NULL");
    TS_REQUIRE(d->last_rows > 0 && d->last_out == d->last_rows,
               "decoder profile: the last launch must have produced one id per row");
    cudaStream_t s = stream_of(d, stream);
    if (!d->gate_flag) TS_CUDA(cudaHostAlloc((void **)&d->gate_flag, 64, cudaHostAllocMapped));
    set_pdl(false);
    for (uint32_t i = 0; i < steps; i++) {
        const uint32_t furthest = d->last_keys + 1;
        TS_REQUIRE(furthest <= d->c.context, "decoder profile: position %u is past the context of %u", furthest - 1,
                   d->c.context);
        d->events_used = 0;
        d->event_names.clear();
        *d->gate_flag = 0;
        int rc = gate(d->gate_flag, s);
        if (rc != TS_OK) return rc;
        d->profiling = true;
        rc = enqueue(d, d->last_rows, keys_bucket(d, furthest), d->last_rows, true, d->last_distinct, s, nullptr);
        d->profiling = false;
        *d->gate_flag = 1;  // every launch of the step is queued: let them run back to back
        if (rc != TS_OK) return rc;
        TS_CUDA(cudaStreamSynchronize(s));
        for (size_t e = 1; e < d->events_used; e++) {
            float ms = 0.0f;
            TS_CUDA(cudaEventElapsedTime(&ms, d->events[e - 1], d->events[e]));
            auto &slot = d->profile[d->event_names[e]];
            slot.first += ms;
            slot.second += 1;
        }
        d->last_keys = furthest;
    }
    return TS_OK;
}

int ts_decoder_take_profile(ts_decoder *d, char *out, size_t capacity) {
    TS_REQUIRE(d && out && capacity > 2, "decoder profile: bad argument");
    std::string text = "{";
    for (auto &kv : d->profile) {
        char line[160];
        snprintf(line, sizeof(line), "%s\"%s\": [%.6f, %llu]", text.size() > 1 ? ", " : "", kv.first.c_str(),
                 kv.second.first, (unsigned long long)kv.second.second);
        text += line;
    }
    text += "}";
    TS_REQUIRE(text.size() + 1 <= capacity, "decoder profile: %zu bytes do not fit in %zu", text.size() + 1, capacity);
    memcpy(out, text.c_str(), text.size() + 1);
    d->profile.clear();
    return TS_OK;
}

}  // extern "C"
#pragma GCC visibility pop
