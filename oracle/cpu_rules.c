/*
 * TEST / BASELINE INFRASTRUCTURE ONLY.  The timed CPU baseline: a C restatement of the
 * reference's native CPU rules, threaded over all host cores and vectorised, for the decode
 * step of the Qwen3-shaped decoder.  Never linked into the shipped library.
 *
 *  - cr_tiled: `cpu_tiled` (engine/rules/cpu/src/dense.rs:32-66, jobs 256-268): one job per
 *    (<= 64-row chunk x 32-column block); the block's 32 weight rows are widened bf16 -> f32
 *    and packed [depth][32] in panels of 128 along k (engine/plan/host/src/simd.rs:366-447,
 *    lockstep.rs:513-541), then a panel micro-kernel accumulates rows x 32 f32 sums.  FMA is
 *    allowed here, as the reference's host path fuses where the ISA does (simd.rs:46-47).
 *  - cr_attend_rows: `cpu_attend_rows` (engine/rules/attention/src/cpu.rs:107-151; host helper
 *    engine/plan/host/src/attend.rs:49-82): per (row, head) scores over the visible keys,
 *    max-subtract softmax, weighted V sum, over an f32 dense store as the reference keeps it
 *    (engine/models/src/decoder.rs:436).
 *  - jobs spread over all cores (engine/plan/run/src/cpu.rs:220-246) with OpenMP.
 *
 * Parity unpinned: this file is a throughput baseline, not a checker; its results are compared
 * with the checker's in tests only to tolerance.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CR_API __attribute__((visibility("default")))
#define CLONES __attribute__((target_clones("avx512f", "avx2,fma", "default")))

static inline float widen(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

CR_API int cr_threads(void) { return omp_get_max_threads(); }

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the baseline is meant to use every host core. */
CR_API void cr_set_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}

/* rows x 32 sums over one k panel; packed is [depth][32]. */
CLONES static void panel(const float *x, size_t x_stride, const float *packed, size_t depth, size_t rows,
                         float *sums /* [rows][32] */) {
    for (size_t r = 0; r < rows; r++) {
        float acc[32];
        for (int c = 0; c < 32; c++) acc[c] = sums[r * 32 + c];
        const float *xr = x + r * x_stride;
        for (size_t d = 0; d < depth; d++) {
            const float xv = xr[d];
            const float *p = packed + d * 32;
            for (int c = 0; c < 32; c++) acc[c] += xv * p[c];
        }
        for (int c = 0; c < 32; c++) sums[r * 32 + c] = acc[c];
    }
}

/* out[m, n] = x[m, k] * w[n, k]^T (+ residual when res != NULL). */
CR_API void cr_tiled(const float *x, const uint16_t *w, const float *res, float *out, size_t m, size_t n,
                     size_t k) {
    const size_t chunk = 64, blocks = (n + 31) / 32, chunks = (m + chunk - 1) / chunk;
#pragma omp parallel
    {
        float *packed = (float *)aligned_alloc(64, sizeof(float) * 128 * 32);
        float *sums = (float *)aligned_alloc(64, sizeof(float) * chunk * 32);
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (size_t ci = 0; ci < chunks; ci++)
            for (size_t b = 0; b < blocks; b++) {
                const size_t row = ci * chunk, col = b * 32;
                const size_t rows = m - row < chunk ? m - row : chunk;
                const size_t cols = n - col < 32 ? n - col : 32;
                memset(sums, 0, sizeof(float) * rows * 32);
                for (size_t k0 = 0; k0 < k; k0 += 128) {
                    const size_t depth = k - k0 < 128 ? k - k0 : 128;
                    for (size_t d = 0; d < depth; d++)
                        for (size_t c = 0; c < 32; c++)
                            packed[d * 32 + c] = c < cols ? widen(w[(col + c) * k + k0 + d]) : 0.0f;
                    panel(x + row * k + k0, k, packed, depth, rows, sums);
                }
                for (size_t r = 0; r < rows; r++)
                    for (size_t c = 0; c < cols; c++) {
                        const size_t at = (row + r) * n + col + c;
                        out[at] = res ? sums[r * 32 + c] + res[at] : sums[r * 32 + c];
                    }
            }
        free(packed);
        free(sums);
    }
}

CLONES static float dotf(const float *a, const float *b, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s += a[i] * b[i];
    return s;
}

CLONES static void axpy(float *o, float p, const float *v, size_t n) {
    for (size_t i = 0; i < n; i++) o[i] += p * v[i];
}

/* q [rows, heads, d]; k, v dense f32 stores [slots, context, kv_heads, d]; causal. */
CR_API void cr_attend_rows(const float *q, const float *k, const float *v, const uint32_t *slots,
                           const uint32_t *positions, float *out, size_t rows, size_t context, size_t heads,
                           size_t kv_heads, size_t d, float scale) {
    const size_t group = heads / kv_heads;
#pragma omp parallel
    {
        float *p = (float *)malloc(sizeof(float) * (context + 1));
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (size_t r = 0; r < rows; r++)
            for (size_t h = 0; h < heads; h++) {
                const size_t n = (size_t)positions[r] + 1;
                const float *kb = k + ((size_t)slots[r] * context * kv_heads + h / group) * d;
                const float *vb = v + ((size_t)slots[r] * context * kv_heads + h / group) * d;
                const float *qr = q + (r * heads + h) * d;
                float max = -INFINITY;
                for (size_t j = 0; j < n; j++) {
                    p[j] = dotf(qr, kb + j * kv_heads * d, d) * scale;
                    max = p[j] > max ? p[j] : max;
                }
                float sum = 0.0f;
                for (size_t j = 0; j < n; j++) {
                    p[j] = expf(p[j] - max);
                    sum += p[j];
                }
                float *o = out + (r * heads + h) * d;
                memset(o, 0, sizeof(float) * d);
                for (size_t j = 0; j < n; j++) axpy(o, p[j] / sum, vb + j * kv_heads * d, d);
            }
        free(p);
    }
}

static void rms_rows(float *x, const float *w, size_t rows, size_t width, float eps) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        float *row = x + r * width;
        float inv = 1.0f / sqrtf(dotf(row, row, width) / (float)width + eps);
        for (size_t i = 0; i < width; i++) row[i] *= inv * w[i];
    }
}

typedef struct {
    uint32_t layers, hidden, heads, kv_heads, head_dim, ffn, vocab, context, slots;
    float eps, theta;
} cr_config;

typedef struct {
    const uint16_t *embed;
    const uint16_t *const *q, *const *k, *const *v, *const *o, *const *gate, *const *up, *const *down;
    const float *const *ln1, *const *ln2, *const *q_norm, *const *k_norm;
    const float *norm;
} cr_weights;

/* One decode step over `rows` rows, f32 activations, as the reference's host plan runs it
 * (engine/models/src/decoder.rs:327-389).  keys/values: per-layer dense f32 stores. */
CR_API void cr_decoder_step(const cr_config *c, const cr_weights *w, float *const *keys, float *const *values,
                            const uint32_t *tokens, const uint32_t *slots, const uint32_t *positions, size_t rows,
                            uint32_t *ids) {
    const size_t H = c->hidden, D = c->head_dim, NH = c->heads, NKV = c->kv_heads, F = c->ffn;
    const size_t QW = NH * D, KW = NKV * D;
    float *x = (float *)malloc(sizeof(float) * rows * H), *h = (float *)malloc(sizeof(float) * rows * H);
    float *q = (float *)malloc(sizeof(float) * rows * QW), *k = (float *)malloc(sizeof(float) * rows * KW);
    float *v = (float *)malloc(sizeof(float) * rows * KW), *a = (float *)malloc(sizeof(float) * rows * QW);
    float *g = (float *)malloc(sizeof(float) * rows * F), *u = (float *)malloc(sizeof(float) * rows * F);
    float *lg = (float *)malloc(sizeof(float) * rows * c->vocab);
    const float scale = 1.0f / sqrtf((float)D);
    for (size_t r = 0; r < rows; r++)
        for (size_t i = 0; i < H; i++) x[r * H + i] = widen(w->embed[(size_t)tokens[r] * H + i]);
    for (uint32_t l = 0; l < c->layers; l++) {
        memcpy(h, x, sizeof(float) * rows * H);
        rms_rows(h, w->ln1[l], rows, H, c->eps);
        cr_tiled(h, w->q[l], NULL, q, rows, QW, H);
        cr_tiled(h, w->k[l], NULL, k, rows, KW, H);
        cr_tiled(h, w->v[l], NULL, v, rows, KW, H);
        rms_rows(q, w->q_norm[l], rows * NH, D, c->eps);
        rms_rows(k, w->k_norm[l], rows * NKV, D, c->eps);
#pragma omp parallel for schedule(static)
        for (size_t r = 0; r < rows; r++) {
            for (size_t hh = 0; hh < NH + NKV; hh++) {
                float *row = hh < NH ? q + (r * NH + hh) * D : k + (r * NKV + hh - NH) * D;
                for (size_t j = 0; j < D / 2; j++) {
                    float ang = (float)positions[r] * powf(c->theta, -((float)(2 * j)) / (float)D);
                    float s = sinf(ang), co = cosf(ang);
                    float ra = row[j] * co - row[j + D / 2] * s, rb = row[j] * s + row[j + D / 2] * co;
                    row[j] = ra;
                    row[j + D / 2] = rb;
                }
            }
            size_t at = ((size_t)slots[r] * c->context + positions[r]) * KW;
            memcpy(keys[l] + at, k + r * KW, sizeof(float) * KW);
            memcpy(values[l] + at, v + r * KW, sizeof(float) * KW);
        }
        cr_attend_rows(q, keys[l], values[l], slots, positions, a, rows, c->context, NH, NKV, D, scale);
        cr_tiled(a, w->o[l], x, x, rows, H, QW);
        memcpy(h, x, sizeof(float) * rows * H);
        rms_rows(h, w->ln2[l], rows, H, c->eps);
        cr_tiled(h, w->gate[l], NULL, g, rows, F, H);
        cr_tiled(h, w->up[l], NULL, u, rows, F, H);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < rows * F; i++) g[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
        cr_tiled(g, w->down[l], x, x, rows, H, F);
    }
    memcpy(h, x, sizeof(float) * rows * H);
    rms_rows(h, w->norm, rows, H, c->eps);
    cr_tiled(h, w->embed, NULL, lg, rows, c->vocab, H);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        uint32_t best = 0;
        for (uint32_t i = 1; i < c->vocab; i++)
            if (lg[r * c->vocab + i] > lg[r * c->vocab + best]) best = i;
        ids[r] = best;
    }
    free(x); free(h); free(q); free(k); free(v); free(a); free(g); free(u); free(lg);
}
