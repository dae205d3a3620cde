/*
 * TEST INFRASTRUCTURE ONLY.  A single-threaded CPU restatement of tessera-interp,
 * the reference interpreter every tessera plan is checked against.  Nothing in the
 * shipped library links, loads or calls this file; only the tests, the smoke check
 * and the CPU-baseline leg of the benchmark do, and only as the checker.
 *
 * Parity pin: every literal known-answer test the reference holds for this path is
 * replayed against this file by tests/test_oracle_golden.py (top_k_ties,
 * rms_divides_rows, softmax_rows, act_values, gather_rows, mean_each_axis,
 * rope_both_pairs, hadamard_blocks, causal_first_row, decode_sees_past_keys,
 * accumulators_follow_numerics, sums_round, window_edges, rows_read_slots,
 * store_keeps_rows).  The reference itself (Rust) cannot be built in this
 * environment, so outputs of the reference binary are not part of the pin.
 *
 * Every function follows the reference file:line cited above it.  All sums run in
 * the reference's fixed order (k ascending, one f32 add per term, no FMA): build
 * with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TO_API __attribute__((visibility("default")))

/* ---- narrow floats: engine/ir/graph/src/scalar.rs:21-58 ------------------ */

/* f32 -> bf16 bits, round to nearest even on the dropped 16 bits, NaN -> quiet. */
TO_API uint16_t to_bf16_narrow(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    if (x != x) return (uint16_t)(((bits >> 31) << 15) | 0x7FC0u);
    uint32_t half = 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + half) >> 16);
}

TO_API float to_bf16_widen(uint16_t b) {
    uint32_t bits = (uint32_t)b << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* f32 -> f16 -> f32 (RNE, subnormals kept, overflow -> inf): scalar.rs:21-58 with E=5,M=10. */
static float round_f16(float x) {
    if (x != x || isinf(x)) return x;
    float a = fabsf(x);
    float sign = signbit(x) ? -1.0f : 1.0f;
    if (a < 6.103515625e-05f) { /* 2^-14: subnormal steps of 2^-24 */
        double steps = nearbyint((double)a * 16777216.0);
        return sign * (float)(steps / 16777216.0);
    }
    uint32_t bits;
    memcpy(&bits, &a, 4);
    uint32_t half = 0xFFFu + ((bits >> 13) & 1u);
    bits = (bits + half) & ~0x1FFFu;
    float r;
    memcpy(&r, &bits, 4);
    if (r > 65504.0f) return sign * INFINITY;
    return sign * r;
}

static float round_bf16(float x) { return to_bf16_widen(to_bf16_narrow(x)); }

TO_API void to_bf16_round_array(const float *x, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = round_bf16(x[i]);
}

TO_API void to_bf16_narrow_array(const float *x, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = to_bf16_narrow(x[i]);
}

TO_API void to_bf16_widen_array(const uint16_t *x, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = to_bf16_widen(x[i]);
}

/* ---- accumulators: engine/ir/interp/src/round.rs:6-34 -------------------- */

enum { ACC_F32 = 0, ACC_F16 = 1, ACC_BF16 = 2 };

static inline float acc_add(int acc, float sum, float v) {
    float s = sum + v;
    if (acc == ACC_F16) return round_f16(s);
    if (acc == ACC_BF16) return round_bf16(s);
    return s;
}

TO_API float to_acc_sum(int acc, const float *v, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s = acc_add(acc, s, v[i]);
    return s;
}

static float acc_dot(int acc, const float *a, const float *b, size_t n) {
    float s = 0.0f;
    if (acc == ACC_F32) {
        for (size_t i = 0; i < n; i++) s = s + a[i] * b[i];
        return s;
    }
    for (size_t i = 0; i < n; i++) s = acc_add(acc, s, a[i] * b[i]);
    return s;
}

/* ---- seeded noise: engine/ir/testkit/src/noise.rs:1-10 ------------------- */

TO_API void to_noise(uint64_t *state, float *out, size_t n) {
    uint64_t s = *state;
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        out[i] = (float)(s >> 40) / 8388608.0f - 1.0f;
    }
    *state = s;
}

/* ---- matmul: engine/ir/interp/src/cpu.rs:82-138 --------------------------- */

/* out[r][c] = dot(x[r,:], w[c,:]); eight columns run side by side, each one still a
 * strictly sequential f32 sum over k, so the bits equal the one-column loop. */
static void matmul_f32(int acc, const float *x, const float *w, float *out, size_t m, size_t n,
                       size_t k) {
    for (size_t r = 0; r < m; r++) {
        const float *xr = x + r * k;
        size_t c = 0;
        if (acc == ACC_F32) {
            for (; c + 8 <= n; c += 8) {
                float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                const float *w0 = w + c * k;
                for (size_t i = 0; i < k; i++) {
                    float xv = xr[i];
                    for (int j = 0; j < 8; j++) s[j] = s[j] + xv * w0[(size_t)j * k + i];
                }
                for (int j = 0; j < 8; j++) out[r * n + c + j] = s[j];
            }
        }
        for (; c < n; c++) out[r * n + c] = acc_dot(acc, xr, w + c * k, k);
    }
}

TO_API void to_matmul(int acc, const float *x, const float *w, float *out, size_t m, size_t n,
                      size_t k) {
    matmul_f32(acc, x, w, out, m, n, k);
}

/* Same product with the weight held as bf16 bits and widened before use
 * (engine/ir/interp/src/run.rs:231-237). */
TO_API void to_matmul_bf16w(const float *x, const uint16_t *w, float *out, size_t m, size_t n,
                            size_t k) {
    enum { COLS = 8 };
    float *wide = (float *)malloc(sizeof(float) * COLS * k);
    for (size_t c = 0; c < n; c += COLS) {
        size_t cols = n - c < COLS ? n - c : COLS;
        for (size_t j = 0; j < cols * k; j++) wide[j] = to_bf16_widen(w[c * k + j]);
        for (size_t r = 0; r < m; r++) {
            const float *xr = x + r * k;
            float s[COLS] = {0};
            for (size_t i = 0; i < k; i++) {
                float xv = xr[i];
                for (size_t j = 0; j < cols; j++) s[j] = s[j] + xv * wide[j * k + i];
            }
            for (size_t j = 0; j < cols; j++) out[r * n + c + j] = s[j];
        }
    }
    free(wide);
}

/* ---- Q8_0 block form: engine/ir/mem/src/block.rs:259-260 (an f16 scale, then 32 signed bytes), packed,
 * unpacked and dotted as block.rs:204-258 does it. ------------------------------------------------------ */

static uint16_t to_f16_bits(float x) { /* round to nearest even, as half::f16::from_f32 */
    uint32_t u;
    memcpy(&u, &x, 4);
    uint32_t sign = (u >> 16) & 0x8000u, mant = u & 0x7FFFFFu;
    int32_t exp = (int32_t)((u >> 23) & 0xFF);
    if (exp == 255) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u : 0));
    int32_t e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        mant |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half = mant >> shift, rest = mant & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rest > mid || (rest == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (mant >> 13), rest = mant & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}

static float to_f16_widen(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, mant = h & 0x3FFu, u;
    if (exp == 0) {
        if (mant == 0) u = sign;
        else {
            int e = -1;
            do { mant <<= 1; e++; } while (!(mant & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mant & 0x3FFu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7F800000u | (mant << 13);
    else u = sign | ((exp - 15 + 127) << 23) | (mant << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

TO_API size_t to_q8_0_bytes(size_t elements) { return (elements + 31) / 32 * 34; }

/* Block::pack with S = F16, C = I8, B = 32, no head: scale = max |x| / 127 stored as f16; codes see the scale
 * as stored; round_ties_even, clamped to [-128, 127]. */
TO_API void to_q8_0_pack(const float *data, size_t elements, uint8_t *out) {
    memset(out, 0, to_q8_0_bytes(elements));
    for (size_t b = 0; b * 32 < elements; b++) {
        size_t n = elements - b * 32 < 32 ? elements - b * 32 : 32;
        float top = 0.0f;
        for (size_t j = 0; j < n; j++) top = fmaxf(top, fabsf(data[b * 32 + j]));
        uint16_t bits = to_f16_bits(top / 127.0f);
        uint8_t *at = out + b * 34;
        at[0] = (uint8_t)(bits & 0xFF);
        at[1] = (uint8_t)(bits >> 8);
        float stored = to_f16_widen(bits);
        for (size_t j = 0; j < n; j++) {
            float scaled = stored == 0.0f ? 0.0f : data[b * 32 + j] / stored;
            float r = rintf(scaled); /* the default rounding mode: ties to even */
            if (r < -128.0f) r = -128.0f;
            if (r > 127.0f) r = 127.0f;
            at[2 + j] = (uint8_t)(int8_t)r;
        }
    }
}

TO_API void to_q8_0_unpack(const uint8_t *bytes, size_t elements, float *out) {
    for (size_t i = 0; i < elements; i++) {
        const uint8_t *at = bytes + i / 32 * 34;
        float scale = to_f16_widen((uint16_t)(at[0] | (at[1] << 8)));
        out[i] = scale * (float)(int8_t)at[2 + i % 32];
    }
}

/* x [m, k] against a Q8_0 matrix [n, k] (k a multiple of 32): every output is Form::dot over its row -
 * per block the plain sum of x times code, times the block's scale, blocks added in order. */
TO_API void to_matmul_q8_0(const float *x, const uint8_t *w, float *out, size_t m, size_t n, size_t k) {
    size_t row_bytes = k / 32 * 34;
    for (size_t r = 0; r < m; r++)
        for (size_t c = 0; c < n; c++) {
            const uint8_t *row = w + c * row_bytes;
            float sum = 0.0f;
            for (size_t b = 0; b < k / 32; b++) {
                const uint8_t *at = row + b * 34;
                float part = 0.0f;
                for (size_t j = 0; j < 32; j++) part = part + x[r * k + b * 32 + j] * (float)(int8_t)at[2 + j];
                sum = sum + to_f16_widen((uint16_t)(at[0] | (at[1] << 8))) * part;
            }
            out[r * n + c] = sum;
        }
}

/* matmul_picked: engine/ir/interp/src/cpu.rs:89-105.  Row r of x meets matrix
 * ids[r] - first of `table` ([experts, n, k]); an id outside the table reads zeros.
 * x has `m` rows; ids has `rows` entries, rows a multiple of m; row r reads x row
 * r / (rows / m)  (cpu.rs:121-125). */
TO_API void to_matmul_picked(const float *x, const float *table, const uint32_t *ids, float *out,
                             size_t m, size_t rows, size_t experts, size_t n, size_t k,
                             size_t first) {
    size_t per = rows / (m ? m : 1);
    for (size_t r = 0; r < rows; r++) {
        const float *xr = x + (r / (per ? per : 1)) * k;
        size_t id = ids[r];
        int inside = id >= first && id - first < experts;
        for (size_t c = 0; c < n; c++) {
            if (!inside) {
                /* dot with a zero row: every term is 0 * x, the sum keeps x's NaNs */
                float s = 0.0f;
                for (size_t i = 0; i < k; i++) s = s + xr[i] * 0.0f;
                out[r * n + c] = s;
            } else {
                out[r * n + c] = acc_dot(ACC_F32, xr, table + ((id - first) * n + c) * k, k);
            }
        }
    }
}

/* ---- row stages: engine/ir/interp/src/cpu.rs:9-59, 353-447, 475-495 ------ */

enum { ACT_GELU_TANH = 0, ACT_SILU, ACT_SIGMOID, ACT_RELU, ACT_SOFTPLUS, ACT_EXP, ACT_TANH };

static float act1(int a, float x) {
    switch (a) {
    case ACT_GELU_TANH: {
        const float coef = 0.7978846f;
        return 0.5f * x * (1.0f + tanhf(coef * (x + 0.044715f * x * x * x)));
    }
    case ACT_SILU: return x / (1.0f + expf(-x));
    case ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case ACT_RELU: return x > 0.0f ? x : 0.0f;
    case ACT_SOFTPLUS: return (x > 0.0f ? x : 0.0f) + log1pf(expf(-fabsf(x)));
    case ACT_EXP: return expf(x);
    default: return tanhf(x);
    }
}

TO_API void to_act(int a, float *x, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] = act1(a, x[i]);
}

static void softmax_row(int acc, float *row, size_t n) {
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++) max = row[i] > max ? row[i] : max; /* f32::max skips NaN */
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        row[i] = expf(row[i] - max);
        sum = acc_add(acc, sum, row[i]);
    }
    for (size_t i = 0; i < n; i++) row[i] /= sum;
}

TO_API void to_softmax(int acc, float *x, size_t rows, size_t width) {
    for (size_t r = 0; r < rows; r++) softmax_row(acc, x + r * width, width);
}

static float rms_inverse(int acc, const float *row, size_t n, float eps) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s = acc_add(acc, s, row[i] * row[i]);
    float mean = s / (float)n;
    return 1.0f / sqrtf(mean + eps);
}

/* Stage::RmsNorm when w != NULL, Stage::Rms otherwise. */
TO_API void to_rms_norm(int acc, float *x, const float *w, size_t rows, size_t width, float eps) {
    for (size_t r = 0; r < rows; r++) {
        float *row = x + r * width;
        float inv = rms_inverse(acc, row, width, eps);
        for (size_t i = 0; i < width; i++) row[i] = w ? row[i] * (inv * w[i]) : row[i] * inv;
    }
}

enum { PAIRS_ADJACENT = 0, PAIRS_HALVES = 1 };

/* angle + turn: cpu.rs:31-47.  x is [positions, span/width, width]. */
TO_API void to_rope(float *x, const uint32_t *positions, size_t count, size_t span, size_t width,
                    float theta, int pairs, size_t turned) {
    size_t half = width / 2;
    size_t upto = half < turned ? half : turned;
    for (size_t p = 0; p < count; p++) {
        for (size_t at = 0; at + width <= span; at += width) {
            float *row = x + p * span + at;
            for (size_t j = 0; j < upto; j++) {
                size_t a = pairs == PAIRS_ADJACENT ? 2 * j : j;
                size_t b = pairs == PAIRS_ADJACENT ? 2 * j + 1 : j + half;
                float ang = (float)positions[p] * powf(theta, -((float)(2 * j)) / (float)width);
                float s = sinf(ang), c = cosf(ang);
                float ra = row[a] * c - row[b] * s;
                float rb = row[a] * s + row[b] * c;
                row[a] = ra;
                row[b] = rb;
            }
        }
    }
}

/* Walsh-Hadamard over blocks, scaled to keep the norm: cpu.rs:475-489. */
TO_API void to_hadamard(float *x, size_t n, size_t block) {
    for (size_t at = 0; at + block <= n; at += block) {
        float *v = x + at;
        for (size_t len = 1; len < block; len *= 2)
            for (size_t p = 0; p < block; p += 2 * len)
                for (size_t i = 0; i < len; i++) {
                    float a = v[p + i], b = v[p + len + i];
                    v[p + i] = a + b;
                    v[p + len + i] = a - b;
                }
        float scale = 1.0f / sqrtf((float)block);
        for (size_t i = 0; i < block; i++) v[i] *= scale;
    }
}

/* mean over an axis, or a weighted sum with `weights` [outer, count]: cpu.rs:449-473. */
TO_API void to_mean(int acc, const float *x, const float *weights, float *out, size_t outer,
                    size_t count, size_t inner) {
    for (size_t o = 0; o < outer; o++)
        for (size_t i = 0; i < inner; i++) {
            float s = 0.0f;
            for (size_t t = 0; t < count; t++) {
                float w = weights ? weights[o * count + t] : 1.0f / (float)count;
                s = acc_add(acc, s, x[(o * count + t) * inner + i] * w);
            }
            out[o * inner + i] = s;
        }
}

/* take: cpu.rs:497-508.  Out-of-range ids read zero. */
TO_API void to_take(const float *x, const uint32_t *ids, float *out, size_t rows, size_t width,
                    size_t picks) {
    for (size_t r = 0; r < rows; r++)
        for (size_t p = 0; p < picks; p++) {
            uint32_t i = ids[r * picks + p];
            out[r * picks + p] = i < width ? x[r * width + i] : 0.0f;
        }
}

/* gather: cpu.rs:510-525.  Rows outside [first, first + rows) read zero. */
TO_API void to_gather(const void *table, const uint32_t *ids, void *out, size_t rows,
                      size_t row_bytes, size_t count, size_t first) {
    for (size_t i = 0; i < count; i++) {
        size_t id = ids[i];
        char *dst = (char *)out + i * row_bytes;
        if (id >= first && id - first < rows)
            memcpy(dst, (const char *)table + (id - first) * row_bytes, row_bytes);
        else
            memset(dst, 0, row_bytes);
    }
}

/* top_k: engine/ir/interp/src/run.rs:577-591.  Finite-or-+inf entries only (x > -inf
 * is false for NaN), best first, a stable sort so ties keep the lower index (0.0 ties
 * -0.0), spare slots hold the width. */
TO_API void to_top_k(const float *x, uint32_t *out, size_t rows, size_t width, size_t k) {
    uint32_t *order = (uint32_t *)malloc(sizeof(uint32_t) * (width + 1));
    for (size_t r = 0; r < rows; r++) {
        const float *row = x + r * width;
        size_t n = 0;
        for (size_t i = 0; i < width; i++)
            if (row[i] > -INFINITY) order[n++] = (uint32_t)i;
        /* stable insertion sort, descending */
        for (size_t i = 1; i < n; i++) {
            uint32_t v = order[i];
            size_t j = i;
            while (j > 0 && row[order[j - 1]] < row[v]) {
                order[j] = order[j - 1];
                j--;
            }
            order[j] = v;
        }
        for (size_t j = 0; j < k; j++) out[r * k + j] = j < n ? order[j] : (uint32_t)width;
    }
    free(order);
}

/* ---- masks: engine/ir/graph/src/node.rs:162-187, cpu.rs:61-77 ------------ */

enum { MASK_CAUSAL = 0, MASK_BIDIRECTIONAL = 1, MASK_WITHIN = 2, MASK_BACK = 3 };

static void mask_window(int mask, size_t n, size_t far, size_t *back, size_t *ahead) {
    switch (mask) {
    case MASK_CAUSAL: *back = far; *ahead = 0; break;
    case MASK_BIDIRECTIONAL: *back = far; *ahead = far; break;
    case MASK_WITHIN: *back = n; *ahead = n; break;
    default: *back = n; *ahead = 0; break;
    }
}

static void seen(int mask, size_t n, size_t position, size_t keys, size_t *from, size_t *to) {
    size_t back, ahead;
    mask_window(mask, n, keys, &back, &ahead);
    *from = position > back ? position - back : 0;
    size_t end = position + ahead + 1;
    *to = end < keys ? end : keys;
}

/* Keys::row: cpu.rs:148-168.  Scores scaled after the dot, one whole-row softmax,
 * then o += p * v in key order. */
static void attend_row(int acc, float scale, const float *q, const float *k, const float *v,
                       size_t d, size_t dv, size_t kv_stride, size_t from, size_t to, float *p,
                       float *o) {
    size_t n = to > from ? to - from : 0;
    for (size_t j = 0; j < n; j++) p[j] = acc_dot(acc, q, k + (from + j) * kv_stride * d, d) * scale;
    if (n) softmax_row(acc, p, n);
    for (size_t j = 0; j < n; j++) {
        const float *vj = v + (from + j) * kv_stride * dv;
        for (size_t i = 0; i < dv; i++) o[i] = acc_add(acc, o[i], p[j] * vj[i]);
    }
}

/* attend: cpu.rs:171-225.  q [seqs, queries, heads, d]; k [seqs, keys, kv_heads, d];
 * v [seqs, keys, kv_heads, dv]; out [seqs, queries, heads, dv].  Returns 1 when a
 * causal mask meets fewer keys than queries (cpu.rs:62-68). */
TO_API int to_attend(int acc, int mask, size_t mask_n, float scale, const float *q, const float *k,
                     const float *v, float *out, size_t seqs, size_t queries, size_t keys,
                     size_t heads, size_t kv_heads, size_t d, size_t dv) {
    size_t past;
    if (keys >= queries) past = keys - queries;
    else if (mask == MASK_BIDIRECTIONAL || mask == MASK_WITHIN) past = 0;
    else return 1;
    size_t group = heads / kv_heads;
    float *p = (float *)malloc(sizeof(float) * (keys + 1));
    memset(out, 0, sizeof(float) * seqs * queries * heads * dv);
    for (size_t s = 0; s < seqs; s++)
        for (size_t t = 0; t < queries; t++) {
            size_t from, to;
            seen(mask, mask_n, past + t, keys, &from, &to);
            for (size_t h = 0; h < heads; h++) {
                size_t row = (s * queries + t) * heads + h;
                const float *kb = k + (s * keys * kv_heads + h / group) * d;
                const float *vb = v + (s * keys * kv_heads + h / group) * dv;
                attend_row(acc, scale, q + row * d, kb, vb, d, dv, kv_heads, from, to, p,
                           out + row * dv);
            }
        }
    free(p);
    return 0;
}

/* attend_rows: cpu.rs:292-351.  q [rows, heads, d]; k/v a dense store
 * [seqs, keys, kv_heads, d|dv]; row r reads slot slots[r] up to positions[r].
 * Returns r + 1 for the first row whose position is past `keys`. */
TO_API int to_attend_rows(int acc, int mask, size_t mask_n, float scale, const float *q,
                          const float *k, const float *v, const uint32_t *slots,
                          const uint32_t *positions, float *out, size_t rows, size_t keys,
                          size_t heads, size_t kv_heads, size_t d, size_t dv) {
    size_t group = heads / kv_heads;
    float *p = (float *)malloc(sizeof(float) * (keys + 1));
    memset(out, 0, sizeof(float) * rows * heads * dv);
    for (size_t r = 0; r < rows; r++) {
        size_t s = slots[r], at = positions[r];
        if (at >= keys) {
            free(p);
            return (int)r + 1;
        }
        size_t from, to;
        seen(mask, mask_n, at, keys, &from, &to);
        for (size_t h = 0; h < heads; h++) {
            size_t row = r * heads + h;
            const float *kb = k + (s * keys * kv_heads + h / group) * d;
            const float *vb = v + (s * keys * kv_heads + h / group) * dv;
            attend_row(acc, scale, q + row * d, kb, vb, d, dv, kv_heads, from, to, p,
                       out + row * dv);
        }
    }
    free(p);
    return 0;
}

/* ---- kept-row layouts: engine/plan/codegen/src/kept.rs:135-194 ----------- */

enum { KEPT_DENSE = 0, KEPT_INTERLEAVED = 1, KEPT_PAGED = 2 };

/* `scalar` is kept_stride, kept_slots or kept_pages; `page` only matters when paged. */
TO_API uint32_t to_kept_row(int layout, uint32_t slot, uint32_t position, uint32_t scalar,
                            uint32_t page, const uint32_t *table) {
    if (layout == KEPT_DENSE) return slot * scalar + position;
    if (layout == KEPT_INTERLEAVED) return position * scalar + slot;
    uint32_t shift = (uint32_t)__builtin_ctz(page);
    uint64_t entry = (uint64_t)slot * scalar + (position >> shift);
    return (table[entry] << shift) | (position & (page - 1));
}

/* ---- the decoder, op by op: engine/models/src/decoder.rs:281-389 --------- */
/*
 * One Qwen3-shaped step over `rows` rows (slot, position, token each), f32 math on
 * values that are bf16 wherever the device path stores bf16: the normed rows, the
 * q/k/v rows after head norm and rotation, the attention output, and the gated
 * inner rows.  The residual stream stays f32.  The dense store is
 * [slots, context, kv_heads, head_dim] per layer for keys and values.
 */
typedef struct {
    uint32_t layers, hidden, heads, kv_heads, head_dim, ffn, vocab, context, slots;
    float eps, theta;
} to_decoder_config;

typedef struct {
    const uint16_t *embed;                /* [vocab, hidden], tied unembed */
    const uint16_t *const *q, *const *k, *const *v, *const *o; /* per layer [out, in] */
    const uint16_t *const *gate, *const *up, *const *down;
    const float *const *ln1, *const *ln2, *const *q_norm, *const *k_norm;
    const float *norm;
} to_decoder_weights;

static void round_rows(float *x, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] = round_bf16(x[i]);
}

/* Runs the trunk and returns the final normed rows in `hidden_out` [rows, hidden]
 * (bf16-valued), logits in `logits` [rows, vocab] when not NULL, greedy ids in `ids`
 * (first maximum, strict >: engine/rules/kernels/src/argmax.rs:72-114) when not NULL.
 * keys/values: per layer dense stores, updated in place.  Returns 0, or 1 when a row
 * sits outside the store. */
TO_API int to_decoder_step(const to_decoder_config *c, const to_decoder_weights *w,
                           float *const *keys, float *const *values, const uint32_t *tokens,
                           const uint32_t *slots, const uint32_t *positions, size_t rows,
                           float *hidden_out, float *logits, uint32_t *ids) {
    size_t H = c->hidden, D = c->head_dim, NH = c->heads, NKV = c->kv_heads, F = c->ffn;
    size_t QW = NH * D, KW = NKV * D;
    float *x = (float *)malloc(sizeof(float) * rows * H);
    float *h = (float *)malloc(sizeof(float) * rows * H);
    float *q = (float *)malloc(sizeof(float) * rows * QW);
    float *k = (float *)malloc(sizeof(float) * rows * KW);
    float *v = (float *)malloc(sizeof(float) * rows * KW);
    float *a = (float *)malloc(sizeof(float) * rows * QW);
    float *t = (float *)malloc(sizeof(float) * rows * (H > F ? H : F));
    float *g = (float *)malloc(sizeof(float) * rows * F);
    float *u = (float *)malloc(sizeof(float) * rows * F);
    int bad = 0;
    float scale = 1.0f / sqrtf((float)D);
    for (size_t r = 0; r < rows; r++)
        if (slots[r] >= c->slots || positions[r] >= c->context || tokens[r] >= c->vocab) bad = 1;
    if (bad) goto done;
    for (size_t r = 0; r < rows; r++)
        for (size_t i = 0; i < H; i++) x[r * H + i] = to_bf16_widen(w->embed[(size_t)tokens[r] * H + i]);
    for (uint32_t l = 0; l < c->layers; l++) {
        memcpy(h, x, sizeof(float) * rows * H);
        to_rms_norm(ACC_F32, h, w->ln1[l], rows, H, c->eps);
        round_rows(h, rows * H);
        to_matmul_bf16w(h, w->q[l], q, rows, QW, H);
        to_matmul_bf16w(h, w->k[l], k, rows, KW, H);
        to_matmul_bf16w(h, w->v[l], v, rows, KW, H);
        /* the projections leave the device as bf16 rows */
        round_rows(q, rows * QW);
        round_rows(k, rows * KW);
        round_rows(v, rows * KW);
        to_rms_norm(ACC_F32, q, w->q_norm[l], rows * NH, D, c->eps);
        to_rms_norm(ACC_F32, k, w->k_norm[l], rows * NKV, D, c->eps);
        to_rope(q, positions, rows, QW, D, c->theta, PAIRS_HALVES, D);
        to_rope(k, positions, rows, KW, D, c->theta, PAIRS_HALVES, D);
        round_rows(q, rows * QW);
        round_rows(k, rows * KW);
        /* append before attention reads: engine/ir/interp/src/run.rs:120-176 */
        for (size_t r = 0; r < rows; r++) {
            size_t at = ((size_t)slots[r] * c->context + positions[r]) * KW;
            memcpy(keys[l] + at, k + r * KW, sizeof(float) * KW);
            memcpy(values[l] + at, v + r * KW, sizeof(float) * KW);
        }
        /* row r reads keys [0, position]; the store's row stride is the full context */
        {
            size_t group = NH / NKV;
            float *p = (float *)malloc(sizeof(float) * (c->context + 1));
            memset(a, 0, sizeof(float) * rows * QW);
            for (size_t r = 0; r < rows; r++)
                for (size_t hh = 0; hh < NH; hh++) {
                    size_t base = ((size_t)slots[r] * c->context * NKV + hh / group) * D;
                    attend_row(ACC_F32, scale, q + (r * NH + hh) * D, keys[l] + base,
                               values[l] + base, D, D, NKV, 0, (size_t)positions[r] + 1, p,
                               a + (r * NH + hh) * D);
                }
            free(p);
        }
        round_rows(a, rows * QW);
        to_matmul_bf16w(a, w->o[l], t, rows, H, QW);
        for (size_t i = 0; i < rows * H; i++) x[i] = t[i] + x[i];
        memcpy(h, x, sizeof(float) * rows * H);
        to_rms_norm(ACC_F32, h, w->ln2[l], rows, H, c->eps);
        round_rows(h, rows * H);
        to_matmul_bf16w(h, w->gate[l], g, rows, F, H);
        to_matmul_bf16w(h, w->up[l], u, rows, F, H);
        for (size_t i = 0; i < rows * F; i++) g[i] = act1(ACT_SILU, g[i]) * u[i];
        round_rows(g, rows * F);
        to_matmul_bf16w(g, w->down[l], t, rows, H, F);
        for (size_t i = 0; i < rows * H; i++) x[i] = t[i] + x[i];
    }
    memcpy(h, x, sizeof(float) * rows * H);
    to_rms_norm(ACC_F32, h, w->norm, rows, H, c->eps);
    round_rows(h, rows * H);
    if (hidden_out) memcpy(hidden_out, h, sizeof(float) * rows * H);
    if (logits || ids) {
        float *lg = logits ? logits : (float *)malloc(sizeof(float) * rows * c->vocab);
        to_matmul_bf16w(h, w->embed, lg, rows, c->vocab, H);
        if (ids)
            for (size_t r = 0; r < rows; r++) {
                uint32_t best = 0;
                for (uint32_t i = 1; i < c->vocab; i++)
                    if (lg[r * c->vocab + i] > lg[r * c->vocab + best]) best = i;
                ids[r] = best;
            }
        if (!logits) free(lg);
    }
done:
    free(x); free(h); free(q); free(k); free(v); free(a); free(t); free(g); free(u);
    return bad;
}
