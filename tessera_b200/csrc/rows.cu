// Row kernels around the two hot rules: RMS norm, embedding gather, the fused per-head
// norm + rotation + kept-row append, plain scatter, top-k / argmax, and the router's
// take + softmax.  Each follows the reference kernel it replaces (cited per kernel).
#include <cmath>

#include "head_prep.cuh"
#include "ts_common.cuh"

namespace ts {
namespace {

__device__ __forceinline__ float block_sum(float v, float *scratch) {
    v = warp_sum(v);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const uint32_t warps = (blockDim.x + 31) / 32;
    float t = 0.0f;
    for (uint32_t w = 0; w < warps; w++) t += scratch[w];  // fixed order
    __syncthreads();
    return t;
}

// ---- rms_norm: engine/rules/kernels/src/lane_norm.rs:10-17; math engine/ir/interp/src/cpu.rs:371-377, 491-495
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) rms_norm_kernel(const TIn *x, const float *w, TOut *out, uint32_t width,
                                                       float eps, const uint32_t *row_ids) {
    __shared__ float scratch[8];
    pdl_wait();
    // With row_ids, output row i reads input row row_ids[i] (the rows whose logits are wanted).
    const size_t base = (size_t)(row_ids ? row_ids[blockIdx.x] : blockIdx.x) * width;
    const size_t obase = (size_t)blockIdx.x * width;
    float ss = 0.0f;
    if (width <= 16 * blockDim.x) {
        // The row fits in registers (16 per thread): one read, all loads in flight at once; the sum of squares
        // runs in the same order as the loop below, so both forms give the same bits.
        float held[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            held[j] = 0.0f;
            if (i < width) {
                if constexpr (sizeof(TIn) == 4) held[j] = x[base + i];
                else held[j] = __uint_as_float((uint32_t)x[base + i] << 16);
            }
        }
#pragma unroll
        for (int j = 0; j < 16; j++)
            if (threadIdx.x + j * blockDim.x < width) ss = fmaf(held[j], held[j], ss);
        ss = block_sum(ss, scratch);
        pdl_launch_dependents();
        const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            if (i < width) {
                const float r = w ? held[j] * (inv * w[i]) : held[j] * inv;
                if constexpr (sizeof(TOut) == 4) out[obase + i] = r;
                else out[obase + i] = bf16_bits(r);
            }
        }
        return;
    }
    for (uint32_t i = threadIdx.x; i < width; i += blockDim.x) {
        float v;
        if constexpr (sizeof(TIn) == 4) v = x[base + i];
        else v = __uint_as_float((uint32_t)x[base + i] << 16);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    pdl_launch_dependents();
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (uint32_t i = threadIdx.x; i < width; i += blockDim.x) {
        float v;
        if constexpr (sizeof(TIn) == 4) v = x[base + i];
        else v = __uint_as_float((uint32_t)x[base + i] << 16);
        float r = w ? v * (inv * w[i]) : v * inv;
        if constexpr (sizeof(TOut) == 4) out[obase + i] = r;
        else out[obase + i] = bf16_bits(r);
    }
}

// Many rows (a prefill or an encoder pass): a warp per row, the row held in registers between the sum
// of squares and the scaling, 16-byte loads and 8- or 16-byte stores.  One read of x instead of two,
// and eight rows per block instead of one.
template <typename TOut, int NV>  // NV 16-byte pieces per lane: width = NV * 128
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(const float *x, const float *w, TOut *out, uint32_t rows,
                                                            float eps, const uint32_t *row_ids) {
    constexpr uint32_t width = NV * 128;
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)(row_ids ? row_ids[row] : row) * width);
    float4 v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        v[i] = src[i * 32 + lane];
        ss = fmaf(v[i].x, v[i].x, ss);
        ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss);
        ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = warp_sum(ss);
    pdl_launch_dependents();
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < NV; i++) {
        float4 g = make_float4(inv, inv, inv, inv);
        if (w) {
            const float4 wv = reinterpret_cast<const float4 *>(w)[i * 32 + lane];
            g = make_float4(inv * wv.x, inv * wv.y, inv * wv.z, inv * wv.w);
        }
        const float4 r = make_float4(v[i].x * g.x, v[i].y * g.y, v[i].z * g.z, v[i].w * g.w);
        const size_t at = (size_t)row * width + (size_t)(i * 32 + lane) * 4;
        if constexpr (sizeof(TOut) == 4) *reinterpret_cast<float4 *>(out + at) = r;
        else *reinterpret_cast<uint2 *>(out + at) = make_uint2(pack_bf16(r.x, r.y), pack_bf16(r.z, r.w));
    }
}

// ---- gather: engine/ir/interp/src/cpu.rs:510-525 (rows outside the table read zero)
template <typename TOut>
__global__ void __launch_bounds__(128) gather_kernel(const uint16_t *table, const uint32_t *ids, TOut *out,
                                                     uint32_t table_rows, uint32_t width, uint32_t first) {
    pdl_wait();
    const uint32_t id = ids[blockIdx.x];
    const bool inside = id >= first && id - first < table_rows;
    const uint16_t *src = table + (size_t)(inside ? id - first : 0) * width;
    for (uint32_t i = threadIdx.x; i < width; i += blockDim.x) {
        uint16_t b = inside ? src[i] : (uint16_t)0;
        if constexpr (sizeof(TOut) == 4) out[(size_t)blockIdx.x * width + i] = __uint_as_float((uint32_t)b << 16);
        else out[(size_t)blockIdx.x * width + i] = b;
    }
    pdl_launch_dependents();
}

// gather for a decoder whose first layer norm is folded into the q,k,v projection: besides the f32
// rows, leaves xs = bf16(row * gain) and the row's sum of squares in ss[row, 0] (ss[row, 1..parts) = 0).
__global__ void __launch_bounds__(128) gather_scaled_kernel(const uint16_t *table, const uint32_t *ids, float *out,
                                                            uint16_t *xs, const float *gain, float *ss, uint32_t parts,
                                                            uint32_t table_rows, uint32_t width) {
    __shared__ float scratch[4];
    pdl_wait();
    const uint32_t id = ids[blockIdx.x];
    const bool inside = id < table_rows;
    const uint16_t *src = table + (size_t)(inside ? id : 0) * width;
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = inside ? __uint_as_float((uint32_t)src[i] << 16) : 0.0f;
        out[(size_t)blockIdx.x * width + i] = v;
        xs[(size_t)blockIdx.x * width + i] = bf16_bits(v * gain[i]);
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    pdl_launch_dependents();
    if (threadIdx.x < parts) ss[(size_t)blockIdx.x * parts + threadIdx.x] = threadIdx.x == 0 ? sq : 0.0f;
}

// ---- scatter: engine/plan/lower/src/kernels/scatter.rs:11-27
__global__ void __launch_bounds__(128) scatter_kernel(const uint16_t *x, const uint32_t *slots,
                                                      const uint32_t *positions, uint16_t *out, KeptDev kept,
                                                      uint32_t width) {
    pdl_wait();
    const uint32_t r = blockIdx.x;
    const size_t dst = (size_t)kept_row(kept, slots[r], positions[r]) * width;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)r * width);
    uint4 *d = reinterpret_cast<uint4 *>(out + dst);
    for (uint32_t i = threadIdx.x; i < width / 8; i += blockDim.x) d[i] = src[i];
    pdl_launch_dependents();
}

// ---- per-head norm + rotation + append.  One warp per (row, head of q|k|v).
// Norm: engine/ir/interp/src/cpu.rs:371-377; rotation with half pairs (j, j + width/2), angle =
// position * inv_freq[j]: cpu.rs:31-47; append at kept_row(slot, position): scatter.rs:11-27.
template <int WIDTH>
__global__ void __launch_bounds__(128) qk_norm_rope_append_kernel(
    const uint16_t *qkv, const float *q_norm, const float *k_norm, const float *inv_freq, const uint32_t *slots,
    const uint32_t *positions, uint16_t *q_out, uint16_t *k_rows, uint16_t *v_rows, KeptDev kept, uint32_t rows,
    uint32_t heads, uint32_t kv_heads, float eps, uint16_t *k_dense, uint16_t *v_dense) {
    constexpr int PER = WIDTH / 64;  // pairs per lane
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t unit = blockIdx.x * 4 + (threadIdx.x >> 5);
    const uint32_t per_row = heads + 2 * kv_heads;
    if (unit >= rows * per_row) return;
    const uint32_t r = unit / per_row, h = unit % per_row;
    const uint16_t *src = qkv + ((size_t)r * per_row + h) * WIDTH;
    const uint32_t pos = positions[r];

    uint16_t *dst, *dst2 = nullptr;  // dst2: the optional packed copy [rows, kv_heads, WIDTH] of k and v
    const float *gain = nullptr;
    bool turn = true;
    if (h < heads) {
        dst = q_out + ((size_t)r * heads + h) * WIDTH;
        gain = q_norm;
    } else {
        const uint32_t kvh = (h - heads) % kv_heads;
        const bool is_v = h >= heads + kv_heads;
        const size_t at = ((size_t)kept_row(kept, slots[r], pos) * kv_heads + kvh) * WIDTH;
        dst = (is_v ? v_rows : k_rows) + at;
        uint16_t *dense = is_v ? v_dense : k_dense;
        if (dense) dst2 = dense + ((size_t)r * kv_heads + kvh) * WIDTH;
        gain = is_v ? nullptr : k_norm;
        turn = !is_v;
    }
    if (!turn) {
        // values pass through
        for (uint32_t i = lane; i < WIDTH / 8; i += 32) {
            const uint4 v = reinterpret_cast<const uint4 *>(src)[i];
            reinterpret_cast<uint4 *>(dst)[i] = v;
            if (dst2) reinterpret_cast<uint4 *>(dst2)[i] = v;
        }
        return;
    }
    // lane owns pairs j = lane * PER + e: elements j and j + WIDTH/2
    uint16_t lo[PER], hi[PER];
    norm_rope_head<WIDTH>(src, gain, inv_freq, pos, eps, lane, lo, hi);
    if constexpr (PER == 4) {
        *reinterpret_cast<uint2 *>(dst + lane * 4) =
            make_uint2((uint32_t)lo[0] | ((uint32_t)lo[1] << 16), (uint32_t)lo[2] | ((uint32_t)lo[3] << 16));
        *reinterpret_cast<uint2 *>(dst + WIDTH / 2 + lane * 4) =
            make_uint2((uint32_t)hi[0] | ((uint32_t)hi[1] << 16), (uint32_t)hi[2] | ((uint32_t)hi[3] << 16));
    } else if constexpr (PER == 2) {
        *reinterpret_cast<uint32_t *>(dst + lane * 2) = (uint32_t)lo[0] | ((uint32_t)lo[1] << 16);
        *reinterpret_cast<uint32_t *>(dst + WIDTH / 2 + lane * 2) = (uint32_t)hi[0] | ((uint32_t)hi[1] << 16);
    } else {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const uint32_t j = lane * PER + e;
            dst[j] = lo[e];
            dst[j + WIDTH / 2] = hi[e];
        }
    }
    if (dst2) {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const uint32_t j = lane * PER + e;
            dst2[j] = lo[e];
            dst2[j + WIDTH / 2] = hi[e];
        }
    }
}

// ---- top-k: engine/rules/kernels/src/argmax.rs:38-114; order engine/ir/interp/src/run.rs:577-591.
// `a` ranks before `b` when its value is larger, or equal with the lower index.  -inf and NaN never rank.
struct Cand {
    float v;
    uint32_t i;
};

__device__ __forceinline__ bool ranks_before(float av, uint32_t ai, float bv, uint32_t bi) {
    return av > bv || (av == bv && ai < bi);
}

__device__ __forceinline__ Cand best_of(Cand a, Cand b, uint32_t none) {
    if (a.i == none) return b;
    if (b.i == none) return a;
    return ranks_before(a.v, a.i, b.v, b.i) ? a : b;
}

template <typename TIn>
__device__ __forceinline__ float load_score(const TIn *x, size_t at) {
    if constexpr (sizeof(TIn) == 4) return x[at];
    else return __uint_as_float((uint32_t)x[at] << 16);
}

// One block per row; round r finds the best entry that ranks after round r - 1's pick.
template <typename TIn>
__global__ void __launch_bounds__(256) top_k_kernel(const TIn *x, uint32_t *ids, uint32_t width, uint32_t k) {
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    __shared__ Cand picked;
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * width;
    const uint32_t none = width;
    Cand prev = {INFINITY, 0};
    bool have_prev = false;
    for (uint32_t round = 0; round < k; round++) {
        Cand best = {0.0f, none};
        for (uint32_t i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = load_score(x, base + i);
            if (!(v > -INFINITY)) continue;  // -inf and NaN never rank
            if (have_prev && !ranks_before(prev.v, prev.i, v, i)) continue;  // already taken
            best = best_of(best, Cand{v, i}, none);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Cand other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
            best = best_of(best, other, none);
        }
        if ((threadIdx.x & 31) == 0) {
            sv[threadIdx.x >> 5] = best.v;
            si[threadIdx.x >> 5] = best.i;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            Cand b = {sv[0], si[0]};
            for (uint32_t w = 1; w < blockDim.x / 32; w++) b = best_of(b, Cand{sv[w], si[w]}, none);
            picked = b;
            ids[(size_t)blockIdx.x * k + round] = b.i;
        }
        __syncthreads();
        prev = picked;
        have_prev = true;
        if (prev.i == none) {
            // nothing left: spare slots hold the width
            if (threadIdx.x == 0)
                for (uint32_t r2 = round + 1; r2 < k; r2++) ids[(size_t)blockIdx.x * k + r2] = none;
            break;
        }
        __syncthreads();
    }
    pdl_launch_dependents();
}

// Narrow rows (router scores: a few hundred entries): a warp per row with the row in registers, no block
// barriers.  The order is total (value, then index), so the picks are the same as the block kernel's.
template <typename TIn, int PER>  // PER entries per lane: width <= 32 * PER
__global__ void __launch_bounds__(128) top_k_warp_kernel(const TIn *x, uint32_t *ids, uint32_t rows, uint32_t width,
                                                         uint32_t k) {
    pdl_wait();
    const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row < rows) {
        const size_t base = (size_t)row * width;
        const uint32_t none = width;
        float held[PER];
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const uint32_t i = lane + 32 * j;
            held[j] = i < width ? load_score(x, base + i) : -INFINITY;
        }
        Cand prev = {INFINITY, 0};
        for (uint32_t round = 0; round < k; round++) {
            Cand best = {0.0f, none};
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const uint32_t i = lane + 32 * j;
                const float v = held[j];
                if (!(v > -INFINITY)) continue;  // -inf and NaN never rank
                if (round > 0 && !ranks_before(prev.v, prev.i, v, i)) continue;  // already taken
                best = best_of(best, Cand{v, i}, none);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                Cand other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
                best = best_of(best, other, none);
            }
            if (lane == 0) ids[(size_t)row * k + round] = best.i;
            prev = best;
            if (best.i == none) {
                if (lane == 0)
                    for (uint32_t r2 = round + 1; r2 < k; r2++) ids[(size_t)row * k + r2] = none;  // spare slots hold the width
                break;
            }
        }
    }
    pdl_launch_dependents();
}

// k = 1 over wide rows, two stages (the reference's `peaks` + `argmax`, argmax.rs:72-114):
// stage 1 writes each part's best (value, index), stage 2 folds the parts in order.
template <typename TIn>
__global__ void __launch_bounds__(256) peaks_kernel(const TIn *x, float *peak_v, uint32_t *peak_i, uint32_t width,
                                                    uint32_t parts) {
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    pdl_wait();
    const uint32_t row = blockIdx.y, part = blockIdx.x;
    const uint32_t span = (width + parts - 1) / parts;
    const uint32_t lo = part * span, hi = min(width, lo + span);
    const uint32_t none = width;
    Cand best = {0.0f, none};
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = load_score(x, (size_t)row * width + i);
        if (!(v > -INFINITY)) continue;
        best = best_of(best, Cand{v, i}, none);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Cand other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
        best = best_of(best, other, none);
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best.v;
        si[threadIdx.x >> 5] = best.i;
    }
    __syncthreads();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        Cand b = {sv[0], si[0]};
        for (uint32_t w = 1; w < blockDim.x / 32; w++) b = best_of(b, Cand{sv[w], si[w]}, none);
        peak_v[(size_t)row * parts + part] = b.v;
        peak_i[(size_t)row * parts + part] = b.i;
    }
}

__global__ void __launch_bounds__(32) argmax_kernel(const float *peak_v, const uint32_t *peak_i, uint32_t *ids,
                                                    uint32_t width, uint32_t parts) {
    pdl_wait();
    const uint32_t row = blockIdx.x, none = width;
    Cand best = {0.0f, none};
    for (uint32_t i = threadIdx.x; i < parts; i += 32)
        best = best_of(best, Cand{peak_v[(size_t)row * parts + i], peak_i[(size_t)row * parts + i]}, none);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Cand other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
        best = best_of(best, other, none);
    }
    pdl_launch_dependents();
    if (threadIdx.x == 0) ids[row] = best.i;
}

// ---- take + softmax over the picks: engine/ir/interp/src/cpu.rs:497-508, 49-59
__global__ void __launch_bounds__(32) take_softmax_kernel(const float *x, const uint32_t *ids, float *gates,
                                                          uint32_t width, uint32_t k) {
    pdl_wait();
    const uint32_t row = blockIdx.x, lane = threadIdx.x;
    float v = -INFINITY;
    if (lane < k) {
        const uint32_t id = ids[(size_t)row * k + lane];
        v = id < width ? x[(size_t)row * width + id] : 0.0f;  // out-of-range ids read zero
    }
    const float mx = warp_max(v);
    const float e = lane < k ? expf(v - mx) : 0.0f;
    // sum in pick order, as the reference's sequential loop does
    float sum = 0.0f;
    for (uint32_t j = 0; j < k; j++) sum += __shfl_sync(0xFFFFFFFFu, e, j);
    pdl_launch_dependents();
    if (lane < k) gates[(size_t)row * k + lane] = e / sum;
}

// The device-resident decode loop's feedback: each row's next token is the id it just produced
// and its position moves on by one (engine/engine/src/lib.rs:166-200 does this on the host).
__global__ void advance_rows_kernel(const uint32_t *ids, uint32_t *tokens, uint32_t *positions, uint32_t rows) {
    pdl_wait();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) {
        tokens[r] = ids[r];
        positions[r] += 1;
    }
    pdl_launch_dependents();
}

__global__ void iota_rows_kernel(uint32_t *slots, uint32_t *positions, uint32_t total, uint32_t queries,
                                 uint32_t past) {
    pdl_wait();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < total) {
        slots[r] = r / queries;
        positions[r] = past + r % queries;
    }
    pdl_launch_dependents();
}

// Mean over each packed sequence's rows, then unit length: the embedding head.  The mean sums
// x * (1 / count) in row order (engine/ir/interp/src/cpu.rs:449-473); the unit scale divides by
// max(sqrt(sum of squares), 1e-12) (frontend/tasks/src/embed.rs:47-52).  One block per sequence.
__global__ void __launch_bounds__(256) mean_pool_kernel(const float *x, const uint32_t *cu_seqlens, float *out,
                                                        uint32_t width, int normalize) {
    __shared__ float scratch[8];
    pdl_wait();
    const uint32_t a = cu_seqlens[blockIdx.x], b = cu_seqlens[blockIdx.x + 1];
    const float w = b > a ? 1.0f / (float)(b - a) : 0.0f;
    float ss = 0.0f;
    for (uint32_t j = threadIdx.x; j < width; j += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t t = a; t < b; t++) acc = __fadd_rn(acc, __fmul_rn(x[(size_t)t * width + j], w));
        out[(size_t)blockIdx.x * width + j] = acc;
        ss = fmaf(acc, acc, ss);
    }
    if (!normalize) return;
    ss = block_sum(ss, scratch);
    const float norm = fmaxf(sqrtf(ss), 1e-12f);
    for (uint32_t j = threadIdx.x; j < width; j += blockDim.x) out[(size_t)blockIdx.x * width + j] /= norm;
}

// Holds the stream until the host sets *flag, so that launches queued behind it run back to back
// and per-kernel event intervals exclude host launch gaps.  One thread; gives up after `spins` reads
// (engine/gpu/gpukit/src/gate.cu does the same with 2^21).
__global__ void gate_kernel(const volatile uint32_t *flag, uint32_t spins) {
    for (uint32_t i = 0; i < spins; i++)
        if (*flag) return;
}

// The reference's two rotary launches (engine/rules/kernels/src/rope.rs:10-60).  `angles`: a thread per
// (position, pair) writes cos and sin of position * theta^(-2 pair / width) side by side; pairs from `turned`
// on keep angle zero.  The powers come from the host in f32 (the table ts_rope_inv_freq writes), as a kernel
// argument: the same bits as a host that computes them, which powf on the device does not promise.
struct TurnTable {
    float turn[256];
};

__global__ void __launch_bounds__(256) rope_angles_kernel(const uint32_t *positions, float *out, uint32_t count,
                                                          uint32_t width, uint32_t turned, const TurnTable table) {
    pdl_wait();
    const uint32_t pairs = width / 2, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count * pairs) {
        const uint32_t at = i / pairs, pair = i % pairs;
        float sn = 0.0f, cs = 1.0f;
        if (pair < turned) sincosf((float)positions[at] * table.turn[pair], &sn, &cs);
        reinterpret_cast<float2 *>(out)[(size_t)at * pairs + pair] = make_float2(cs, sn);
    }
    pdl_launch_dependents();
}

// `rope` / `rope_adjacent`: a thread per (position, head, pair) rotates its pair in place by the position's
// (cos, sin); pairs lie side by side (adjacent) or one in each half of the head.
template <typename T, bool ADJACENT>
__global__ void __launch_bounds__(256) rope_kernel(T *x, const float *freqs, uint32_t positions, uint32_t heads,
                                                   uint32_t width) {
    pdl_wait();
    const uint32_t pairs = width / 2;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (size_t)positions * heads * pairs) {
        const uint32_t pair = (uint32_t)(i % pairs), s = (uint32_t)(i / pairs / heads);
        T *row = x + (i / pairs) * width;
        const float2 cs = reinterpret_cast<const float2 *>(freqs)[(size_t)s * pairs + pair];
        const uint32_t a = ADJACENT ? 2 * pair : pair, b = ADJACENT ? a + 1 : pairs + pair;
        float x0, x1;
        if constexpr (sizeof(T) == 2) {
            x0 = __uint_as_float((uint32_t)row[a] << 16);
            x1 = __uint_as_float((uint32_t)row[b] << 16);
        } else {
            x0 = row[a];
            x1 = row[b];
        }
        const float ra = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
        const float rb = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
        if constexpr (sizeof(T) == 2) {
            row[a] = bf16_bits(ra);
            row[b] = bf16_bits(rb);
        } else {
            row[a] = ra;
            row[b] = rb;
        }
    }
    pdl_launch_dependents();
}

constexpr uint32_t kPeakParts = 64;

}  // namespace

int iota_rows(uint32_t *slots, uint32_t *positions, uint32_t seqs, uint32_t queries, uint32_t past,
              cudaStream_t stream) {
    const uint32_t total = seqs * queries;
    if (total == 0) return TS_OK;
    cudaError_t e = launch(iota_rows_kernel, dim3(ceil_div(total, 256)), dim3(256), 0, stream, pdl_enabled(), slots,
                           positions, total, queries, past);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of iota_rows failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int mean_pool(const float *x, const uint32_t *cu_seqlens, float *out, uint32_t seqs, uint32_t width, int normalize,
              cudaStream_t stream) {
    if (seqs == 0) return TS_OK;
    cudaError_t e = launch(mean_pool_kernel, dim3(seqs), dim3(256), 0, stream, pdl_enabled(), x, cu_seqlens, out, width,
                           normalize);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of mean_pool failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int gate(const volatile uint32_t *flag, cudaStream_t stream) {
    gate_kernel<<<1, 1, 0, stream>>>(flag, 1u << 21);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of gate failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int rope_angles(const uint32_t *positions, float *out, uint32_t count, uint32_t width, float theta, uint32_t turned,
                cudaStream_t stream) {
    TS_REQUIRE(width >= 2 && width % 2 == 0 && width <= 512, "rope angles: width %u is not an even number up to 512", width);
    if (count == 0) return TS_OK;
    TurnTable table;
    for (uint32_t j = 0; j < width / 2; j++) table.turn[j] = powf(theta, -((float)(2 * j)) / (float)width);
    const uint32_t threads = count * (width / 2);
    cudaError_t e = launch(rope_angles_kernel, dim3(ceil_div(threads, 256)), dim3(256), 0, stream, pdl_enabled(), positions,
                           out, count, width, turned, table);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of rope angles failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int rope(void *x, int dtype, const float *freqs, uint32_t positions, uint32_t heads, uint32_t width, int adjacent,
         cudaStream_t stream) {
    TS_REQUIRE(width >= 2 && width % 2 == 0, "rope: width %u is odd", width);
    const size_t threads = (size_t)positions * heads * (width / 2);
    if (threads == 0) return TS_OK;
    const dim3 grid((unsigned)((threads + 255) / 256));
    const bool pdl = pdl_enabled();
    cudaError_t e;
    if (dtype == TS_BF16)
        e = adjacent ? launch(rope_kernel<uint16_t, true>, grid, dim3(256), 0, stream, pdl, (uint16_t *)x, freqs, positions, heads, width)
                     : launch(rope_kernel<uint16_t, false>, grid, dim3(256), 0, stream, pdl, (uint16_t *)x, freqs, positions, heads, width);
    else
        e = adjacent ? launch(rope_kernel<float, true>, grid, dim3(256), 0, stream, pdl, (float *)x, freqs, positions, heads, width)
                     : launch(rope_kernel<float, false>, grid, dim3(256), 0, stream, pdl, (float *)x, freqs, positions, heads, width);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of rope failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int advance_rows(const uint32_t *ids, uint32_t *tokens, uint32_t *positions, uint32_t rows, cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    cudaError_t e = launch(advance_rows_kernel, dim3(ceil_div(rows, 128)), dim3(128), 0, stream, pdl_enabled(), ids,
                           tokens, positions, rows);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of advance_rows failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int rms_norm(const void *x, int x_dtype, const float *w, void *out, int out_dtype, uint32_t rows, uint32_t width,
             float eps, const uint32_t *row_ids, cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    cudaError_t e;
    const uint32_t threads = width >= 1024 ? 256 : 128;
    const bool pdl = pdl_enabled();
    if (x_dtype == TS_F32 && rows >= 1024 && (width == 768 || width == 1024 || width == 2048) && aligned16(x) &&
        aligned16(out) && (!w || aligned16(w))) {
        const dim3 grid(ceil_div(rows, 8));
#define TS_ROWS_CASE(NV)                                                                                              \
    (out_dtype == TS_BF16 ? launch(rms_norm_rows_kernel<uint16_t, NV>, grid, dim3(256), 0, stream, pdl, (const float *)x, w, \
                                   (uint16_t *)out, rows, eps, row_ids)                                               \
                          : launch(rms_norm_rows_kernel<float, NV>, grid, dim3(256), 0, stream, pdl, (const float *)x, w,    \
                                   (float *)out, rows, eps, row_ids))
        e = width == 768 ? TS_ROWS_CASE(6) : width == 1024 ? TS_ROWS_CASE(8) : TS_ROWS_CASE(16);
#undef TS_ROWS_CASE
        if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of rms_norm failed: %s", cudaGetErrorString(e));
        return TS_OK;
    }
    if (x_dtype == TS_F32 && out_dtype == TS_BF16)
        e = launch(rms_norm_kernel<float, uint16_t>, dim3(rows), dim3(threads), 0, stream, pdl, (const float *)x, w,
                   (uint16_t *)out, width, eps, row_ids);
    else if (x_dtype == TS_F32)
        e = launch(rms_norm_kernel<float, float>, dim3(rows), dim3(threads), 0, stream, pdl, (const float *)x, w,
                   (float *)out, width, eps, row_ids);
    else if (out_dtype == TS_BF16)
        e = launch(rms_norm_kernel<uint16_t, uint16_t>, dim3(rows), dim3(threads), 0, stream, pdl,
                   (const uint16_t *)x, w, (uint16_t *)out, width, eps, row_ids);
    else
        e = launch(rms_norm_kernel<uint16_t, float>, dim3(rows), dim3(threads), 0, stream, pdl, (const uint16_t *)x,
                   w, (float *)out, width, eps, row_ids);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of rms_norm failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int gather_rows(const void *table, const uint32_t *ids, void *out, int out_dtype, uint32_t rows,
                uint32_t table_rows, uint32_t width, uint32_t first, cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    cudaError_t e;
    if (out_dtype == TS_F32)
        e = launch(gather_kernel<float>, dim3(rows), dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)table, ids,
                   (float *)out, table_rows, width, first);
    else
        e = launch(gather_kernel<uint16_t>, dim3(rows), dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)table,
                   ids, (uint16_t *)out, table_rows, width, first);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of gather failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int gather_scaled(const void *table, const uint32_t *ids, float *out, void *xs, const float *gain, float *ss,
                  uint32_t parts, uint32_t rows, uint32_t table_rows, uint32_t width, cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    TS_REQUIRE(parts >= 1 && parts <= 128, "gather (scaled): %u partial sums per row", parts);
    cudaError_t e = launch(gather_scaled_kernel, dim3(rows), dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)table, ids,
                           out, (uint16_t *)xs, gain, ss, parts, table_rows, width);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of gather (scaled) failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int scatter_rows(const void *x, const uint32_t *slots, const uint32_t *positions, void *out, const KeptDev &kept,
                 uint32_t rows, uint32_t width, cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    cudaError_t e = launch(scatter_kernel, dim3(rows), dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)x, slots,
                           positions, (uint16_t *)out, kept, width);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of scatter failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int qk_norm_rope_append(const void *qkv, const float *q_norm, const float *k_norm, const float *inv_freq,
                        const uint32_t *slots, const uint32_t *positions, void *q_out, void *k_rows, void *v_rows,
                        const KeptDev &kept, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t width,
                        float eps, cudaStream_t stream, void *k_dense, void *v_dense) {
    if (rows == 0) return TS_OK;
    const uint32_t units = rows * (heads + 2 * kv_heads);
    dim3 grid(ceil_div(units, 4));
    cudaError_t e;
    if (width == 128)
        e = launch(qk_norm_rope_append_kernel<128>, grid, dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)qkv,
                   q_norm, k_norm, inv_freq, slots, positions, (uint16_t *)q_out, (uint16_t *)k_rows,
                   (uint16_t *)v_rows, kept, rows, heads, kv_heads, eps, (uint16_t *)k_dense, (uint16_t *)v_dense);
    else if (width == 256)
        e = launch(qk_norm_rope_append_kernel<256>, grid, dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)qkv,
                   q_norm, k_norm, inv_freq, slots, positions, (uint16_t *)q_out, (uint16_t *)k_rows,
                   (uint16_t *)v_rows, kept, rows, heads, kv_heads, eps, (uint16_t *)k_dense, (uint16_t *)v_dense);
    else if (width == 64)
        e = launch(qk_norm_rope_append_kernel<64>, grid, dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)qkv,
                   q_norm, k_norm, inv_freq, slots, positions, (uint16_t *)q_out, (uint16_t *)k_rows,
                   (uint16_t *)v_rows, kept, rows, heads, kv_heads, eps, (uint16_t *)k_dense, (uint16_t *)v_dense);
    else
        return fail(TS_ERR_BAD_INPUT, "qk_norm_rope_append: width %u is not 64, 128 or 256", width);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of qk_norm_rope_append failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

size_t top_k_workspace_bytes(uint32_t rows, uint32_t width, uint32_t k) {
    if (k == 1 && width > 8192) return (size_t)rows * kPeakParts * 8;
    return 0;
}

int top_k(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, uint32_t k, void *workspace,
          size_t workspace_bytes, cudaStream_t stream) {
    if (rows == 0 || k == 0) return TS_OK;
    cudaError_t e;
    const bool pdl = pdl_enabled();
    if (k == 1 && width > 8192) {
        size_t need = top_k_workspace_bytes(rows, width, k);
        TS_REQUIRE(workspace && workspace_bytes >= need, "top_k: workspace of %zu bytes is smaller than the %zu needed",
                   workspace_bytes, need);
        float *pv = (float *)workspace;
        uint32_t *pi = (uint32_t *)(pv + (size_t)rows * kPeakParts);
        if (x_dtype == TS_F32)
            e = launch(peaks_kernel<float>, dim3(kPeakParts, rows), dim3(256), 0, stream, pdl, (const float *)x, pv, pi,
                       width, kPeakParts);
        else
            e = launch(peaks_kernel<uint16_t>, dim3(kPeakParts, rows), dim3(256), 0, stream, pdl, (const uint16_t *)x,
                       pv, pi, width, kPeakParts);
        if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of peaks failed: %s", cudaGetErrorString(e));
        e = launch(argmax_kernel, dim3(rows), dim3(32), 0, stream, pdl, (const float *)pv, (const uint32_t *)pi, ids,
                   width, kPeakParts);
        if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of argmax failed: %s", cudaGetErrorString(e));
        return TS_OK;
    }
    if (width <= 1024) {
        const dim3 grid(ceil_div(rows, 4));
#define TS_TOPK_WARP(T, PER) launch(top_k_warp_kernel<T, PER>, grid, dim3(128), 0, stream, pdl, (const T *)x, ids, rows, width, k)
        if (x_dtype == TS_F32)
            e = width <= 128 ? TS_TOPK_WARP(float, 4) : width <= 256 ? TS_TOPK_WARP(float, 8) : TS_TOPK_WARP(float, 32);
        else
            e = width <= 128 ? TS_TOPK_WARP(uint16_t, 4) : width <= 256 ? TS_TOPK_WARP(uint16_t, 8) : TS_TOPK_WARP(uint16_t, 32);
#undef TS_TOPK_WARP
        if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of top_k failed: %s", cudaGetErrorString(e));
        return TS_OK;
    }
    if (x_dtype == TS_F32)
        e = launch(top_k_kernel<float>, dim3(rows), dim3(256), 0, stream, pdl, (const float *)x, ids, width, k);
    else
        e = launch(top_k_kernel<uint16_t>, dim3(rows), dim3(256), 0, stream, pdl, (const uint16_t *)x, ids, width, k);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of top_k failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

// ---- greedy top-1 that brings its own scratch -----------------------------------------------
// The two-stage top-1 above needs rows x 64 (value, index) pairs of scratch between its launches.
// Some hosts cannot hand a kernel any: a plug-in inside a runtime that sized every device buffer
// when it built its plan (tessera's runner does, and gives kernels no allocator), or a caller whose
// memory budget is fixed and already spent.  For them the scratch lives in this library's image: a
// file-scope device array of kStaticTopRows * 64 * 8 bytes (512 KiB), which every GPU that loads the
// library carries until the process exits.
constexpr uint32_t kStaticTopRows = 1024;
static __device__ __align__(256) unsigned char g_top1_scratch[kStaticTopRows * kPeakParts * 8];

// In host code `g_top1_scratch` is only a stand-in for the symbol, not a device address: the real
// address is looked up once per device, with that device current, and cached.
static std::atomic<void *> g_top1_scratch_addr[64] = {};  // atomic: two host threads may make their first call at once

static int top1_scratch(void **out) {
    int dev = -1;
    TS_CUDA(cudaGetDevice(&dev));
    TS_REQUIRE(dev >= 0 && dev < 64, "top_1_static: device ordinal %d is outside 0..63", dev);
    void *p = g_top1_scratch_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        TS_CUDA(cudaGetSymbolAddress(&p, g_top1_scratch));
        g_top1_scratch_addr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return TS_OK;
}

int top_1_static(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, cudaStream_t stream) {
    TS_REQUIRE(rows <= kStaticTopRows, "top_1_static: %u rows, the built-in scratch holds at most %u", rows,
               kStaticTopRows);
    if (rows == 0) return TS_OK;
    void *scratch = nullptr;
    int rc = top1_scratch(&scratch);
    if (rc != TS_OK) return rc;
    // Stage 1 writes every (row, part) pair before stage 2 reads it, so nothing has to start at zero;
    // what an earlier call left behind is simply overwritten.
    float *pv = (float *)scratch;
    uint32_t *pi = (uint32_t *)(pv + (size_t)kStaticTopRows * kPeakParts);
    const bool pdl = pdl_enabled();
    cudaError_t e;
    if (x_dtype == TS_F32)
        e = launch(peaks_kernel<float>, dim3(kPeakParts, rows), dim3(256), 0, stream, pdl, (const float *)x, pv, pi,
                   width, kPeakParts);
    else
        e = launch(peaks_kernel<uint16_t>, dim3(kPeakParts, rows), dim3(256), 0, stream, pdl, (const uint16_t *)x, pv,
                   pi, width, kPeakParts);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of peaks failed: %s", cudaGetErrorString(e));
    e = launch(argmax_kernel, dim3(rows), dim3(32), 0, stream, pdl, (const float *)pv, (const uint32_t *)pi, ids, width,
               kPeakParts);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of argmax failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

int take_softmax(const float *x, const uint32_t *ids, float *gates, uint32_t rows, uint32_t width, uint32_t k,
                 cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    cudaError_t e = launch(take_softmax_kernel, dim3(rows), dim3(32), 0, stream, pdl_enabled(), x, ids, gates, width, k);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of take_softmax failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
