// Ragged attention over kept (paged) K/V rows, one query row per (slot, position): the decode
// step's attention.  HBM-bound: every K and V row of the visible range is read exactly once per
// kv head, with 16-byte loads, and shared by the G query heads that map to that kv head.
//
// Block = 4 warps on one (row, kv head, key chunk).  A warp walks 32 keys at a time.  A key row
// of `WIDTH` bf16 is covered by WIDTH / 8 neighbouring lanes, so one load instruction fetches
// 32 * 8 / WIDTH whole keys as contiguous 16-byte pieces.  Each lane first accumulates partial
// dot products for the keys its lane group sees, then a butterfly exchange leaves every lane with
// the full score of exactly one key (log2 steps, halving the payload each time) - the softmax
// running maximum and the rescale are then plain warp shuffles.  Probabilities return to the
// lanes that hold the matching V pieces by shuffle.  The four warps merge (max, sum, output) in
// shared memory in warp order; when a row spans several chunks, per-chunk results go to the
// caller's workspace and a second kernel merges them in chunk order.  No float atomics anywhere:
// a re-run gives the same bits.
//
// Stands in for `attend_rows` (engine/rules/attention/src/attend.rs:124-167) and `flash_rows`
// (engine/rules/attention/src/flash.rs:505-580); `scatter`
// (engine/plan/lower/src/kernels/scatter.rs:11-83) and the per-head norm + rotation that precede
// it in the decoder (engine/models/src/decoder.rs:354-389) are the append kernels below.
#include <cmath>

#include "ts_common.cuh"

namespace ts {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

struct RowsParams {
    const uint16_t *q, *k, *v;
    uint16_t *out;
    const uint32_t *slots, *positions;
    KeptDev kept;
    uint32_t rows, keys, heads, kv_heads, back, ahead;
    const uint32_t *lens;  // per slot: keys that exist, or NULL
    uint32_t chunk, chunks;  // keys per chunk, chunks per row
    float scale;
    float *part_o;   // [rows, heads, chunks, WIDTH]
    float *part_ml;  // [rows, heads, chunks, 2]
    uint32_t contiguous;  // a 32-aligned block of 32 positions is 32 consecutive kept rows
};

__device__ __forceinline__ uint4 ldg16(const uint16_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int WIDTH, int G>
__global__ void __launch_bounds__(kThreads) attend_rows_kernel(const RowsParams p) {
    constexpr int LPK = WIDTH / 8;   // lanes per key
    constexpr int KPI = 32 / LPK;    // keys per load instruction
    constexpr int N = LPK;           // load instructions per 32-key block
    constexpr int NB = N < 8 ? N : 8;  // loads issued back to back before their math
    static_assert(N * KPI == 32, "a block is 32 keys");

    const uint32_t row = blockIdx.x, hg = blockIdx.y, chunk = blockIdx.z;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t group = p.heads / p.kv_heads;
    const uint32_t head0 = hg * G;
    const uint32_t kvh = head0 / group;
    const uint32_t gidx = lane / LPK, piece = lane % LPK;

    pdl_wait();
    const uint32_t slot = p.slots[row], pos = p.positions[row];
    // Visible keys [first, last): engine/ir/graph/src/node.rs:162-187 with ends aligned.
    uint32_t reach = pos + p.ahead;
    if (reach < pos || reach == 0xFFFFFFFFu) reach = 0xFFFFFFFEu;  // saturate so that reach + 1 cannot wrap
    uint32_t last = min(reach + 1, p.keys);
    if (p.lens) last = min(last, p.lens[slot]);
    const uint32_t first = pos > p.back ? pos - p.back : 0;
    const uint32_t lo = max(first, chunk * p.chunk), hi = min(last, (chunk + 1) * p.chunk);

    __shared__ float sm_o[kWarps][G][WIDTH];
    __shared__ float sm_ml[kWarps][G][2];

    const bool single = p.chunks == 1;
    if (lo >= hi) {
        // Nothing visible in this chunk.  The merge kernel skips it; a row with nothing visible
        // at all (cannot happen for causal rows) would write zeros.
        if (!single && threadIdx.x < G) {
            size_t at = (((size_t)row * p.heads + head0 + threadIdx.x) * p.chunks + chunk) * 2;
            p.part_ml[at] = -INFINITY;
            p.part_ml[at + 1] = 0.0f;
        }
        if (single) {
            for (uint32_t i = threadIdx.x; i < G * WIDTH; i += kThreads)
                p.out[((size_t)row * p.heads + head0) * WIDTH + i] = 0;
        }
        return;
    }

    // This lane's 8 dims of each of the G query heads.
    float q[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) {
        uint4 v = *reinterpret_cast<const uint4 *>(p.q + ((size_t)row * p.heads + head0 + g) * WIDTH + piece * 8);
        q[g][0] = bf16_lo(v.x); q[g][1] = bf16_hi(v.x); q[g][2] = bf16_lo(v.y); q[g][3] = bf16_hi(v.y);
        q[g][4] = bf16_lo(v.z); q[g][5] = bf16_hi(v.z); q[g][6] = bf16_lo(v.w); q[g][7] = bf16_hi(v.w);
    }

    float m[G], l[G], o[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; e++) o[g][e] = 0.0f;
    }

    const size_t row_stride = (size_t)p.kv_heads * WIDTH;  // elements between kept rows
    const size_t head_off = (size_t)kvh * WIDTH + piece * 8;

    // 32-key blocks, aligned to 32 positions so a block never straddles a page of >= 32 rows.
    const uint32_t blk_lo = lo / 32, blk_hi = (hi + 31) / 32;
    for (uint32_t blk = blk_lo + warp; blk < blk_hi; blk += kWarps) {
        const uint32_t base = blk * 32;
        // Key handled by load instruction i in this lane: base + i * KPI + gidx.
        // Key whose full score this lane ends up owning: base + piece * KPI + gidx.
        const uint32_t own = base + piece * KPI + gidx;
        const bool own_ok = own >= lo && own < hi;
        uint32_t row0 = 0, own_row = 0;
        if (p.contiguous) {
            row0 = kept_row(p.kept, slot, base);
        } else {
            own_row = kept_row(p.kept, slot, min(own, last - 1));
        }
        auto key_row = [&](int i) -> uint32_t {
            if (p.contiguous) {
                uint32_t j = base + i * KPI + gidx;
                return row0 + (min(j, last - 1) - base);
            }
            return __shfl_sync(0xFFFFFFFFu, own_row, gidx * LPK + i);
        };

        // ---- scores ----
        float s[G][N];
#pragma unroll
        for (int i0 = 0; i0 < N; i0 += NB) {
            uint4 kv[NB];
#pragma unroll
            for (int i = 0; i < NB; i++) kv[i] = ldg16(p.k + (size_t)key_row(i0 + i) * row_stride + head_off);
#pragma unroll
            for (int i = 0; i < NB; i++) {
                float f[8] = {bf16_lo(kv[i].x), bf16_hi(kv[i].x), bf16_lo(kv[i].y), bf16_hi(kv[i].y),
                              bf16_lo(kv[i].z), bf16_hi(kv[i].z), bf16_lo(kv[i].w), bf16_hi(kv[i].w)};
#pragma unroll
                for (int g = 0; g < G; g++) {
                    float a = 0.0f;
#pragma unroll
                    for (int e = 0; e < 8; e++) a = fmaf(q[g][e], f[e], a);
                    s[g][i0 + i] = a;
                }
            }
        }
        // Butterfly: after log2(LPK) exchanges lane `piece` of a group holds the group's sum for
        // load instruction i = piece.
        float score[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
#pragma unroll
            for (int off = LPK / 2; off >= 1; off /= 2) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < off; i++) {
                    float keep = upper ? s[g][i + off] : s[g][i];
                    float send = upper ? s[g][i] : s[g][i + off];
                    s[g][i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
                }
            }
            score[g] = own_ok ? s[g][0] * p.scale : -INFINITY;
        }

        // ---- online softmax (warp-wide maximum, per-lane partial sums) ----
        float prob[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            float m_new = fmaxf(m[g], warp_max(score[g]));
            float alpha = __expf(m[g] - m_new);  // m_new is finite: the block holds a visible key
            prob[g] = own_ok ? __expf(score[g] - m_new) : 0.0f;
            l[g] = l[g] * alpha + prob[g];
#pragma unroll
            for (int e = 0; e < 8; e++) o[g][e] *= alpha;
            m[g] = m_new;
        }

        // ---- values ----
#pragma unroll
        for (int i0 = 0; i0 < N; i0 += NB) {
            uint4 vv[NB];
#pragma unroll
            for (int i = 0; i < NB; i++) vv[i] = ldg16(p.v + (size_t)key_row(i0 + i) * row_stride + head_off);
#pragma unroll
            for (int i = 0; i < NB; i++) {
                float f[8] = {bf16_lo(vv[i].x), bf16_hi(vv[i].x), bf16_lo(vv[i].y), bf16_hi(vv[i].y),
                              bf16_lo(vv[i].z), bf16_hi(vv[i].z), bf16_lo(vv[i].w), bf16_hi(vv[i].w)};
#pragma unroll
                for (int g = 0; g < G; g++) {
                    // probability of key base + (i0 + i) * KPI + gidx lives in lane gidx * LPK + i0 + i
                    float pr = __shfl_sync(0xFFFFFFFFu, prob[g], gidx * LPK + i0 + i);
#pragma unroll
                    for (int e = 0; e < 8; e++) o[g][e] = fmaf(pr, f[e], o[g][e]);
                }
            }
        }
    }

    // ---- fold the KPI lane groups of a warp, then the warps of the block ----
#pragma unroll
    for (int g = 0; g < G; g++) {
        l[g] = warp_sum(l[g]);
#pragma unroll
        for (int off = LPK; off < 32; off *= 2)
#pragma unroll
            for (int e = 0; e < 8; e++) o[g][e] += __shfl_xor_sync(0xFFFFFFFFu, o[g][e], off);
        if (gidx == 0) {
#pragma unroll
            for (int e = 0; e < 8; e++) sm_o[warp][g][piece * 8 + e] = o[g][e];
        }
        if (lane == 0) {
            sm_ml[warp][g][0] = m[g];
            sm_ml[warp][g][1] = l[g];
        }
    }
    __syncthreads();
    pdl_launch_dependents();
    for (uint32_t i = threadIdx.x; i < G * WIDTH; i += kThreads) {
        const uint32_t g = i / WIDTH, d = i % WIDTH;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; w++) mm = fmaxf(mm, sm_ml[w][g][0]);
        float ll = 0.0f, oo = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            float mw = sm_ml[w][g][0];
            float f = mw == -INFINITY ? 0.0f : __expf(mw - mm);
            ll += sm_ml[w][g][1] * f;
            oo += sm_o[w][g][d] * f;
        }
        if (single) {
            p.out[((size_t)row * p.heads + head0 + g) * WIDTH + d] = bf16_bits(oo / ll);
        } else {
            size_t at = ((size_t)row * p.heads + head0 + g) * p.chunks + chunk;
            p.part_o[at * WIDTH + d] = oo;
            if (d == 0) {
                p.part_ml[at * 2] = mm;
                p.part_ml[at * 2 + 1] = ll;
            }
        }
    }
}

// One block per (row, head): folds the chunks in ascending order.
template <int WIDTH>
__global__ void __launch_bounds__(WIDTH) attend_rows_merge_kernel(const RowsParams p) {
    pdl_wait();
    const uint32_t row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    const size_t at = ((size_t)row * p.heads + head) * p.chunks;
    float mm = -INFINITY;
    for (uint32_t c = 0; c < p.chunks; c++) mm = fmaxf(mm, p.part_ml[(at + c) * 2]);
    float ll = 0.0f, oo = 0.0f;
    for (uint32_t c = 0; c < p.chunks; c++) {
        float mc = p.part_ml[(at + c) * 2];
        if (mc == -INFINITY) continue;
        float f = __expf(mc - mm);
        ll += p.part_ml[(at + c) * 2 + 1] * f;
        oo += p.part_o[(at + c) * WIDTH + d] * f;
    }
    pdl_launch_dependents();
    p.out[((size_t)row * p.heads + head) * WIDTH + d] = ll > 0.0f ? bf16_bits(oo / ll) : (uint16_t)0;
}

struct RowsPlan {
    uint32_t chunk, chunks, g;
};

RowsPlan plan_rows(uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads) {
    RowsPlan s;
    const uint32_t group = heads / kv_heads;
    s.g = group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1;
    const uint32_t base = rows * (heads / s.g);
    const uint32_t want = ceil_div((uint32_t)sm_count() * 4, base ? base : 1);
    uint32_t chunk = ceil_div(ceil_div(keys ? keys : 1, want), 128) * 128;
    chunk = chunk < 128 ? 128 : chunk > 512 ? 512 : chunk;
    // Short contexts with plenty of rows: one chunk, no merge launch.
    if (base >= 2 * (uint32_t)sm_count() && keys <= 512) chunk = ceil_div(keys, 128) * 128;
    s.chunk = chunk;
    s.chunks = ceil_div(keys ? keys : 1, chunk);
    return s;
}

template <int WIDTH, int G>
cudaError_t launch_rows(const RowsParams &p, dim3 grid, cudaStream_t stream) {
    return launch(attend_rows_kernel<WIDTH, G>, grid, dim3(kThreads), 0, stream, pdl_enabled(), p);
}

}  // namespace

size_t attend_rows_workspace_bytes(uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads, uint32_t width) {
    if (rows == 0 || heads == 0 || kv_heads == 0) return 0;
    RowsPlan s = plan_rows(rows, keys, heads, kv_heads);
    if (s.chunks <= 1) return 0;
    return (size_t)rows * heads * s.chunks * (width + 2) * sizeof(float);
}

int attend_rows(const void *q, const void *k, const void *v, void *out, const uint32_t *slots,
                const uint32_t *positions, const KeptDev &kept, bool contiguous, uint32_t rows, uint32_t keys,
                uint32_t heads, uint32_t kv_heads, uint32_t width, uint32_t back, float scale, void *workspace,
                size_t workspace_bytes, cudaStream_t stream, uint32_t ahead, const uint32_t *lens) {
    RowsPlan s = plan_rows(rows, keys, heads, kv_heads);
    size_t need = s.chunks > 1 ? (size_t)rows * heads * s.chunks * (width + 2) * sizeof(float) : 0;
    TS_REQUIRE(workspace_bytes >= need && (need == 0 || workspace != nullptr),
               "attend_rows: workspace of %zu bytes is smaller than the %zu needed", workspace_bytes, need);
    RowsParams p = {};
    p.q = (const uint16_t *)q;
    p.k = (const uint16_t *)k;
    p.v = (const uint16_t *)v;
    p.out = (uint16_t *)out;
    p.slots = slots;
    p.positions = positions;
    p.kept = kept;
    p.rows = rows;
    p.keys = keys;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.back = back;
    p.ahead = ahead;
    p.lens = lens;
    p.chunk = s.chunk;
    p.chunks = s.chunks;
    p.scale = scale;
    p.part_o = (float *)workspace;
    p.part_ml = p.part_o ? p.part_o + (size_t)rows * heads * s.chunks * width : nullptr;
    p.contiguous = contiguous ? 1 : 0;
    dim3 grid(rows, heads / s.g, s.chunks);
    cudaError_t e = cudaErrorInvalidValue;
    if (width == 128) {
        e = s.g == 4 ? launch_rows<128, 4>(p, grid, stream)
            : s.g == 2 ? launch_rows<128, 2>(p, grid, stream)
                       : launch_rows<128, 1>(p, grid, stream);
    } else if (width == 256) {
        e = s.g == 4 ? launch_rows<256, 2>(p, dim3(rows, heads / 2, s.chunks), stream)
            : s.g == 2 ? launch_rows<256, 2>(p, grid, stream)
                       : launch_rows<256, 1>(p, grid, stream);
    } else if (width == 64) {
        e = s.g == 4 ? launch_rows<64, 4>(p, grid, stream)
            : s.g == 2 ? launch_rows<64, 2>(p, grid, stream)
                       : launch_rows<64, 1>(p, grid, stream);
    }
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of attend_rows failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    if (s.chunks > 1) {
        if (width == 128) e = launch(attend_rows_merge_kernel<128>, dim3(rows, heads), dim3(128), 0, stream, pdl_enabled(), p);
        else if (width == 256) e = launch(attend_rows_merge_kernel<256>, dim3(rows, heads), dim3(256), 0, stream, pdl_enabled(), p);
        else e = launch(attend_rows_merge_kernel<64>, dim3(rows, heads), dim3(64), 0, stream, pdl_enabled(), p);
        if (e != cudaSuccess)
            return fail(TS_ERR_CUDA, "launch of attend_rows_merge failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                        cudaGetErrorString(e));
    }
    return TS_OK;
}

}  // namespace ts
