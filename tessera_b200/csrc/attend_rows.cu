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
//
// Two kernels share the arithmetic.  `attend_rows_tma_kernel` (head width 128, layouts where 32
// aligned positions are 32 consecutive kept rows) is persistent: a producer warp walks the block's
// (row, kv head, chunk) items and streams 32-key K and V tiles into a shared-memory ring with TMA,
// four consumer warps take the tiles in turn.  The copies of the next item are in flight while the
// current one is being reduced; three blocks share an SM, so twelve tile pairs (192 KB) per SM can
// be in flight, which is what keeps HBM busy (0.96 of the copy rate at 4096 keys per row).  `attend_rows_kernel` loads straight into registers and covers every other width and layout.
#include <cmath>
#include <cstdlib>

#include "head_prep.cuh"
#include "ts_common.cuh"
#include "ts_kernels.cuh"
#include "ts_ptx.cuh"

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
    // Fused front (TMA-fed kernel only; qkv NULL = off): q, k, v come raw from the projection as
    // qkv [rows, (heads + 2 kv_heads) * 128]; the kernel norms and rotates q and k itself, appends k and
    // v at kept_row(slot, position) (k, v are then written, not only read) and attends.
    const uint16_t *qkv;
    const float *q_norm, *k_norm, *inv_freq;
    uint16_t *k_out, *v_out;
    float eps;
    // With the fused front: the producer warp starts fetching key and value tiles without waiting for the
    // upstream launch.  Only for callers whose kept rows below the rows' own positions, slots, positions and
    // page table were all written two or more launches earlier in the stream (a launch starts only after
    // its predecessor has seen its own predecessor complete); the rows' own keys never come from memory.
    uint32_t early_keys;
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

// ---- TMA-fed variant ------------------------------------------------------------------------

// One ring stage per consumer warp: block n of a thread block's sequence lands in stage n % 4 and is
// reduced by consumer warp n % 4, so a stage's barrier is only ever waited on by one warp and its
// phase parity cannot be mistaken for an older one.  Depth comes from co-resident blocks.
constexpr int kTmaStages = 4;
static_assert(kTmaStages == kWarps, "one ring stage per consumer warp");
constexpr int kTmaTile = 32 * 128 * 2;  // 32 keys x 128 bf16
constexpr int kTmaThreads = 32 + kThreads;  // producer warp + the four consumer warps

template <int G>
struct TmaShared {
    static constexpr size_t ring = (size_t)kTmaStages * 2 * kTmaTile;
    static constexpr size_t o = ring;                                   // float [kWarps][G][128]
    static constexpr size_t ml = o + sizeof(float) * kWarps * G * 128;  // float [kWarps][G][2]
    static constexpr size_t bars = ml + sizeof(float) * kWarps * G * 2; // full[kTmaStages], empty[kTmaStages]
    static constexpr size_t flag = bars + sizeof(uint64_t) * 2 * kTmaStages;
    static constexpr size_t prep = flag + 16;                       // bf16 [G + 2][128]: prepared q heads, k, v
    static constexpr size_t bytes = prep + (G + 2) * 256;
};

struct ItemRange {
    uint32_t row, hg, chunk, slot, pos, lo, hi, last;
};

__device__ __forceinline__ ItemRange item_range(const RowsParams &p, uint32_t item, uint32_t n_hg) {
    ItemRange r;
    r.chunk = item % p.chunks;
    const uint32_t t = item / p.chunks;
    r.hg = t % n_hg;
    r.row = t / n_hg;
    r.slot = p.slots[r.row];
    const uint32_t pos = r.pos = p.positions[r.row];
    uint32_t reach = pos + p.ahead;
    if (reach < pos || reach == 0xFFFFFFFFu) reach = 0xFFFFFFFEu;
    r.last = min(reach + 1, p.keys);
    if (p.lens) r.last = min(r.last, p.lens[r.slot]);
    const uint32_t first = pos > p.back ? pos - p.back : 0;
    r.lo = max(first, r.chunk * p.chunk);
    r.hi = min(r.last, (r.chunk + 1) * p.chunk);
    return r;
}

template <int G>
__global__ void __launch_bounds__(kTmaThreads, G == 4 ? 2 : 3)
attend_rows_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const RowsParams p, const uint32_t items, int *status) {
    using namespace ptx;
    using Sh = TmaShared<G>;
    constexpr int WIDTH = 128, LPK = 16, KPI = 2, N = 16, NB = 8;
    extern __shared__ __align__(1024) uint8_t smem[];
    float (*sm_o)[G][WIDTH] = reinterpret_cast<float (*)[G][WIDTH]>(smem + Sh::o);
    float (*sm_ml)[G][2] = reinterpret_cast<float (*)[G][2]>(smem + Sh::ml);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + Sh::bars);
    uint64_t *empty = full + kTmaStages;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + Sh::flag);

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n_hg = p.heads / G, group = p.heads / p.kv_heads;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTmaStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    __syncthreads();
    if (!(p.early_keys && warp == 0)) {
        pdl_wait();  // q, the positions and the newest kept rows come from the upstream kernels
        pdl_launch_dependents();
    }

    if (warp == 0) {
        // ---- producer: one tile pair per 32-key block, in item order ----
        bool ok = true;
        uint32_t odd = 0, any = 0;  // per stage: parity of the copies issued so far, and whether there were any
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            const ItemRange r = item_range(p, item, n_hg);
            if (r.lo >= r.hi) continue;
            const int32_t x = (int32_t)((r.hg * G / group) * WIDTH);
            const uint32_t blk_lo = r.lo / 32, blk_hi = (r.hi + 31) / 32;
            for (uint32_t b0 = blk_lo; b0 < blk_hi; b0 += 32) {
                // the lanes look up the kept rows of up to 32 blocks side by side
                const uint32_t mine = b0 + lane;
                const uint32_t row0 = mine < blk_hi ? kept_row(p.kept, r.slot, mine * 32) : 0;
                const uint32_t cnt = min(32u, blk_hi - b0);
                for (uint32_t j = 0; j < cnt; j++) {
                    const uint32_t y = __shfl_sync(0xFFFFFFFFu, row0, j);
                    // block b of an item goes to stage (and consumer warp) b % 4, whatever came before
                    const uint32_t s = (b0 - blk_lo + j) & (kTmaStages - 1);
                    if (lane == 0 && ok) {
                        ok = mbar_wait_or_abort(&empty[s], ((odd >> s) & 1) ^ 1, abort_flag);
                        if (ok) {
                            odd ^= 1u << s;
                            any |= 1u << s;
                            uint8_t *dst = smem + (size_t)s * 2 * kTmaTile;
                            mbar_expect_tx(&full[s], 2 * kTmaTile);
                            tma_load_2d(dst, &map_k, &full[s], x, (int32_t)y);
                            tma_load_2d(dst + kTmaTile, &map_v, &full[s], x, (int32_t)y);
                        }
                    }
                }
            }
        }
        // Every copy issued has been waited for by a consumer before that consumer leaves, or the
        // block gave up: then wait (bounded) for the copies still in flight so none lands after exit.
        if (lane == 0 && !ok) {
            for (uint32_t s = 0; s < (uint32_t)kTmaStages; s++)
                if (((any >> s) & 1) && !mbar_wait(&full[s], ((odd >> s) & 1) ^ 1)) break;
        }
    } else {
        // ---- consumers ----
        const uint32_t cw = warp - 1, ct = threadIdx.x - 32;
        const uint32_t gidx = lane / LPK, piece = lane % LPK;
        bool ok = true;
        uint32_t used = 0;  // tiles this warp has taken from its stage
        const uint32_t s = cw;
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            const ItemRange r = item_range(p, item, n_hg);
            const uint32_t head0 = r.hg * G;
            const bool single = p.chunks == 1;
            if (r.lo >= r.hi) {
                if (!single && ct < G) {
                    size_t at = (((size_t)r.row * p.heads + head0 + ct) * p.chunks + r.chunk) * 2;
                    p.part_ml[at] = -INFINITY;
                    p.part_ml[at + 1] = 0.0f;
                }
                if (single)
                    for (uint32_t i = ct; i < G * WIDTH; i += kThreads)
                        p.out[((size_t)r.row * p.heads + head0) * WIDTH + i] = 0;
                continue;
            }
            const bool own_key_here = p.qkv && r.pos >= r.lo && r.pos < r.hi;  // this item holds the row's new key
            if (p.qkv) {
                // Prepare the G query heads and the row's new key and value: a warp per head, as the
                // stand-alone append kernel does it (same code, same bits), into shared memory.
                uint16_t *prep = reinterpret_cast<uint16_t *>(smem + Sh::prep);
                const uint32_t per_row = p.heads + 2 * p.kv_heads, kvh = head0 / group;
                for (uint32_t u = cw; u < (uint32_t)G + 2; u += kWarps) {
                    const bool is_q = u < (uint32_t)G, is_v = u == (uint32_t)G + 1;
                    if (!is_q && !own_key_here) continue;
                    const uint32_t h = is_q ? head0 + u : (is_v ? p.heads + p.kv_heads + kvh : p.heads + kvh);
                    const uint16_t *src = p.qkv + ((size_t)r.row * per_row + h) * WIDTH;
                    uint16_t *dst = prep + u * WIDTH;
                    if (is_v) {
                        if (lane < 16) reinterpret_cast<uint4 *>(dst)[lane] = reinterpret_cast<const uint4 *>(src)[lane];
                    } else {
                        uint16_t lo[2], hi[2];
                        norm_rope_head<WIDTH>(src, is_q ? p.q_norm : p.k_norm, p.inv_freq, r.pos, p.eps, lane, lo, hi);
                        *reinterpret_cast<uint32_t *>(dst + lane * 2) = (uint32_t)lo[0] | ((uint32_t)lo[1] << 16);
                        *reinterpret_cast<uint32_t *>(dst + WIDTH / 2 + lane * 2) = (uint32_t)hi[0] | ((uint32_t)hi[1] << 16);
                    }
                    __syncwarp();
                    // The first query-head group of a kv head also stores the new row for later steps.
                    if (!is_q && head0 % group == 0 && lane < 16) {
                        const size_t at = ((size_t)kept_row(p.kept, r.slot, r.pos) * p.kv_heads + kvh) * WIDTH;
                        reinterpret_cast<uint4 *>((is_v ? p.v_out : p.k_out) + at)[lane] = reinterpret_cast<const uint4 *>(dst)[lane];
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
            }
            float q[G][8];
#pragma unroll
            for (int g = 0; g < G; g++) {
                uint4 v;
                if (p.qkv) v = *reinterpret_cast<const uint4 *>(smem + Sh::prep + g * 256 + piece * 16);
                else v = *reinterpret_cast<const uint4 *>(p.q + ((size_t)r.row * p.heads + head0 + g) * WIDTH + piece * 8);
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
            const uint32_t blk_lo = r.lo / 32, blk_hi = (r.hi + 31) / 32;
            for (uint32_t blk = blk_lo + cw; blk < blk_hi; blk += kWarps) {
                if (ok) ok = mbar_wait_or_abort(&full[s], used & 1, abort_flag);
                used++;
                if (ok) {
                    const uint8_t *tile_k = smem + (size_t)s * 2 * kTmaTile;
                    uint8_t *tile_v = smem + (size_t)s * 2 * kTmaTile + kTmaTile;
                    const uint32_t base = blk * 32;
                    const uint32_t own = base + piece * KPI + gidx;
                    const bool own_ok = own >= r.lo && own < r.hi;
                    if (own_key_here && r.pos - base < 32) {
                        // The copy read this row before (or while) it was appended: take it from the
                        // prepared values instead.
                        const uint8_t *from = smem + Sh::prep + (G + (lane >> 4)) * 256 + (lane & 15) * 16;
                        uint8_t *to = (lane < 16 ? const_cast<uint8_t *>(tile_k) : tile_v) + (r.pos - base) * 256 + (lane & 15) * 16;
                        *reinterpret_cast<uint4 *>(to) = *reinterpret_cast<const uint4 *>(from);
                        fence_async_shared();
                        __syncwarp();
                    }
                    if (base < r.lo || base + 32 > r.hi) {
                        // An edge block: rows outside the range may hold anything (a page's unwritten
                        // tail); zero their V so that a zero probability cannot meet a NaN.
                        for (uint32_t j = 0; j < 32; j++) {
                            const uint32_t key = base + j;
                            if (key < r.lo || key >= r.hi)
                                *reinterpret_cast<uint2 *>(tile_v + j * 256 + lane * 8) = make_uint2(0, 0);
                        }
                        fence_async_shared();  // these stores precede the next copy into this stage
                        __syncwarp();
                    }
                    // ---- scores ----
                    float sc[G][N];
#pragma unroll
                    for (int i0 = 0; i0 < N; i0 += NB) {
                        uint4 kv[NB];
#pragma unroll
                        for (int i = 0; i < NB; i++)
                            kv[i] = *reinterpret_cast<const uint4 *>(tile_k + ((i0 + i) * KPI + gidx) * 256 + piece * 16);
#pragma unroll
                        for (int i = 0; i < NB; i++) {
                            float f[8] = {bf16_lo(kv[i].x), bf16_hi(kv[i].x), bf16_lo(kv[i].y), bf16_hi(kv[i].y),
                                          bf16_lo(kv[i].z), bf16_hi(kv[i].z), bf16_lo(kv[i].w), bf16_hi(kv[i].w)};
#pragma unroll
                            for (int g = 0; g < G; g++) {
                                float a = 0.0f;
#pragma unroll
                                for (int e = 0; e < 8; e++) a = fmaf(q[g][e], f[e], a);
                                sc[g][i0 + i] = a;
                            }
                        }
                    }
                    float prob[G];
#pragma unroll
                    for (int g = 0; g < G; g++) {
#pragma unroll
                        for (int off = LPK / 2; off >= 1; off /= 2) {
                            const bool upper = (lane & off) != 0;
#pragma unroll
                            for (int i = 0; i < off; i++) {
                                float keep = upper ? sc[g][i + off] : sc[g][i];
                                float send = upper ? sc[g][i] : sc[g][i + off];
                                sc[g][i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
                            }
                        }
                        const float score = own_ok ? sc[g][0] * p.scale : -INFINITY;
                        const float m_new = fmaxf(m[g], warp_max(score));
                        const float alpha = __expf(m[g] - m_new);
                        prob[g] = own_ok ? __expf(score - m_new) : 0.0f;
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
                        for (int i = 0; i < NB; i++)
                            vv[i] = *reinterpret_cast<const uint4 *>(tile_v + ((i0 + i) * KPI + gidx) * 256 + piece * 16);
#pragma unroll
                        for (int i = 0; i < NB; i++) {
                            float f[8] = {bf16_lo(vv[i].x), bf16_hi(vv[i].x), bf16_lo(vv[i].y), bf16_hi(vv[i].y),
                                          bf16_lo(vv[i].z), bf16_hi(vv[i].z), bf16_lo(vv[i].w), bf16_hi(vv[i].w)};
#pragma unroll
                            for (int g = 0; g < G; g++) {
                                float pr = __shfl_sync(0xFFFFFFFFu, prob[g], gidx * LPK + i0 + i);
#pragma unroll
                                for (int e = 0; e < 8; e++) o[g][e] = fmaf(pr, f[e], o[g][e]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            // ---- fold the two lane groups of a warp, then the four warps ----
#pragma unroll
            for (int g = 0; g < G; g++) {
                l[g] = warp_sum(l[g]);
#pragma unroll
                for (int e = 0; e < 8; e++) o[g][e] += __shfl_xor_sync(0xFFFFFFFFu, o[g][e], 16);
                if (gidx == 0) {
#pragma unroll
                    for (int e = 0; e < 8; e++) sm_o[cw][g][piece * 8 + e] = o[g][e];
                }
                if (lane == 0) {
                    sm_ml[cw][g][0] = m[g];
                    sm_ml[cw][g][1] = l[g];
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
            for (uint32_t i = ct; i < G * WIDTH; i += kThreads) {
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
                    p.out[((size_t)r.row * p.heads + head0 + g) * WIDTH + d] = ll > 0.0f ? bf16_bits(oo / ll) : (uint16_t)0;
                } else {
                    size_t at = ((size_t)r.row * p.heads + head0 + g) * p.chunks + r.chunk;
                    p.part_o[at * WIDTH + d] = oo;
                    if (d == 0) {
                        p.part_ml[at * 2] = mm;
                        p.part_ml[at * 2 + 1] = ll;
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(status, TS_ERR_TIMEOUT);
}

// ---- four query heads per kv head: the arithmetic on the tensor cores -------------------------
//
// With four heads sharing every key the scalar kernel above is bound by its FMA and shuffle count, not
// by HBM.  This variant keeps its skeleton (persistent blocks, producer warp, one ring stage per consumer
// warp, split-KV merge) and does the two products of a 32-key tile with warp MMAs (m16n8k16, bf16 in,
// f32 out): S[16 x 32] = Q[16 x 128] K^T with the four heads in rows 0-3 of the 16-row operand (the rest
// zero), then O[16 x 128] += P[16 x 32] V.  About 170 instructions per tile and warp instead of 1700.
// K and V tiles arrive as two 64-column halves with the 128-byte swizzle so that ldmatrix reads them
// without bank conflicts (K as is for the B operand of Q K^T, V transposed for the B operand of P V).
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// d (+)= a * b; rows 8-15 of a are zero here, so their two accumulators (z0, z1) stay zero.
__device__ __forceinline__ void mma_16816(float &d0, float &d1, float &z0, float &z1, uint32_t a0, uint32_t a2, uint32_t b0,
                                          uint32_t b1) {
    const uint32_t zero = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d0), "+f"(d1), "+f"(z0), "+f"(z1)
                 : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}
// byte offset of 16-byte piece `chunk16` (of 16) of row `row` in a tile held as two swizzled 64-column halves
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk16) {
    return (chunk16 >> 3) * 4096 + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4);
}

// CW consumer warps (and ring stages) per block.  Three: 53 KB and 128 threads, so four blocks share an SM
// and a decode batch of 64 rows x 8 kv heads (512 short items) is resident at once instead of queueing a
// second item behind a third of the blocks.  Four (two blocks per SM, no register cap to speak of): long items.
template <int G, int CW>
struct MmaShared {
    static constexpr size_t ring = (size_t)CW * 2 * kTmaTile;
    static constexpr size_t o = ring;                               // float [CW][G][128]
    static constexpr size_t ml = o + sizeof(float) * CW * G * 128;  // float [CW][G][2]
    static constexpr size_t bars = ml + sizeof(float) * CW * G * 2; // full[CW], empty[CW]
    static constexpr size_t flag = bars + sizeof(uint64_t) * 2 * CW;
    static constexpr size_t prep = (flag + 16 + 15) / 16 * 16;      // bf16 [G + 2][128]
    static constexpr size_t bytes = prep + (G + 2) * 256;
};

template <int G, int CW>
__global__ void __launch_bounds__(32 + CW * 32, CW == 3 ? 4 : 2)
attend_rows_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const RowsParams p, const uint32_t items, int *status) {
    using namespace ptx;
    constexpr int WIDTH = 128;
    using Sh = MmaShared<G, CW>;
    constexpr int kMmaWarps = CW, kMmaConsumers = CW * 32;
    extern __shared__ __align__(1024) uint8_t smem[];
    float (*sm_o)[G][WIDTH] = reinterpret_cast<float (*)[G][WIDTH]>(smem + Sh::o);
    float (*sm_ml)[G][2] = reinterpret_cast<float (*)[G][2]>(smem + Sh::ml);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + Sh::bars);
    uint64_t *empty = full + kMmaWarps;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + Sh::flag);

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n_hg = p.heads / G, group = p.heads / p.kv_heads;
    if (threadIdx.x == 0) STAMP(0);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMmaWarps; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    __syncthreads();
    if (threadIdx.x == 0) STAMP(1);
    // With early keys nothing waits for the upstream launch here: the producer never needs it, and the consumers
    // first fetch what their item needs that the projection does not write (slot, position, angles, norm gains).
    bool upstream_seen = false;
    if (!p.early_keys) {
        pdl_wait();
        pdl_launch_dependents();
        upstream_seen = true;
    }
    if (threadIdx.x == 32) STAMP(2);

    if (warp == 0) {
        // ---- producer: as in the scalar kernel, each tile as two 64-column halves ----
        bool ok = true;
        uint32_t odd = 0, any = 0;
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            const ItemRange r = item_range(p, item, n_hg);
            if (r.lo >= r.hi) continue;
            const int32_t x = (int32_t)((r.hg * G / group) * WIDTH);
            const uint32_t blk_lo = r.lo / 32, blk_hi = (r.hi + 31) / 32;
            for (uint32_t b0 = blk_lo; b0 < blk_hi; b0 += 32) {
                const uint32_t mine = b0 + lane;
                const uint32_t row0 = mine < blk_hi ? kept_row(p.kept, r.slot, mine * 32) : 0;
                const uint32_t cnt = min(32u, blk_hi - b0);
                for (uint32_t j = 0; j < cnt; j++) {
                    const uint32_t y = __shfl_sync(0xFFFFFFFFu, row0, j);
                    const uint32_t s = (b0 - blk_lo + j) % kMmaWarps;
                    if (lane == 0 && ok) {
                        ok = mbar_wait_or_abort(&empty[s], ((odd >> s) & 1) ^ 1, abort_flag);
                        if (ok) {
                            odd ^= 1u << s;
                            any |= 1u << s;
                            uint8_t *dst = smem + (size_t)s * 2 * kTmaTile;
                            mbar_expect_tx(&full[s], 2 * kTmaTile);
                            tma_load_2d(dst, &map_k, &full[s], x, (int32_t)y);
                            tma_load_2d(dst + 4096, &map_k, &full[s], x + 64, (int32_t)y);
                            tma_load_2d(dst + kTmaTile, &map_v, &full[s], x, (int32_t)y);
                            tma_load_2d(dst + kTmaTile + 4096, &map_v, &full[s], x + 64, (int32_t)y);
                            if (b0 - blk_lo + j == 0) STAMP(3);
                            STAMP(4);
                        }
                    }
                }
            }
        }
        if (lane == 0 && !ok) {
            for (uint32_t s = 0; s < (uint32_t)kMmaWarps; s++)
                if (((any >> s) & 1) && !mbar_wait(&full[s], ((odd >> s) & 1) ^ 1)) break;
        }
    } else {
        // ---- consumers ----
        const uint32_t cw = warp - 1, ct = threadIdx.x - 32;
        const uint32_t hrow = lane >> 2, quad = lane & 3;  // fragment row (= head when < 4) and column pair
        bool ok = true;
        uint32_t used = 0;
        const uint32_t s = cw;
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            const ItemRange r = item_range(p, item, n_hg);
            const uint32_t head0 = r.hg * G;
            const bool single = p.chunks == 1;
            if (r.lo >= r.hi) {
                if (!upstream_seen) {
                    pdl_wait();
                    pdl_launch_dependents();
                    upstream_seen = true;
                }
                if (!single && ct < G) {
                    size_t at = (((size_t)r.row * p.heads + head0 + ct) * p.chunks + r.chunk) * 2;
                    p.part_ml[at] = -INFINITY;
                    p.part_ml[at + 1] = 0.0f;
                }
                if (single)
                    for (uint32_t i = ct; i < G * WIDTH; i += kMmaConsumers)
                        p.out[((size_t)r.row * p.heads + head0) * WIDTH + i] = 0;
                continue;
            }
            const bool own_key_here = p.qkv && r.pos >= r.lo && r.pos < r.hi;
            HeadTurn<WIDTH> turn = {};
            float gq[WIDTH / 32], gk[WIDTH / 32];
            uint32_t own_row = 0;
            if (p.qkv) {  // none of this is the projection's output: it is in registers before the wait below ends
                turn = head_turn<WIDTH>(p.inv_freq, r.pos, lane);
                head_gains<WIDTH>(p.q_norm, lane, gq);
                head_gains<WIDTH>(p.k_norm, lane, gk);
                own_row = kept_row(p.kept, r.slot, r.pos);
            }
            if (!upstream_seen) {
                pdl_wait();
                pdl_launch_dependents();
                upstream_seen = true;
            }
            if (p.qkv) {
                uint16_t *prep = reinterpret_cast<uint16_t *>(smem + Sh::prep);
                const uint32_t per_row = p.heads + 2 * p.kv_heads, kvh = head0 / group;
                for (uint32_t u = cw; u < (uint32_t)G + 2; u += kMmaWarps) {
                    const bool is_q = u < (uint32_t)G, is_v = u == (uint32_t)G + 1;
                    if (!is_q && !own_key_here) continue;
                    const uint32_t h = is_q ? head0 + u : (is_v ? p.heads + p.kv_heads + kvh : p.heads + kvh);
                    const uint16_t *src = p.qkv + ((size_t)r.row * per_row + h) * WIDTH;
                    uint16_t *dst = prep + u * WIDTH;
                    if (is_v) {
                        if (lane < 16) reinterpret_cast<uint4 *>(dst)[lane] = reinterpret_cast<const uint4 *>(src)[lane];
                    } else {
                        uint16_t lo[2], hi[2];
                        norm_rope_head_with<WIDTH>(src, (is_q ? p.q_norm : p.k_norm) != nullptr, is_q ? gq : gk, turn, p.eps, lane, lo, hi);
                        *reinterpret_cast<uint32_t *>(dst + lane * 2) = (uint32_t)lo[0] | ((uint32_t)lo[1] << 16);
                        *reinterpret_cast<uint32_t *>(dst + WIDTH / 2 + lane * 2) = (uint32_t)hi[0] | ((uint32_t)hi[1] << 16);
                    }
                    __syncwarp();
                    if (!is_q && head0 % group == 0 && lane < 16) {
                        const size_t at = ((size_t)own_row * p.kv_heads + kvh) * WIDTH;
                        reinterpret_cast<uint4 *>((is_v ? p.v_out : p.k_out) + at)[lane] = reinterpret_cast<const uint4 *>(dst)[lane];
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kMmaConsumers) : "memory");
            }
            if (threadIdx.x == 32) STAMP(5);
            // Q as the A operand: rows 0-3 are the four heads (lanes 0-15), rows 4-15 zero.  Per 16-wide
            // k step: qa[t][0] = dims 16 t + 2 quad, +1; qa[t][1] = the same + 8.
            uint32_t qa[8][2];
#pragma unroll
            for (int t = 0; t < 8; t++) {
                qa[t][0] = qa[t][1] = 0;
                if (hrow < (uint32_t)G) {
                    const uint32_t d = 16 * t + 2 * quad;
                    if (p.qkv) {
                        const uint8_t *qs = smem + Sh::prep + hrow * 256;
                        qa[t][0] = *reinterpret_cast<const uint32_t *>(qs + d * 2);
                        qa[t][1] = *reinterpret_cast<const uint32_t *>(qs + (d + 8) * 2);
                    } else {
                        const uint16_t *qg = p.q + ((size_t)r.row * p.heads + head0 + hrow) * WIDTH;
                        qa[t][0] = *reinterpret_cast<const uint32_t *>(qg + d);
                        qa[t][1] = *reinterpret_cast<const uint32_t *>(qg + d + 8);
                    }
                }
            }
            float m_row = -INFINITY, l_row = 0.0f;  // of head `hrow` (rows 4-7: never read)
            float oacc[16][2];                       // O[hrow][8 n + 2 quad, +1]
            float z0 = 0.0f, z1 = 0.0f;              // rows 8-15 of every product: stay zero
#pragma unroll
            for (int n = 0; n < 16; n++) oacc[n][0] = oacc[n][1] = 0.0f;

            const uint32_t blk_lo = r.lo / 32, blk_hi = (r.hi + 31) / 32;
            for (uint32_t blk = blk_lo + cw; blk < blk_hi; blk += kMmaWarps) {
                if (ok) ok = mbar_wait_or_abort(&full[s], used & 1, abort_flag);
                if (threadIdx.x == 32) { if (blk == blk_lo + cw) STAMP(6); STAMP(7); }
                used++;
                if (ok) {
                    uint8_t *tile_k = smem + (size_t)s * 2 * kTmaTile;
                    uint8_t *tile_v = tile_k + kTmaTile;
                    const uint32_t base = blk * 32;
                    if (own_key_here && r.pos - base < 32) {
                        // the row's own key and value, from the prepared copies (the tile was read before or
                        // while they were appended)
                        const uint32_t c16 = lane & 15, row = r.pos - base;
                        const uint8_t *from = smem + Sh::prep + (G + (lane >> 4)) * 256 + c16 * 16;
                        uint8_t *to = (lane < 16 ? tile_k : tile_v) + swz(row, c16);
                        *reinterpret_cast<uint4 *>(to) = *reinterpret_cast<const uint4 *>(from);
                        fence_async_shared();
                        __syncwarp();
                    }
                    if (base < r.lo || base + 32 > r.hi) {
                        // rows outside the range may hold anything: zero their V (both halves)
                        for (uint32_t j = 0; j < 32; j++) {
                            const uint32_t key = base + j;
                            if (key < r.lo || key >= r.hi)
                                *reinterpret_cast<uint2 *>(tile_v + (lane >> 4) * 4096 + j * 128 + (lane & 15) * 8) = make_uint2(0, 0);
                        }
                        fence_async_shared();
                        __syncwarp();
                    }
                    // ---- S = Q K^T: four 8-key column tiles ----
                    const uint32_t k_addr = smem_addr(tile_k), v_addr = smem_addr(tile_v);
                    const uint32_t mtx = lane >> 3, mrow = lane & 7;
                    float sc[4][2];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        sc[j][0] = sc[j][1] = 0.0f;
#pragma unroll
                        for (int p4 = 0; p4 < 4; p4++) {
                            uint32_t b[4];
                            ldsm_x4(k_addr + swz(8 * j + mrow, 4 * p4 + mtx), b);
                            mma_16816(sc[j][0], sc[j][1], z0, z1, qa[2 * p4][0], qa[2 * p4][1], b[0], b[1]);
                            mma_16816(sc[j][0], sc[j][1], z0, z1, qa[2 * p4 + 1][0], qa[2 * p4 + 1][1], b[2], b[3]);
                        }
                    }
                    // ---- softmax over the tile's keys; this lane holds keys base + 8 j + 2 quad, +1 of head hrow ----
                    float mx = -INFINITY;
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const uint32_t key = base + 8 * j + 2 * quad + e;
                            sc[j][e] = (key >= r.lo && key < r.hi) ? sc[j][e] * p.scale : -INFINITY;
                            mx = fmaxf(mx, sc[j][e]);
                        }
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
                    const float m_new = fmaxf(m_row, mx);  // finite: the tile holds a visible key
                    const float alpha = __expf(m_row - m_new);
                    m_row = m_new;
                    uint32_t pa[2][2];  // P as the A operand of the two 16-key steps
                    float sum = 0.0f;
#pragma unroll
                    for (int u = 0; u < 2; u++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const float p0 = __expf(sc[2 * u + h][0] - m_new), p1 = __expf(sc[2 * u + h][1] - m_new);
                            sum += p0 + p1;
                            pa[u][h] = pack_bf16(p0, p1);
                        }
                    l_row = l_row * alpha + sum;
#pragma unroll
                    for (int n = 0; n < 16; n++) {
                        oacc[n][0] *= alpha;
                        oacc[n][1] *= alpha;
                    }
                    // ---- O += P V: two 16-key steps, sixteen 8-dim column tiles two at a time ----
#pragma unroll
                    for (int u = 0; u < 2; u++)
#pragma unroll
                        for (int n2 = 0; n2 < 8; n2++) {
                            uint32_t b[4];
                            ldsm_x4_trans(v_addr + swz(16 * u + (mtx & 1) * 8 + mrow, 2 * n2 + (mtx >> 1)), b);
                            mma_16816(oacc[2 * n2][0], oacc[2 * n2][1], z0, z1, pa[u][0], pa[u][1], b[0], b[1]);
                            mma_16816(oacc[2 * n2 + 1][0], oacc[2 * n2 + 1][1], z0, z1, pa[u][0], pa[u][1], b[2], b[3]);
                        }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (threadIdx.x == 32) STAMP(8);
            // ---- this warp's partial to shared memory, then the four warps fold ----
            l_row += __shfl_xor_sync(0xFFFFFFFFu, l_row, 1);
            l_row += __shfl_xor_sync(0xFFFFFFFFu, l_row, 2);
            if (hrow < (uint32_t)G) {
#pragma unroll
                for (int n = 0; n < 16; n++)
                    *reinterpret_cast<float2 *>(&sm_o[cw][hrow][8 * n + 2 * quad]) = make_float2(oacc[n][0], oacc[n][1]);
                if (quad == 0) {
                    sm_ml[cw][hrow][0] = m_row;
                    sm_ml[cw][hrow][1] = l_row;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kMmaConsumers) : "memory");
            for (uint32_t i = ct; i < G * WIDTH; i += kMmaConsumers) {
                const uint32_t g = i / WIDTH, d = i % WIDTH;
                float mm = -INFINITY;
#pragma unroll
                for (int w = 0; w < kMmaWarps; w++) mm = fmaxf(mm, sm_ml[w][g][0]);
                float ll = 0.0f, oo = 0.0f;
#pragma unroll
                for (int w = 0; w < kMmaWarps; w++) {
                    float mw = sm_ml[w][g][0];
                    float f = mw == -INFINITY ? 0.0f : __expf(mw - mm);
                    ll += sm_ml[w][g][1] * f;
                    oo += sm_o[w][g][d] * f;
                }
                if (single) {
                    p.out[((size_t)r.row * p.heads + head0 + g) * WIDTH + d] = ll > 0.0f ? bf16_bits(oo / ll) : (uint16_t)0;
                } else {
                    size_t at = ((size_t)r.row * p.heads + head0 + g) * p.chunks + r.chunk;
                    p.part_o[at * WIDTH + d] = oo;
                    if (d == 0) {
                        p.part_ml[at * 2] = mm;
                        p.part_ml[at * 2 + 1] = ll;
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kMmaConsumers) : "memory");
            if (threadIdx.x == 32) STAMP(9);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) STAMP(10);
    if (threadIdx.x == 0 && *abort_flag) atomicExch(status, TS_ERR_TIMEOUT);
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

__device__ int g_rows_status = 0;

// TS_ROWS_MMA=0 keeps the scalar TMA-fed kernel (for A/B timing).
bool rows_mma_enabled() {
    static const bool off = [] {
        const char *v = getenv("TS_ROWS_MMA");
        return v && v[0] == '0';
    }();
    return !off;
}

template <int G>
int launch_rows_tma(const CUtensorMap &map_k, const CUtensorMap &map_v, const RowsParams &p, uint32_t items,
                    cudaStream_t stream) {
    using Sh = TmaShared<G>;
    static OncePerDevice configured;
    if (configured.needs()) {
        TS_CUDA(cudaFuncSetAttribute(attend_rows_tma_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sh::bytes));
        configured.done();
    }
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_rows_status));
    const uint32_t grid = min(items, (uint32_t)sm_count() * (G == 4 ? 2 : 3));
    cudaError_t e = launch(attend_rows_tma_kernel<G>, dim3(grid), dim3(kTmaThreads), Sh::bytes, stream, pdl_enabled(),
                           map_k, map_v, p, items, status);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of attend_rows (tma) failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

template <int G, int CW>
int launch_rows_mma(const CUtensorMap &map_k, const CUtensorMap &map_v, const RowsParams &p, uint32_t items,
                    cudaStream_t stream) {
    using Sh = MmaShared<G, CW>;
    static OncePerDevice configured;
    if (configured.needs()) {
        TS_CUDA(cudaFuncSetAttribute(attend_rows_mma_kernel<G, CW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sh::bytes));
        configured.done();
    }
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_rows_status));
    const uint32_t grid = min(items, (uint32_t)sm_count() * (CW == 3 ? 4 : 2));
    cudaError_t e = launch(attend_rows_mma_kernel<G, CW>, dim3(grid), dim3(32 + CW * 32), Sh::bytes, stream, pdl_enabled(), map_k,
                           map_v, p, items, status);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of attend_rows (mma) failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace

#ifdef TS_DEBUG_STAMPS
extern "C" __attribute__((visibility("default"))) int ts_debug_attend_stamps(unsigned long long *out) {
    return cudaMemcpyFromSymbol(out, g_stamps, sizeof(unsigned long long) * 16 * 32) == cudaSuccess ? 0 : 6;
}
#endif

bool attend_rows_fused_supports(bool contiguous, uint32_t width, uint32_t kept_rows) {
    return width == 128 && contiguous && kept_rows > 0;
}

int rows_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_rows_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_rows_status, &zero, sizeof(int));
    return v;
}

size_t attend_rows_workspace_bytes(uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads, uint32_t width) {
    if (rows == 0 || heads == 0 || kv_heads == 0) return 0;
    RowsPlan s = plan_rows(rows, keys, heads, kv_heads);
    if (s.chunks <= 1) return 0;
    return (size_t)rows * heads * s.chunks * (width + 2) * sizeof(float);
}

int attend_rows(const void *q, const void *k, const void *v, void *out, const uint32_t *slots,
                const uint32_t *positions, const KeptDev &kept, bool contiguous, uint32_t rows, uint32_t keys,
                uint32_t heads, uint32_t kv_heads, uint32_t width, uint32_t back, float scale, void *workspace,
                size_t workspace_bytes, cudaStream_t stream, uint32_t ahead, const uint32_t *lens, uint32_t kept_rows,
                const RowsFused *fused) {
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
    // The TMA-fed kernel: width 128, 32 aligned positions = 32 consecutive kept rows, and a known
    // row count to bound the tensor maps with.
    const bool tma = width == 128 && contiguous && kept_rows > 0 &&
                     (uint64_t)rows * (heads / s.g) * s.chunks < 0xFFFFFFFFull;
    if (fused) {
        TS_REQUIRE(tma && ahead == 0 && lens == nullptr && back == 0xFFFFFFFFu,
                   "attend_rows (fused front): needs head width 128, a dense or >= 32-row paged layout with a known "
                   "row count, and the causal mask");
        TS_REQUIRE(fused->qkv && fused->inv_freq, "attend_rows (fused front): qkv or inv_freq is NULL");
        p.qkv = (const uint16_t *)fused->qkv;
        p.q_norm = fused->q_norm;
        p.k_norm = fused->k_norm;
        p.inv_freq = fused->inv_freq;
        p.eps = fused->eps;
        p.early_keys = fused->early_keys ? 1 : 0;
        p.k_out = (uint16_t *)const_cast<void *>(k);
        p.v_out = (uint16_t *)const_cast<void *>(v);
    }
    if (tma) {
        CUtensorMap map_k, map_v;
        const uint64_t cols = (uint64_t)kv_heads * width;
        // The warp-MMA variants: four heads per key always (the scalar kernel is instruction-bound there); one or
        // two heads per key for short items (a chunk of at most 256 keys), where what counts is that every item
        // of the launch is resident at once.  Long items of one or two heads stay on the scalar kernel, which
        // keeps more tiles in flight per SM and reaches 0.98 of the copy rate.
        const bool tensor = rows_mma_enabled() && (s.g == 4 || s.chunk <= 256);
        int rc = tensor ? make_tensor_map_2d(&map_k, k, kept_rows, cols, cols, 32, 64)
                        : make_tensor_map_2d_plain(&map_k, k, kept_rows, cols, cols, 32, 128);
        if (rc != TS_OK) return rc;
        rc = tensor ? make_tensor_map_2d(&map_v, v, kept_rows, cols, cols, 32, 64)
                    : make_tensor_map_2d_plain(&map_v, v, kept_rows, cols, cols, 32, 128);
        if (rc != TS_OK) return rc;
        const uint32_t items = rows * (heads / s.g) * s.chunks;
        rc = tensor     ? (s.g == 4   ? launch_rows_mma<4, 4>(map_k, map_v, p, items, stream)
                           : s.g == 2 ? launch_rows_mma<2, 3>(map_k, map_v, p, items, stream)
                                      : launch_rows_mma<1, 3>(map_k, map_v, p, items, stream))
             : s.g == 4 ? launch_rows_tma<4>(map_k, map_v, p, items, stream)
             : s.g == 2 ? launch_rows_tma<2>(map_k, map_v, p, items, stream)
                        : launch_rows_tma<1>(map_k, map_v, p, items, stream);
        if (rc != TS_OK) return rc;
        e = cudaSuccess;
    } else if (width == 128) {
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
    } else if (width == 32) {   // narrow heads: the reference's own attention cases run 16 wide
        e = s.g == 4 ? launch_rows<32, 4>(p, grid, stream)
            : s.g == 2 ? launch_rows<32, 2>(p, grid, stream)
                       : launch_rows<32, 1>(p, grid, stream);
    } else if (width == 16) {
        e = s.g == 4 ? launch_rows<16, 4>(p, grid, stream)
            : s.g == 2 ? launch_rows<16, 2>(p, grid, stream)
                       : launch_rows<16, 1>(p, grid, stream);
    } else {
        return fail(TS_ERR_BAD_INPUT, "attend_rows: width %u is not 16, 32, 64, 128 or 256", width);
    }
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of attend_rows failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    if (s.chunks > 1) {
        if (width == 128) e = launch(attend_rows_merge_kernel<128>, dim3(rows, heads), dim3(128), 0, stream, pdl_enabled(), p);
        else if (width == 256) e = launch(attend_rows_merge_kernel<256>, dim3(rows, heads), dim3(256), 0, stream, pdl_enabled(), p);
        else if (width == 64) e = launch(attend_rows_merge_kernel<64>, dim3(rows, heads), dim3(64), 0, stream, pdl_enabled(), p);
        else if (width == 32) e = launch(attend_rows_merge_kernel<32>, dim3(rows, heads), dim3(32), 0, stream, pdl_enabled(), p);
        else e = launch(attend_rows_merge_kernel<16>, dim3(rows, heads), dim3(16), 0, stream, pdl_enabled(), p);
        if (e != cudaSuccess)
            return fail(TS_ERR_CUDA, "launch of attend_rows_merge failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                        cudaGetErrorString(e));
    }
    return TS_OK;
}

}  // namespace ts
