// The layer stack of a decode step as ONE persistent kernel: clusters of eight blocks, one block per SM, stay
// resident for the whole step.
//
// A decode step at batch 64 is a chain of five dependent stages per layer (q,k,v -> attention -> o ->
// gate/up -> down), each worth 1-2 microseconds of HBM time.  As separate launches each link of the chain
// pays a launch prologue (barrier set-up, TMEM allocation, tensor-map fetch) and the first-byte latency of its
// weights: 9-12 microseconds a link.  Here the links are phases of one kernel:
//
//   * a producer warp streams the block's weight tiles of ALL phases and layers, in schedule order, through a
//     shared-memory ring by TMA, a few tiles in flight at a time.  Weights depend on nothing, so the stream
//     never stops at a phase boundary: while a block waits at a barrier or attends, the tiles of its next
//     products are already landing;
//   * a cluster owns whole 128-row weight tiles; its eight blocks split k.  A control thread issues the
//     tcgen05 MMAs of the block's k slice (weight rows on the TMEM lanes, the batch on the columns) and runs
//     the device-wide barrier that separates phases: one release-add and an acquire-poll on a counter;
//   * four worker warps reduce the eight partial accumulators through distributed shared memory (block r of
//     the cluster ends up with batch columns 8 r .. 8 r + 7, added in rank order) and apply the stage chain on
//     the way out: 1/rms and bf16 for q,k,v; residual add, the next norm's scaled copy and sums of squares
//     for o and down; SwiGLU for gate/up.  No partial sum touches global memory.  The same warps do the
//     embedding gather and the decode attention (a warp per (row, kv head): per-head norm, rotation, append,
//     warp-MMA flash attention over 32-key tiles it fetches for itself).
//
// Phases of layer l (a device-wide barrier after each):
//   QKV   qkv = bf16((xs . Wqkv^T) / rms)              (xs = bf16(residual * ln1 gain))
//   ATTN  per-head norm, rotation, append of k,v; attention over the kept rows -> attn (bf16)
//   O     x += attn . Wo^T; xs = bf16(x * ln2 gain); sums of squares per 128 columns
//   GU    act = bf16(silu(g / rms) * (u / rms)), [g; u] = xs . [Wgate; Wup]^T
//   DOWN  x += act . Wdown^T; xs = bf16(x * next ln1 gain); sums of squares
// Every sum runs in a fixed order (k blocks inside a slice in the MMA, slices in rank order): a re-run gives
// the same bits.  Every wait is bounded (two seconds); a block that gives up raises a device-wide flag,
// every role of every block leaves, waits for its own copies in flight, TMEM is freed and the host reads
// TS_ERR_TIMEOUT from the status word (the reference bounds its device spins the same way:
// engine/rules/device/include/tessera/status.h:9-39, grid.h:22-42).  The only unbounded primitive is the
// hardware cluster barrier at entry and exit, which every path reaches.
//
// Stands in for the per-layer step list of engine/models/src/decoder.rs:281-389 at decode sizes (<= 64 rows,
// one row per slot, head width 128), i.e. for the `lanes`/`thin` matmul rules
// (engine/rules/linear/src/lanes.rs:20-65) and `attend_rows`/`flash_rows`
// (engine/rules/attention/src/attend.rs:124-167, flash.rs:505-580) with their fused stage chains
// (engine/plan/lower/src/sites/matmul.rs:148-176).
#include <cstdlib>
#include <vector>

#include "head_prep.cuh"
#include "ts_common.cuh"
#include "ts_kernels.cuh"
#include "ts_ptx.cuh"

namespace ts {
namespace {

using namespace ptx;

constexpr uint32_t kCluster = 8;               // blocks of a cluster: the k slices of a weight tile
constexpr uint32_t kRing = 5;                  // weight stages
constexpr uint32_t kAhead = 10;                // weight tiles asked of L2 ahead of the ring (most of a layer for a block)
constexpr uint32_t kTile = 128 * 64 * 2;       // one stage: 128 weight rows x 64 k
constexpr uint32_t kXkb = 64 * 64 * 2;         // one k block of the batch operand: 64 rows x 64 k
constexpr uint32_t kMaxKb = 8;                 // most k blocks a block's k slice may hold
constexpr uint32_t kWorkers = 4;
constexpr uint32_t kThreads = (2 + kWorkers) * 32;
constexpr uint32_t kKvStages = 2;              // per worker warp
constexpr uint32_t kKvStage = 2 * 32 * 128 * 2;  // a 32-key K tile and its V tile
constexpr uint32_t kBatch = 64;                // batch columns of the MMA
constexpr uint32_t kOwn = kBatch / kCluster;   // batch columns a block owns after the cluster reduce
constexpr uint32_t kXfer = 128 * kOwn * 4;     // bytes one block sends another per tile: 128 rows x 8 columns f32
constexpr uint32_t kPrepHeads = 6;             // up to 4 query heads + k + v per item
constexpr uint32_t kAccStages = 2;
constexpr uint32_t kMaxItems = 2;              // attention items a worker warp may own in one phase

// The union region: x slice + receive + send buffers in the linear phases, the workers' K,V tile stages in the
// attention phase.
struct Smem {
    static constexpr uint32_t ring = 0;
    static constexpr uint32_t uni = ring + kRing * kTile;
    static constexpr uint32_t x = uni;                                   // kMaxKb k blocks
    static constexpr uint32_t recv = x + kMaxKb * kXkb;                  // [kCluster][128][kOwn] f32, by source rank
    static constexpr uint32_t send = recv + kCluster * kXfer;            // same shape, by destination rank
    static constexpr uint32_t uni_bytes = kMaxKb * kXkb + 2 * kCluster * kXfer;
    static_assert(uni_bytes == kWorkers * kKvStages * kKvStage, "the two uses of the union region have the same size");
    static constexpr uint32_t prep = uni + uni_bytes;                    // bf16 [kWorkers][kPrepHeads][128]
    static constexpr uint32_t red = prep + kWorkers * kPrepHeads * 256;  // f32 [kWorkers][kOwn] + inv_s [kOwn]
    // What the control thread needs to feed a worker's key tiles: per item the kept rows of its 32-key blocks, the
    // number of blocks and the column of its kv head (written once per step by the worker that owns the item).
    static constexpr uint32_t ytab = red + (kWorkers + 1) * kOwn * 4;    // u32 [kWorkers][kMaxItems][32]
    static constexpr uint32_t item_info = ytab + kWorkers * kMaxItems * 32 * 4;  // u32 [kWorkers][kMaxItems][2]: blocks, column
    static constexpr uint32_t bars = item_info + kWorkers * kMaxItems * 2 * 4;
    static constexpr uint32_t n_bars = 2 * kRing + 1 + 2 * kAccStages + 2 + 2 * kWorkers * kKvStages + 5;
    static constexpr uint32_t misc = bars + ((n_bars * 8 + 63) / 64) * 64;   // tmem slot, abort flag
    static constexpr uint32_t bytes = misc + 64 + 1024;                  // slack for the 1024-byte alignment
};
static_assert(Smem::bytes <= 227 * 1024, "shared memory budget");

enum { LIN_QKV = 0, LIN_O = 1, LIN_GU = 2, LIN_DOWN = 3 };
enum { EPI_QKV = 0, EPI_RESIDUAL = 1, EPI_GATED = 2 };

struct LinPhase {
    uint32_t n;         // weight rows
    uint32_t kb_total;  // k / 64
    uint32_t tiles;     // 128-row tiles (gated: 64 gate rows + their 64 up rows)
    uint32_t cum;       // tiles of the layer's earlier phases (deals tiles round robin over the clusters)
    uint32_t gated;
    uint32_t x_map;     // which activation map feeds it
    uint32_t epilogue;
};

struct LayerDev {
    const float *ln1, *ln2, *q_norm, *k_norm;
    uint16_t *k_rows, *v_rows;
};

struct StepParams {
    // Every tensor map rides in the kernel's parameters, where a copy need not fetch its map from global memory;
    // one map covers all layers of a weight (the layers' copies lie back to back).
    CUtensorMap x_maps[3];     // xs, attn, act
    CUtensorMap w_maps[4];     // q|k|v, o, gate|up, down: [layers * n, k]
    CUtensorMap kv_maps[2];    // kept K and V rows: [layers * kept_rows, kv_heads * 128]
    uint32_t kept_rows;
    const LayerDev *layers;
    LinPhase lin[4];
    uint32_t n_layers, clusters, blocks, rows, hidden, qw, ffn, heads, kv_heads, qkv_n, tiles_per_layer;
    uint32_t ss_parts;         // hidden / 128
    uint32_t max_blk;          // 32-key blocks up to the furthest position of the launch
    float *x;                  // residual rows f32 [rows, hidden]
    uint16_t *xs, *attn, *act, *qkv;
    float *ss;                 // [rows, ss_parts]
    const uint16_t *embed;
    const uint32_t *tokens, *slots, *positions;
    KeptDev kept;
    const float *inv_freq;
    float eps, scale;
    uint32_t *sync;            // [0] barrier counter (zeroed before the launch), [1] device-wide abort flag
    int *status;
    uint64_t wait_ns;          // bound of every wait
};

// Debug builds only (-DTS_DEBUG_STAMPS): %globaltimer stamps of four blocks per phase boundary, the reference's
// TS_MARK idea (engine/plan/run/src/marks.cuh).  Compiled out of the shipped library.
#ifdef TS_DEBUG_STAMPS
__device__ unsigned long long g_step_stamps[4][2048];
#define STEP_STAMP(phase, k)                                                                   \
    do {                                                                                       \
        const uint32_t c__ = blockIdx.x, i__ = (phase) * 12 + (k);                              \
        const int s__ = c__ == 0 ? 0 : c__ == 1 ? 1 : c__ == gridDim.x / 2 ? 2 : c__ == gridDim.x - 1 ? 3 : -1; \
        if (s__ >= 0 && i__ < 2048) {                                                          \
            unsigned long long t__;                                                            \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                            \
            g_step_stamps[s__][i__] = t__;                                                     \
        }                                                                                      \
    } while (0)
#else
#define STEP_STAMP(phase, k) do { } while (0)
#endif

// ---- bounded waits ---------------------------------------------------------------------------------------

struct Bounds {
    volatile uint32_t *abort_s;  // this block
    uint32_t *abort_g;           // every block
    uint64_t wait_ns;
};

__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void give_up(const Bounds &b) {
    *b.abort_s = 1;
    atomicExch(b.abort_g, 1u);
}

// (Not inlined, like the other rarely-run or once-a-phase pieces below: the kernel's code has to stay small enough
// for the instruction cache, or every phase of every layer begins by fetching its instructions again.)
__device__ __noinline__ bool wait_bar_impl(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_s, uint32_t *abort_g, uint64_t wait_ns) {
    const Bounds b = {abort_s, abort_g, wait_ns};
    uint64_t start = 0;
    for (uint32_t i = 0;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*b.abort_s) return false;
            const uint64_t now = now_ns();
            if (start == 0) start = now;
            else if (now - start > b.wait_ns) break;
        }
    }
    give_up(b);
    return false;
}

// After an abort: a copy this thread issued may still be in flight; wait for it (bounded) so that nothing
// lands in shared memory after the block has left.
__device__ __noinline__ void drain_bar(uint64_t *bar, uint32_t parity, uint64_t wait_ns) {
    const uint64_t start = now_ns();
    for (uint32_t i = 0;; i++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 63u) == 63u && now_ns() - start > wait_ns) return;
    }
}

// Arguments of the out-of-line pieces travel as scalars: a struct or array handed to a real call by reference
// lives on the thread's stack, and with nearly all of the SM's L1 given to shared memory a stack access is an L2
// round trip.
__device__ __forceinline__ bool wait_bar(uint64_t *bar, uint32_t parity, const Bounds &b) {
    return wait_bar_impl(bar, parity, b.abort_s, b.abort_g, b.wait_ns);
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Device-wide barrier, one thread per block.  Everything this block wrote (observed by this thread through
// the workers' arrivals) is released to the other blocks; what they wrote is acquired, for the async proxy
// (TMA) too.
__device__ __noinline__ bool grid_sync_impl(uint32_t *counter, uint32_t target, volatile uint32_t *abort_s, uint32_t *abort_g, uint64_t wait_ns) {
    const Bounds b = {abort_s, abort_g, wait_ns};
    __threadfence();
    fence_proxy_async_all();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
    uint64_t start = 0;
    for (uint32_t i = 0;; i++) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= target) break;
        if ((i & 31u) == 31u) {
            uint32_t a;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(a) : "l"(b.abort_g) : "memory");
            if (a || *b.abort_s) {
                *b.abort_s = 1;
                return false;
            }
            const uint64_t now = now_ns();
            if (start == 0) start = now;
            else if (now - start > b.wait_ns) {
                give_up(b);
                return false;
            }
        }
    }
    fence_proxy_async_all();
    return true;
}

__device__ __forceinline__ bool grid_sync(uint32_t *counter, uint32_t target, const Bounds &b) {
    return grid_sync_impl(counter, target, b.abort_s, b.abort_g, b.wait_ns);
}

// ---- small helpers -----------------------------------------------------------------------------------------

// Asks L2 for the box a later tma_load_2d with the same map and coordinates will copy.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y)
                 : "memory");
}

// The k blocks of rank `r`'s slice.
__device__ __forceinline__ void k_slice(const LinPhase &P, uint32_t r, uint32_t &kb0, uint32_t &kb1) {
    kb0 = (uint32_t)(((uint64_t)r * P.kb_total) / kCluster);
    kb1 = (uint32_t)(((uint64_t)(r + 1) * P.kb_total) / kCluster);
}

// First tile of phase `ph` of layer `l` that cluster `cid` owns; its tiles are that one and every `clusters`-th
// after it.  Tiles are dealt round robin over the clusters, carrying on across phases and layers, so that phases
// with fewer tiles than clusters (o, down) land on different clusters.
__device__ __forceinline__ uint32_t first_tile(const StepParams &p, uint32_t l, uint32_t ph, uint32_t cid) {
    const uint32_t rot = (l * p.tiles_per_layer + p.lin[ph].cum) % p.clusters;  // a few thousand tiles at most: 32 bits do
    return (cid + p.clusters - rot) % p.clusters;
}

// Word offset of 4-column group `half` (0, 1) of row `row` in a [128][8] f32 exchange block; the groups of rows
// 4-7 of every eight swap places, which keeps a quarter warp's 16-byte accesses on distinct banks.
__device__ __forceinline__ uint32_t xfer_at(uint32_t row, uint32_t half) { return row * kOwn + ((half ^ ((row >> 2) & 1)) << 2); }

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
// d += a * b with rows 8-15 of a zero: their accumulators (z0, z1) stay zero.
__device__ __forceinline__ void mma_16816(float &d0, float &d1, float &z0, float &z1, uint32_t a0, uint32_t a2, uint32_t b0,
                                          uint32_t b1) {
    const uint32_t zero = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d0), "+f"(d1), "+f"(z0), "+f"(z1)
                 : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}
// byte offset of 16-byte piece `c16` (of 16) of row `row` in a 32 x 128 tile held as two swizzled 64-column halves
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t c16) {
    return (c16 >> 3) * 4096 + row * 128 + (((c16 & 7) ^ (row & 7)) << 4);
}

// ---- worker phases -------------------------------------------------------------------------------------------

// Embedding rows: x = f32(row), xs = bf16(row * gain), sums of squares per 128 columns.
__device__ __noinline__ void gather_phase(const StepParams &p, const float *gain, uint32_t wid, uint32_t lane) {
    const uint32_t nch = p.ss_parts, units = p.rows * nch;
    for (uint32_t u = wid; u < units; u += kWorkers * p.blocks) {
        const uint32_t m = u / nch, col = (u % nch) * 128 + lane * 4;
        const uint32_t tok = p.tokens[m];
        const uint2 e = __ldg(reinterpret_cast<const uint2 *>(p.embed + (size_t)tok * p.hidden + col));
        const float4 a = make_float4(bf16_lo(e.x), bf16_hi(e.x), bf16_lo(e.y), bf16_hi(e.y));
        *reinterpret_cast<float4 *>(p.x + (size_t)m * p.hidden + col) = a;
        const float4 g = __ldg(reinterpret_cast<const float4 *>(gain + col));
        *reinterpret_cast<uint2 *>(p.xs + (size_t)m * p.hidden + col) =
            make_uint2(pack_bf16(a.x * g.x, a.y * g.y), pack_bf16(a.z * g.z, a.w * g.w));
        float ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, a.w * a.w)));
        ss = warp_sum(ss);
        if (lane == 0) p.ss[(size_t)m * nch + u % nch] = ss;
    }
}

// What an attention item needs that does not change from layer to layer: where the row sits, the rotation of its
// position (lane l owns the pairs j = 2 l, 2 l + 1 of a head: elements j and j + 64) and the kept rows of the
// slot's first 32 key blocks (lane b holds block b's).  A warp computes it once per step for its first item.
struct ItemCtx {
    uint32_t row, kvh, slot, pos, y_lane;
    float cs[2], sn[2];
};

__device__ __forceinline__ ItemCtx make_item(const StepParams &p, uint32_t item, uint32_t lane) {
    ItemCtx c;
    c.row = item / p.kv_heads;
    c.kvh = item % p.kv_heads;
    c.slot = p.slots[c.row];
    c.pos = p.positions[c.row];
#pragma unroll
    for (int e = 0; e < 2; e++) sincosf((float)c.pos * p.inv_freq[lane * 2 + e], &c.sn[e], &c.cs[e]);
    c.y_lane = lane * 32 <= c.pos ? kept_row(p.kept, c.slot, lane * 32) : 0;
    return c;
}

// Per-head RMS norm (gains g: elements j and j + 64 of the lane's two pairs; none when `normed` is false) and the
// half-pair rotation of one 128-wide head held as bf16 in shared memory, in place: the arithmetic of
// norm_rope_head (head_prep.cuh) with the angles' sines and cosines computed once per step instead of per head.
__device__ __forceinline__ void norm_rotate(uint16_t *h, const float (&g)[4], bool normed, const ItemCtx &c, float eps,
                                            uint32_t lane) {
    const uint32_t va = *reinterpret_cast<const uint32_t *>(h + lane * 2), vb = *reinterpret_cast<const uint32_t *>(h + 64 + lane * 2);
    float a[2] = {bf16_lo(va), bf16_hi(va)}, b[2] = {bf16_lo(vb), bf16_hi(vb)};
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        ss = fmaf(a[e], a[e], ss);
        ss = fmaf(b[e], b[e], ss);
    }
    if (normed) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
        for (int e = 0; e < 2; e++) {
            a[e] = a[e] * (inv * g[e]);
            b[e] = b[e] * (inv * g[2 + e]);
        }
    }
    uint16_t lo[2], hi[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
        lo[e] = bf16_bits(a[e] * c.cs[e] - b[e] * c.sn[e]);
        hi[e] = bf16_bits(a[e] * c.sn[e] + b[e] * c.cs[e]);
    }
    __syncwarp();
    *reinterpret_cast<uint32_t *>(h + lane * 2) = (uint32_t)lo[0] | ((uint32_t)lo[1] << 16);
    *reinterpret_cast<uint32_t *>(h + 64 + lane * 2) = (uint32_t)hi[0] | ((uint32_t)hi[1] << 16);
}

// One (row, kv head) of the decode attention on one warp: q, k, v of the row from the projection (bf16), per-head
// norm and rotation, append, then flash attention over the slot's kept rows in 32-key tiles.  The block's control
// thread copies the tiles into the warp's two stages by TMA and keeps them full across items (kv_full: a tile has
// landed; kv_empty: the warp has read it), so the first tiles of the warp's next item are already on their way
// while it finishes this one.  The products run on warp MMAs with the GRP query heads in rows 0..GRP-1 of the
// 16-row operand.
template <int GRP>
__device__ __forceinline__ bool attend_item(const StepParams &p, const LayerDev &L, const ItemCtx &c, const float (&qg)[4],
                                            const float (&kg)[4], bool normed, uint32_t lane, uint8_t *stages,
                                            uint16_t *prep, uint64_t *kv_full, uint64_t *kv_empty, uint32_t &kv_parity,
                                            uint32_t &kv_count, const Bounds &bd, uint32_t stamp_phase) {
    constexpr int WIDTH = 128;
    (void)stamp_phase;
    const uint32_t row = c.row, kvh = c.kvh, slot = c.slot, pos = c.pos;
    const uint32_t head0 = kvh * GRP;
    const uint32_t hi = pos + 1, n_blk = (hi + 31) / 32;
    // ---- q heads, k, v of this row: four values a lane and head, asked for before the key tiles ----
    uint2 raw[GRP + 2];
#pragma unroll
    for (uint32_t u = 0; u < (uint32_t)GRP + 2; u++) {
        const bool is_q = u < (uint32_t)GRP, is_v = u == (uint32_t)GRP + 1;
        const uint32_t h = is_q ? head0 + u : (is_v ? p.heads + p.kv_heads + kvh : p.heads + kvh);
        raw[u] = __ldcg(reinterpret_cast<const uint2 *>(p.qkv + (size_t)row * p.qkv_n + h * WIDTH + lane * 4));
    }
    if (lane == 0 && stamp_phase) STEP_STAMP(stamp_phase, 4);
#pragma unroll
    for (uint32_t u = 0; u < (uint32_t)GRP + 2; u++) *reinterpret_cast<uint2 *>(prep + u * WIDTH + lane * 4) = raw[u];
    __syncwarp();
#pragma unroll 1
    for (uint32_t u = 0; u < (uint32_t)GRP + 1; u++) norm_rotate(prep + u * WIDTH, u < (uint32_t)GRP ? qg : kg, normed, c, p.eps, lane);
    __syncwarp();
    {   // the new kept row, for later steps: lanes 0-15 the key, 16-31 the value
        const size_t at = ((size_t)kept_row(p.kept, slot, pos) * p.kv_heads + kvh) * WIDTH;
        const uint16_t *from = prep + (GRP + (lane >> 4)) * WIDTH;
        reinterpret_cast<uint4 *>((lane < 16 ? L.k_rows : L.v_rows) + at)[lane & 15] = reinterpret_cast<const uint4 *>(from)[lane & 15];
    }
    bool ok = true;
    const uint32_t hrow = lane >> 2, quad = lane & 3;
    uint32_t qa[8][2];
#pragma unroll
    for (int t = 0; t < 8; t++) {
        qa[t][0] = qa[t][1] = 0;
        if (hrow < (uint32_t)GRP) {
            const uint32_t d = 16 * t + 2 * quad;
            qa[t][0] = *reinterpret_cast<const uint32_t *>(prep + hrow * WIDTH + d);
            qa[t][1] = *reinterpret_cast<const uint32_t *>(prep + hrow * WIDTH + d + 8);
        }
    }
    float m_row = -INFINITY, l_row = 0.0f;
    float oacc[16][2];
    float z0 = 0.0f, z1 = 0.0f;
#pragma unroll
    for (int n = 0; n < 16; n++) oacc[n][0] = oacc[n][1] = 0.0f;

    for (uint32_t blk = 0; blk < n_blk; blk++, kv_count++) {
        const uint32_t s = kv_count % kKvStages;  // the stages carry on from item to item, as the feeder's do
        ok = wait_bar(&kv_full[s], (kv_parity >> s) & 1, bd);
        if (!ok) break;
        kv_parity ^= 1u << s;
        if (lane == 0 && stamp_phase && blk == 0) STEP_STAMP(stamp_phase, 7);
        uint8_t *tile_k = stages + s * kKvStage;
        uint8_t *tile_v = tile_k + kKvStage / 2;
        const uint32_t base = blk * 32;
        if (pos - base < 32) {
            // the row's own key and value come from the prepared copies: the tile was read before or while
            // they were appended
            const uint32_t c16 = lane & 15, r = pos - base;
            const uint8_t *from = reinterpret_cast<const uint8_t *>(prep) + (GRP + (lane >> 4)) * 256 + c16 * 16;
            uint8_t *to = (lane < 16 ? tile_k : tile_v) + swz(r, c16);
            *reinterpret_cast<uint4 *>(to) = *reinterpret_cast<const uint4 *>(from);
            __syncwarp();
        }
        if (base + 32 > hi) {
            // rows past the position may hold anything (a page's unwritten tail): zero their V so that a zero
            // probability cannot meet a NaN
            for (uint32_t j = hi - base; j < 32; j++)
                *reinterpret_cast<uint2 *>(tile_v + (lane >> 4) * 4096 + j * 128 + (lane & 15) * 8) = make_uint2(0, 0);
            __syncwarp();
        }
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
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const uint32_t key = base + 8 * j + 2 * quad + e;
                sc[j][e] = key < hi ? sc[j][e] * p.scale : -INFINITY;
                mx = fmaxf(mx, sc[j][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        const float m_new = fmaxf(m_row, mx);  // finite: the tile holds a visible key
        const float alpha = __expf(m_row - m_new);
        m_row = m_new;
        uint32_t pa[2][2];
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
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int n2 = 0; n2 < 8; n2++) {
                uint32_t b[4];
                ldsm_x4_trans(v_addr + swz(16 * u + (mtx & 1) * 8 + mrow, 2 * n2 + (mtx >> 1)), b);
                mma_16816(oacc[2 * n2][0], oacc[2 * n2][1], z0, z1, pa[u][0], pa[u][1], b[0], b[1]);
                mma_16816(oacc[2 * n2 + 1][0], oacc[2 * n2 + 1][1], z0, z1, pa[u][0], pa[u][1], b[2], b[3]);
            }
        // the stage is free once every lane has read it; the patches above were generic-proxy writes
        fence_async_shared();
        __syncwarp();
        if (lane == 0) mbar_arrive(&kv_empty[s]);
    }
    if (ok) {
        l_row += __shfl_xor_sync(0xFFFFFFFFu, l_row, 1);
        l_row += __shfl_xor_sync(0xFFFFFFFFu, l_row, 2);
        if (hrow < (uint32_t)GRP) {
            const float r = l_row > 0.0f ? 1.0f / l_row : 0.0f;
            uint16_t *out = p.attn + ((size_t)row * p.heads + head0 + hrow) * WIDTH + 2 * quad;
#pragma unroll
            for (int n = 0; n < 16; n++)
                *reinterpret_cast<uint32_t *>(out + 8 * n) = pack_bf16(oacc[n][0] * r, oacc[n][1] * r);
        }
    }
    __syncwarp();
    return ok;
}

// ---- the kernel ------------------------------------------------------------------------------------------------

template <int GRP>
__global__ void __launch_bounds__(kThreads, 1) decode_layers_kernel(const __grid_constant__ StepParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, cta = blockIdx.x, G = p.blocks;
    const uint32_t rank = cluster_ctarank(), cid = cta / kCluster;
    unsigned char *ring = smem + Smem::ring;
    unsigned char *xbuf = smem + Smem::x;
    float *recv = reinterpret_cast<float *>(smem + Smem::recv);
    float *send = reinterpret_cast<float *>(smem + Smem::send);
    float *red = reinterpret_cast<float *>(smem + Smem::red);  // [kWorkers][kOwn]
    float *inv_s = red + kWorkers * kOwn;                      // [kOwn]: 1/rms of the batch rows this block owns
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Smem::bars);
    uint64_t *ring_full = bars, *ring_empty = bars + kRing;
    uint64_t *x_full = ring_empty + kRing;
    uint64_t *acc_full = x_full + 1, *acc_empty = acc_full + kAccStages;
    uint64_t *workers_done = acc_empty + kAccStages, *phase_go = workers_done + 1;
    uint64_t *kv_full = phase_go + 1;  // [kWorkers][kKvStages]: a key tile has landed
    uint64_t *kv_empty = kv_full + kWorkers * kKvStages;   // [kWorkers][kKvStages]: its warp has read it
    uint64_t *send_full = kv_empty + kWorkers * kKvStages;  // the four warps have staged their partials
    uint64_t *recv_full = send_full + 1;                   // the eight blocks' partials of my columns have landed
    uint64_t *peers_free = recv_full + 1;                  // every block of the cluster has read its receive buffer
    uint64_t *red_full = peers_free + 1;                   // the four warps' sums of squares are in shared memory
    uint64_t *inv_full = red_full + 1;                     // inv_s is written
    uint32_t *ytab = reinterpret_cast<uint32_t *>(smem + Smem::ytab);            // [kWorkers][kMaxItems][32]
    uint32_t *item_info = reinterpret_cast<uint32_t *>(smem + Smem::item_info);  // [kWorkers][kMaxItems][2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + Smem::misc);
    volatile uint32_t *abort_s = tmem_slot + 1;
    const Bounds bd = {abort_s, p.sync + 1, p.wait_ns};

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kRing; s++) {
            mbar_init(&ring_full[s], 1);
            mbar_init(&ring_empty[s], 1);
        }
        mbar_init(x_full, 1);
        for (uint32_t s = 0; s < kAccStages; s++) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kWorkers);
        }
        mbar_init(workers_done, kWorkers);
        mbar_init(phase_go, 1);
        for (uint32_t s = 0; s < kWorkers * kKvStages; s++) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        mbar_init(send_full, kWorkers);
        mbar_init(recv_full, 1);
        mbar_init(peers_free, kCluster * kWorkers);
        mbar_init(red_full, kWorkers);
        mbar_init(inv_full, 1);
        *abort_s = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kAccStages * kBatch);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    cluster_sync();  // every block's barriers exist before a peer signals them
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t L = p.n_layers, C = p.clusters;

    if (warp == 0) {
        // ---- weight producer: the block's k slice of its cluster's tiles, every phase and layer, in order.  A
        // second cursor runs kAhead tiles in front and asks L2 for them, so that a stage freed at the end of a
        // phase refills from L2 in about a microsecond instead of from HBM in three or four.
        if (lane == 0) {
            struct Cursor {
                uint32_t l, ph, tile, kb, kb1;
            };
            auto settle = [&](Cursor &c) {  // moves to the next (layer, phase) that has a tile for this cluster
                while (c.l < L) {
                    const LinPhase &P = p.lin[c.ph];
                    if (c.tile == 0xFFFFFFFFu) {
                        c.tile = first_tile(p, c.l, c.ph, cid);
                        uint32_t kb0;
                        k_slice(P, rank, kb0, c.kb1);
                        c.kb = kb0;
                    }
                    if (c.tile < P.tiles) return true;
                    c.tile = 0xFFFFFFFFu;
                    if (++c.ph == 4) {
                        c.ph = 0;
                        c.l++;
                    }
                }
                return false;
            };
            auto advance = [&](Cursor &c) {
                const LinPhase &P = p.lin[c.ph];
                if (++c.kb < c.kb1) return;
                uint32_t kb0;
                k_slice(P, rank, kb0, c.kb1);
                c.kb = kb0;
                c.tile += C;
                if (c.tile >= P.tiles) {
                    c.tile = 0xFFFFFFFFu;
                    if (++c.ph == 4) {
                        c.ph = 0;
                        c.l++;
                    }
                }
            };
            auto coords = [&](const Cursor &c, int32_t &y0, int32_t &y1) {
                const LinPhase &P = p.lin[c.ph];
                const uint32_t base = c.l * P.n;  // the layer's rows in the all-layers tensor
                y0 = (int32_t)(base + (P.gated ? c.tile * 64 : c.tile * 128));
                y1 = (int32_t)(base + P.n / 2 + c.tile * 64);
            };
            Cursor cur = {0, 0, 0xFFFFFFFFu, 0, 0}, ahead = cur;
            uint32_t it = 0, asked = 0;
            bool ok = true;
#pragma unroll 1
            while (ok && settle(cur)) {
                // keep the look-ahead cursor kAhead tiles in front
#pragma unroll 1
                while (asked < it + kAhead && settle(ahead)) {
                    const CUtensorMap *ma = &p.w_maps[ahead.ph];
                    int32_t y0, y1;
                    coords(ahead, y0, y1);
                    tma_prefetch_2d(ma, (int32_t)(ahead.kb * 64), y0);
                    if (p.lin[ahead.ph].gated) tma_prefetch_2d(ma, (int32_t)(ahead.kb * 64), y1);
                    advance(ahead);
                    asked++;
                }
                const uint32_t s = it % kRing;
                ok = wait_bar(&ring_empty[s], ((it / kRing) & 1) ^ 1, bd);
                if (!ok) break;
                const CUtensorMap *mw = &p.w_maps[cur.ph];
                unsigned char *dst = ring + s * kTile;
                int32_t y0, y1;
                coords(cur, y0, y1);
                mbar_expect_tx(&ring_full[s], kTile);
                const int32_t kx = (int32_t)(cur.kb * 64);
                if (p.lin[cur.ph].gated) {
                    tma_load_2d(dst, mw, &ring_full[s], kx, y0);
                    tma_load_2d(dst + kTile / 2, mw, &ring_full[s], kx, y1);
                } else {
                    tma_load_2d(dst, mw, &ring_full[s], kx, y0);
                }
                advance(cur);
                it++;
            }
            if (!ok) {  // copies still in flight must land before the block leaves
                for (uint32_t back = 0; back < kRing && back < it; back++) {
                    const uint32_t j = it - 1 - back;
                    drain_bar(&ring_full[j % kRing], (j / kRing) & 1, p.wait_ns);
                }
            }
        }
    } else if (warp == 1) {
        // ---- control: the MMAs of the block's k slice and the barrier between phases ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(128, kBatch);
            uint32_t it = 0, xi = 0, ai = 0, bar = 0;
            bool ok = true, x_pending = false;
            auto sync_phase = [&]() {
                if (ok) ok = wait_bar(workers_done, bar & 1, bd);
                STEP_STAMP(bar, 1);
                if (ok) ok = grid_sync(p.sync, (bar + 1) * G, bd);
                STEP_STAMP(bar, 0);
                if (ok) mbar_arrive(phase_go);
                bar++;
            };
            auto linear = [&](uint32_t l, uint32_t ph) {
                const LinPhase &P = p.lin[ph];
                uint32_t tile = first_tile(p, l, ph, cid);
                if (tile >= P.tiles || !ok) return;
                uint32_t kb0, kb1;
                k_slice(P, rank, kb0, kb1);
                const uint32_t nkb = kb1 - kb0;
                // the block's k slice of the batch rows: the same for every tile of the phase
                mbar_expect_tx(x_full, nkb * kXkb);
                for (uint32_t j = 0; j < nkb; j++) tma_load_2d(xbuf + j * kXkb, &p.x_maps[P.x_map], x_full, (int32_t)((kb0 + j) * 64), 0);
                x_pending = true;
                ok = wait_bar(x_full, xi & 1, bd);
                if (!ok) return;
                x_pending = false;
                xi++;
                STEP_STAMP(bar, 4);
                for (; tile < P.tiles; tile += C) {
                    const uint32_t as = ai % kAccStages;
                    ok = wait_bar(&acc_empty[as], ((ai / kAccStages) & 1) ^ 1, bd);
                    if (!ok) return;
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + as * kBatch;
                    for (uint32_t kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t s = it % kRing;
                        ok = wait_bar(&ring_full[s], (it / kRing) & 1, bd);
                        if (!ok) return;
                        if (kb == 0) STEP_STAMP(bar, 8);
                        if (kb + 1 == nkb) STEP_STAMP(bar, 9);
                        tc_fence_after_sync();
                        const uint64_t da = umma_desc_k_sw128(smem_addr(ring + s * kTile));
                        const uint64_t db = umma_desc_k_sw128(smem_addr(xbuf + kb * kXkb));
#pragma unroll
                        for (uint32_t k16 = 0; k16 < 4; k16++) umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                        umma_commit(&ring_empty[s]);
                    }
                    umma_commit(&acc_full[as]);
                    STEP_STAMP(bar, 5);
                    ai++;
                }
            };
            // The attention phase: keeps every worker's two key-tile stages full, across the worker's items (the
            // table of kept rows per item was left in shared memory by the workers before their first arrival).  A
            // stage is refilled as soon as its warp has released it; the four workers are visited in turn and
            // none is waited for.
            uint32_t fed0 = 0, fed1 = 0, fed2 = 0, fed3 = 0;  // tiles fed to each worker so far, all layers
            auto feed = [&](uint32_t l) {
                const uint32_t y_base = l * p.kept_rows;  // the layer's rows in the all-layers tensor
                uint32_t at0 = 0, at1 = 0, at2 = 0, at3 = 0;  // per worker: item * 32 + block
                uint32_t left = 0;
                for (uint32_t i = 0; i < kWorkers * kMaxItems; i++) left += item_info[i * 2];
                uint64_t start = 0;
                uint32_t idle = 0;
                auto one = [&](uint32_t w, uint32_t &at, uint32_t &fed) __attribute__((always_inline)) {
                    uint32_t item = at >> 5, blk = at & 31;
                    if (item >= kMaxItems) return;
                    uint32_t n_blk = item_info[(w * kMaxItems + item) * 2];
                    if (blk >= n_blk) {  // this item is fed: on to the worker's next one, if it has one
                        item++;
                        blk = 0;
                        at = item << 5;
                        if (item >= kMaxItems) return;
                        n_blk = item_info[(w * kMaxItems + item) * 2];
                        if (n_blk == 0) {
                            at = kMaxItems << 5;
                            return;
                        }
                    }
                    const uint32_t s = fed % kKvStages, use = fed / kKvStages;
                    if (use > 0 && !mbar_try_wait(&kv_empty[w * kKvStages + s], (use - 1) & 1)) return;
                    const int32_t x = (int32_t)item_info[(w * kMaxItems + item) * 2 + 1];
                    const int32_t y = (int32_t)(y_base + ytab[(w * kMaxItems + item) * 32 + blk]);
                    unsigned char *dst = smem + Smem::uni + (w * kKvStages + s) * kKvStage;
                    uint64_t *full = &kv_full[w * kKvStages + s];
                    mbar_expect_tx(full, kKvStage);
                    tma_load_2d(dst, &p.kv_maps[0], full, x, y);
                    tma_load_2d(dst + 4096, &p.kv_maps[0], full, x + 64, y);
                    tma_load_2d(dst + kKvStage / 2, &p.kv_maps[1], full, x, y);
                    tma_load_2d(dst + kKvStage / 2 + 4096, &p.kv_maps[1], full, x + 64, y);
                    fed++;
                    at++;
                    left--;
                    idle = 0;
                };
                while (left && ok) {
                    one(0, at0, fed0);
                    one(1, at1, fed1);
                    one(2, at2, fed2);
                    one(3, at3, fed3);
                    if ((++idle & 63u) == 63u) {
                        if (*abort_s) ok = false;
                        const uint64_t now = now_ns();
                        if (start == 0) start = now;
                        else if (now - start > p.wait_ns) {
                            give_up(bd);
                            ok = false;
                        }
                    }
                }
            };
            sync_phase();  // the gather
            // One copy of the phase code, walked by a loop that is not unrolled: the kernel's instructions must stay
            // within the instruction cache, or every phase of every layer starts by fetching its code again.
#pragma unroll 1
            for (uint32_t step = 0; step < 5 * L; step++) {
                const uint32_t l = step / 5, k5 = step % 5;  // q,k,v | attention | o | gate,up | down
                if (k5 != 1) linear(l, k5 == 0 ? LIN_QKV : k5 - 1);
                else if (ok) feed(l);
                if (step + 1 < 5 * L) sync_phase();  // nothing follows the last one
            }
            if (x_pending) drain_bar(x_full, xi & 1, p.wait_ns);
            if (!ok) {  // key tiles this thread asked for must land before the block leaves
                auto drain = [&](uint32_t w, uint32_t fed) {
                    for (uint32_t back = 0; back < kKvStages && back < fed; back++) {
                        const uint32_t j = fed - 1 - back;
                        drain_bar(&kv_full[w * kKvStages + j % kKvStages], (j / kKvStages) & 1, p.wait_ns);
                    }
                };
                drain(0, fed0);
                drain(1, fed1);
                drain(2, fed2);
                drain(3, fed3);
            }
        }
    } else {
        // ---- workers ----
        const uint32_t w = warp - 2, q = warp & 3;
        const uint32_t wid = w * G + cta;  // spreads consecutive units over the blocks first
        const uint32_t row = q * 32 + lane;  // the tile row (TMEM lane) this thread owns
        uint32_t ai = 0, bar = 0, unit = 0, n_inv = 0, n_red = 0;
        uint32_t kv_parity = 0, kv_count = 0;  // bit s: parity of the next completion of stage s; tiles read so far
        bool ok = true, sent = false;
        uint8_t *stages = smem + Smem::uni + w * kKvStages * kKvStage;
        uint16_t *prep = reinterpret_cast<uint16_t *>(smem + Smem::prep) + w * kPrepHeads * 128;
        uint64_t *my_kv_full = kv_full + w * kKvStages, *my_kv_empty = kv_empty + w * kKvStages;
        const uint32_t recv_addr = smem_addr(recv), send_addr = smem_addr(send);
        const uint32_t recv_full_addr = smem_addr(recv_full), peers_free_addr = smem_addr(peers_free);
        auto begin = [&]() {  // the barrier that ended the previous phase
            if (ok && bar > 0) ok = wait_bar(phase_go, (bar - 1) & 1, bd);
            if (w == 0 && lane == 0) STEP_STAMP(bar, 2);
        };
        auto done = [&]() {
            if (w == 0 && lane == 0) STEP_STAMP(bar, 3);
            fence_proxy_async_all();  // what this warp stored is read by other blocks' TMA loads
            __syncwarp();
            if (lane == 0) mbar_arrive(workers_done);
            bar++;
        };
        // The cluster's tiles of a linear phase: partial accumulators out of TMEM, exchanged through distributed
        // shared memory, added in rank order, finished with the phase's stage chain and stored.
        auto finish = [&](uint32_t l, uint32_t ph, const float *gain) {
            const LinPhase &P = p.lin[ph];
            uint32_t tile = first_tile(p, l, ph, cid);
            if (tile >= P.tiles) return;
            const uint32_t m0 = rank * kOwn;  // the batch rows this block owns
            if (P.epilogue != EPI_RESIDUAL) {
                // 1/rms of the owned batch rows, from the sums of squares the last residual-feeding phase left
                if (w == 0 && ok) {
                    const uint32_t i = lane >> 2, sub = lane & 3;
                    float ss = 0.0f;
                    for (uint32_t part = sub; part < p.ss_parts; part += 4) ss += __ldcg(p.ss + (size_t)(m0 + i) * p.ss_parts + part);
                    ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 1);
                    ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 2);
                    if (sub == 0) inv_s[i] = 1.0f / sqrtf(ss / (float)p.hidden + p.eps);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(inv_full);
                }
                if (ok) ok = wait_bar(inv_full, n_inv & 1, bd);
                n_inv++;
            }
            for (; tile < P.tiles && ok; tile += C, unit++) {
                const uint32_t as = ai % kAccStages;
                ok = wait_bar(&acc_full[as], (ai / kAccStages) & 1, bd);
                if (!ok) break;
                ai++;
                if (w == 0 && lane == 0) STEP_STAMP(bar, 6);
                tc_fence_after_sync();
                float v[kBatch];
#pragma unroll
                for (uint32_t c0 = 0; c0 < kBatch; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + as * kBatch + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) v[c0 + i] = __uint_as_float(r[i]);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[as]);
                // What the stage chain reads besides the sum, asked for now: it arrives under the exchange.
                const bool upper = P.gated && row >= 64;  // an up row: its gate row's thread finishes the pair
                const uint32_t n = P.gated ? tile * 64 + (row & 63) : tile * 128 + row;
                float res[kOwn];
                float g = 0.0f;
                if (P.epilogue == EPI_RESIDUAL) {
#pragma unroll
                    for (uint32_t i = 0; i < kOwn; i++) res[i] = m0 + i < p.rows ? __ldcg(p.x + (size_t)(m0 + i) * P.n + n) : 0.0f;
                    if (gain) g = __ldg(gain + n);
                }
                // The previous tile's exchange must be over in every block of the cluster: its buffers are reused.
                if (sent) {
                    ok = wait_bar(peers_free, (unit - 1) & 1, bd);
                    if (!ok) break;
                }
                // Stage the partial by destination block, then one thread sends each block its 128 x 8 share.
#pragma unroll
                for (uint32_t d = 0; d < kCluster; d++) {
                    float *to = send + d * (kXfer / 4);
                    *reinterpret_cast<float4 *>(to + xfer_at(row, 0)) = make_float4(v[8 * d], v[8 * d + 1], v[8 * d + 2], v[8 * d + 3]);
                    *reinterpret_cast<float4 *>(to + xfer_at(row, 1)) = make_float4(v[8 * d + 4], v[8 * d + 5], v[8 * d + 6], v[8 * d + 7]);
                }
                fence_async_shared();  // the copy engine reads what these threads wrote
                __syncwarp();
                if (lane == 0) mbar_arrive(send_full);
                if (w == 0 && lane == 0) {
                    mbar_expect_tx(recv_full, kCluster * kXfer);
                    if (wait_bar(send_full, unit & 1, bd)) {
                        for (uint32_t d = 0; d < kCluster; d++)
                            bulk_copy_to_peer(map_to_rank(recv_addr + rank * kXfer, d), send_addr + d * kXfer, kXfer,
                                              map_to_rank(recv_full_addr, d));
                    }
                }
                sent = true;
                if (w == 0 && lane == 0) STEP_STAMP(bar, 7);
                ok = wait_bar(recv_full, unit & 1, bd);
                if (!ok) break;
                if (w == 0 && lane == 0) STEP_STAMP(bar, 10);
                // Add the eight partials of the owned columns in rank order.
                float a[kOwn], b[kOwn];
                auto sum_row = [&](uint32_t r, float (&out)[kOwn]) {
                    const float4 lo = *reinterpret_cast<const float4 *>(recv + xfer_at(r, 0));
                    const float4 hi = *reinterpret_cast<const float4 *>(recv + xfer_at(r, 1));
                    out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
                    out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
#pragma unroll
                    for (uint32_t s = 1; s < kCluster; s++) {
                        const float4 l2 = *reinterpret_cast<const float4 *>(recv + s * (kXfer / 4) + xfer_at(r, 0));
                        const float4 h2 = *reinterpret_cast<const float4 *>(recv + s * (kXfer / 4) + xfer_at(r, 1));
                        out[0] += l2.x; out[1] += l2.y; out[2] += l2.z; out[3] += l2.w;
                        out[4] += h2.x; out[5] += h2.y; out[6] += h2.z; out[7] += h2.w;
                    }
                };
                sum_row(row, a);
                if (P.gated && !upper) sum_row(row + 64, b);
                // this block has read its receive buffer: tell every block of the cluster (itself included)
                __syncwarp();
                if (lane == 0) {
                    for (uint32_t d = 0; d < kCluster; d++) mbar_arrive_remote(map_to_rank(peers_free_addr, d));
                }
                if (P.epilogue == EPI_QKV) {
#pragma unroll
                    for (uint32_t i = 0; i < kOwn; i++)
                        if (m0 + i < p.rows) p.qkv[(size_t)(m0 + i) * P.n + n] = bf16_bits(a[i] * inv_s[i]);
                } else if (P.epilogue == EPI_GATED) {
                    if (!upper) {
#pragma unroll
                        for (uint32_t i = 0; i < kOwn; i++)
                            if (m0 + i < p.rows) p.act[(size_t)(m0 + i) * (P.n / 2) + n] = bf16_bits(silu(a[i] * inv_s[i]) * (b[i] * inv_s[i]));
                    }
                } else {
#pragma unroll
                    for (uint32_t i = 0; i < kOwn; i++) {
                        const float r = a[i] + res[i];
                        const size_t at = (size_t)(m0 + i) * P.n + n;
                        if (m0 + i < p.rows) {
                            p.x[at] = r;
                            if (gain) p.xs[at] = bf16_bits(r * g);
                        }
                        if (gain) {  // sums of squares of the finished rows over this tile's 128 columns
                            const float t = warp_sum(r * r);
                            if (lane == 0) red[w * kOwn + i] = t;
                        }
                    }
                    if (gain) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(red_full);
                        ok = wait_bar(red_full, n_red & 1, bd);
                        n_red++;
                        if (!ok) break;
                        if (w == 0 && lane < kOwn && m0 + lane < p.rows)
                            p.ss[(size_t)(m0 + lane) * p.ss_parts + tile] = ((red[lane] + red[kOwn + lane]) + red[2 * kOwn + lane]) + red[3 * kOwn + lane];
                        __syncwarp();
                        // (the next tile's partial sums are written only after the next exchange, which every warp joins)
                    }
                }
            }
        };
        const uint32_t items = p.rows * p.kv_heads;
        ItemCtx first_item = {};
        if (wid < items) first_item = make_item(p, wid, lane);
        {
            // Pin the values here: without this the compiler is free to recompute them where they are first used,
            // which is inside every layer's attention phase (two dependent loads, a table look-up and two sincosf).
            asm volatile("" : "+r"(first_item.row), "+r"(first_item.kvh), "+r"(first_item.slot), "+r"(first_item.pos), "+r"(first_item.y_lane));
            asm volatile("" : "+f"(first_item.cs[0]), "+f"(first_item.cs[1]), "+f"(first_item.sn[0]), "+f"(first_item.sn[1]));
        }
        float qg[4] = {1.0f, 1.0f, 1.0f, 1.0f}, kg[4] = {1.0f, 1.0f, 1.0f, 1.0f};
        // The control thread's table: this warp's items (the same in every layer), the kept rows of their key blocks.
        for (uint32_t i = 0; i < kMaxItems; i++) {
            const uint32_t item = wid + i * kWorkers * G;
            uint32_t n_blk = 0, col = 0;
            if (item < items) {
                const ItemCtx c = i == 0 ? first_item : make_item(p, item, lane);
                ytab[(w * kMaxItems + i) * 32 + lane] = c.y_lane;
                n_blk = c.pos / 32 + 1;
                col = c.kvh * 128;
            }
            if (lane == 0) {
                item_info[(w * kMaxItems + i) * 2] = n_blk;
                item_info[(w * kMaxItems + i) * 2 + 1] = col;
            }
        }
        // phase 0: the gather
        gather_phase(p, p.layers[0].ln1, wid, lane);
        done();
        bool normed = false;
#pragma unroll 1
        for (uint32_t step = 0; step < 5 * L; step++) {
            const uint32_t l = step / 5, k5 = step % 5;  // q,k,v | attention | o | gate,up | down
            const LayerDev &Ly = p.layers[l];
            begin();
            if (k5 == 0) {
                normed = Ly.q_norm != nullptr;
                if (ok && normed && wid < items) {  // the per-head gains of this layer, long before the attention phase wants them
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        qg[e] = __ldg(Ly.q_norm + lane * 2 + e);
                        qg[2 + e] = __ldg(Ly.q_norm + 64 + lane * 2 + e);
                        kg[e] = __ldg(Ly.k_norm + lane * 2 + e);
                        kg[2 + e] = __ldg(Ly.k_norm + 64 + lane * 2 + e);
                    }
                }
            }
            if (k5 == 1) {
                if (ok) {
#pragma unroll 1
                    for (uint32_t item = wid; item < items && ok; item += kWorkers * G) {
                        ItemCtx c = first_item;
                        if (item != wid) c = make_item(p, item, lane);
                        ok = attend_item<GRP>(p, Ly, c, qg, kg, normed, lane, stages, prep, my_kv_full, my_kv_empty, kv_parity,
                                              kv_count, bd, w == 0 ? bar : 0);
                        if (w == 0 && lane == 0 && item == wid) STEP_STAMP(bar, 5);
                    }
                }
            } else {
                const float *gain = k5 == 2 ? Ly.ln2 : (k5 == 4 && l + 1 < L) ? p.layers[l + 1].ln1 : nullptr;
                finish(l, k5 == 0 ? LIN_QKV : k5 - 1, gain);
            }
            done();
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();  // no block leaves while a peer may still write into it or signal it
    if (threadIdx.x == 0 && *abort_s) atomicExch(p.status, TS_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kAccStages * kBatch);
    }
}

// A block that waits on a barrier nothing arrives at: exercises the give-up path of the waits above
// (bounded wait -> device-wide flag -> status word) without touching anything else.
__global__ void wait_runs_out_kernel(uint32_t *sync, int *status, uint64_t wait_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_s;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_s = 0;
        fence_barrier_init();
        const Bounds bd = {&abort_s, sync + 1, wait_ns};
        const bool ok = wait_bar(&bar, 0, bd);
        if (!ok) atomicExch(status, TS_ERR_TIMEOUT);
    }
}

__device__ int g_step_status = 0;

bool step_kernel_enabled() {
    static const bool off = [] {
        const char *v = getenv("TS_STEP_KERNEL");
        return v && v[0] == '0';
    }();
    return !off;
}

template <typename Kernel>
cudaError_t cluster_config(Kernel kernel, uint32_t blocks, cudaStream_t stream, cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem::bytes);
    if (e != cudaSuccess) return e;
    *cfg = {};
    cfg->gridDim = dim3(blocks);
    cfg->blockDim = dim3(kThreads);
    cfg->dynamicSmemBytes = Smem::bytes;
    cfg->stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
    return cudaSuccess;
}

// Clusters of eight blocks of this kernel that the device holds at once.
template <typename Kernel>
int resident_clusters(Kernel kernel, uint32_t *out) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    TS_CUDA(cluster_config(kernel, (uint32_t)sm_count() / kCluster * kCluster, nullptr, &cfg, attr));
    int n = 0;
    TS_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    *out = n > 0 ? (uint32_t)n : 0;
    return TS_OK;
}

}  // namespace

#ifdef TS_DEBUG_STAMPS
extern "C" __attribute__((visibility("default"))) int ts_debug_step_stamps(unsigned long long *out) {
    return cudaMemcpyFromSymbol(out, g_step_stamps, sizeof(unsigned long long) * 4 * 2048) == cudaSuccess ? 0 : 6;
}
#endif

int step_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_step_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_step_status, &zero, sizeof(int));
    return v;
}

// ---- host: the plan -------------------------------------------------------------------------------------------

struct StepKernel {
    StepParams p = {};
    uint32_t group = 0;
    void *layers = nullptr, *sync = nullptr;
    std::vector<void *> owned;
};

bool step_kernel_supports(const StepKernelShape &s) {
    if (!step_kernel_enabled()) return false;
    if (s.head_dim != 128 || s.kv_heads == 0 || s.heads % s.kv_heads != 0) return false;
    const uint32_t group = s.heads / s.kv_heads;
    if (group != 1 && group != 2 && group != 4) return false;
    const uint32_t qw = s.heads * 128;
    // every product's k splits eight ways into slices of one to kMaxKb 64-wide blocks; tiles are whole
    for (uint32_t k : {s.hidden, qw, s.ffn})
        if (k % 64 != 0 || k / 64 < kCluster || ceil_div(k / 64, kCluster) > kMaxKb) return false;
    if (s.hidden % 128 != 0 || s.ffn % 64 != 0 || s.hidden > 8192) return false;
    if (!(s.page == 0 || s.page >= 32)) return false;  // 32 aligned positions must be 32 consecutive kept rows
    return s.kept_rows > 0;
}

static void plan_linear(LinPhase *P, uint32_t n, uint32_t k, bool gated, uint32_t x_map, uint32_t epilogue) {
    P->n = n;
    P->kb_total = k / 64;
    P->gated = gated ? 1 : 0;
    P->tiles = gated ? (n / 2) / 64 : n / 128;
    P->x_map = x_map;
    P->epilogue = epilogue;
}

int step_kernel_create(const StepKernelShape &s, const StepKernelBuffers &b, StepKernel **out) {
    StepKernel *k = new StepKernel();
    auto bail = [&](int rc) {
        step_kernel_destroy(k);
        return rc;
    };
    StepParams &p = k->p;
    const uint32_t H = s.hidden, QW = s.heads * 128, KW = s.kv_heads * 128, F = s.ffn, L = s.layers;
    k->group = s.heads / s.kv_heads;
    int rc;
    uint32_t clusters = 0;
    rc = k->group == 1 ? resident_clusters(decode_layers_kernel<1>, &clusters)
         : k->group == 2 ? resident_clusters(decode_layers_kernel<2>, &clusters)
                         : resident_clusters(decode_layers_kernel<4>, &clusters);
    if (rc != TS_OK) return bail(rc);
    if (clusters == 0) return bail(fail(TS_ERR_CUDA, "step kernel: no cluster of %u blocks fits this device", kCluster));
    if (kBatch * s.kv_heads > kMaxItems * kWorkers * clusters * kCluster)
        return bail(fail(TS_ERR_BAD_INPUT, "step kernel: %u kv heads over %u resident blocks: a worker warp would own more than %u "
                                           "attention items", s.kv_heads, clusters * kCluster, kMaxItems));
    p.clusters = clusters;
    p.blocks = clusters * kCluster;
    p.n_layers = L;
    p.hidden = H;
    p.qw = QW;
    p.ffn = F;
    p.heads = s.heads;
    p.kv_heads = s.kv_heads;
    p.qkv_n = QW + 2 * KW;
    p.ss_parts = H / 128;
    plan_linear(&p.lin[LIN_QKV], p.qkv_n, H, false, 0, EPI_QKV);
    plan_linear(&p.lin[LIN_O], H, QW, false, 1, EPI_RESIDUAL);
    plan_linear(&p.lin[LIN_GU], 2 * F, H, true, 0, EPI_GATED);
    plan_linear(&p.lin[LIN_DOWN], H, F, false, 2, EPI_RESIDUAL);
    uint32_t cum = 0;
    for (int i = 0; i < 4; i++) {
        p.lin[i].cum = cum;
        cum += p.lin[i].tiles;
    }
    p.tiles_per_layer = cum;
    auto dev = [&](void **ptr, size_t bytes) -> int {
        TS_CUDA(cudaMalloc(ptr, bytes));
        k->owned.push_back(*ptr);
        TS_CUDA(cudaMemset(*ptr, 0, bytes));
        return TS_OK;
    };
    if ((rc = dev(&k->sync, 256)) != TS_OK) return bail(rc);
    p.sync = (uint32_t *)k->sync;
    // One tensor map per weight over all layers (the layers' copies must lie back to back, which the runner's slabs
    // guarantee), one each for the kept K and V rows, three for the activations.
    std::vector<LayerDev> layers(L);
    for (uint32_t l = 0; l < L; l++) {
        const StepKernelLayer &Y = b.layers[l], &Z = b.layers[0];
        const bool packed = (const uint16_t *)Y.wqkv == (const uint16_t *)Z.wqkv + (size_t)l * p.qkv_n * H &&
                            (const uint16_t *)Y.wo == (const uint16_t *)Z.wo + (size_t)l * H * QW &&
                            (const uint16_t *)Y.wgu == (const uint16_t *)Z.wgu + (size_t)l * 2 * F * H &&
                            (const uint16_t *)Y.wdown == (const uint16_t *)Z.wdown + (size_t)l * H * F &&
                            (const uint16_t *)Y.k_rows == (const uint16_t *)Z.k_rows + (size_t)l * s.kept_rows * KW &&
                            (const uint16_t *)Y.v_rows == (const uint16_t *)Z.v_rows + (size_t)l * s.kept_rows * KW;
        if (!packed) return bail(fail(TS_ERR_BAD_INPUT, "step kernel: layer %u's weights do not follow layer 0's back to back", l));
        layers[l] = {Y.ln1, Y.ln2, s.qk_norm ? Y.q_norm : nullptr, s.qk_norm ? Y.k_norm : nullptr, (uint16_t *)Y.k_rows,
                     (uint16_t *)Y.v_rows};
    }
    const StepKernelLayer &Z = b.layers[0];
    if ((rc = make_tensor_map_2d(&p.w_maps[LIN_QKV], Z.wqkv, (uint64_t)L * p.qkv_n, H, H, 128, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.w_maps[LIN_O], Z.wo, (uint64_t)L * H, QW, QW, 128, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.w_maps[LIN_GU], Z.wgu, (uint64_t)L * 2 * F, H, H, 64, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.w_maps[LIN_DOWN], Z.wdown, (uint64_t)L * H, F, F, 128, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.kv_maps[0], Z.k_rows, (uint64_t)L * s.kept_rows, KW, KW, 32, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.kv_maps[1], Z.v_rows, (uint64_t)L * s.kept_rows, KW, KW, 32, 64)) != TS_OK) return bail(rc);
    p.kept_rows = s.kept_rows;
    if ((rc = make_tensor_map_2d(&p.x_maps[0], b.xs, s.max_rows, H, H, kBatch, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.x_maps[1], b.attn, s.max_rows, QW, QW, kBatch, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.x_maps[2], b.act, s.max_rows, F, F, kBatch, 64)) != TS_OK) return bail(rc);
    if ((rc = dev(&k->layers, layers.size() * sizeof(LayerDev))) != TS_OK) return bail(rc);
    cudaError_t e = cudaMemcpy(k->layers, layers.data(), layers.size() * sizeof(LayerDev), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return bail(fail(TS_ERR_CUDA, "step kernel: uploads failed: %s", cudaGetErrorString(e)));
    p.layers = (const LayerDev *)k->layers;
    p.x = b.x;
    p.xs = (uint16_t *)b.xs;
    p.attn = (uint16_t *)b.attn;
    p.act = (uint16_t *)b.act;
    p.qkv = (uint16_t *)b.qkv;
    float *ss = nullptr;
    if ((rc = dev((void **)&ss, (size_t)kBatch * p.ss_parts * sizeof(float))) != TS_OK) return bail(rc);
    p.ss = ss;
    p.embed = (const uint16_t *)b.embed;
    p.tokens = b.tokens;
    p.slots = b.slots;
    p.positions = b.positions;
    p.inv_freq = b.inv_freq;
    p.eps = s.eps;
    p.scale = 1.0f / sqrtf(128.0f);
    p.wait_ns = 2000000000ull;
    int *status = nullptr;
    e = cudaGetSymbolAddress((void **)&status, g_step_status);
    if (e != cudaSuccess) return bail(fail(TS_ERR_CUDA, "step kernel: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)));
    p.status = status;
    *out = k;
    return TS_OK;
}

void step_kernel_destroy(StepKernel *k) {
    if (!k) return;
    for (void *q : k->owned) cudaFree(q);
    delete k;
}

uint32_t step_kernel_max_rows() { return kBatch; }

int step_kernel_launch(StepKernel *k, uint32_t rows, uint32_t keys, const KeptDev &kept, cudaStream_t stream) {
    TS_REQUIRE(k && rows >= 1 && rows <= kBatch, "step kernel: %u rows, it takes 1..%u", rows, kBatch);
    TS_REQUIRE(keys <= 32 * 32, "step kernel: %u keys, the feeder's table holds 32 blocks of 32 keys per item", keys);
    StepParams p = k->p;
    p.rows = rows;
    p.kept = kept;
    p.max_blk = ceil_div(keys ? keys : 1, 32);
    auto go = [&](auto kernel) -> int {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        TS_CUDA(cluster_config(kernel, p.blocks, stream, &cfg, attr));
        TS_CUDA(cudaMemsetAsync(p.sync, 0, 8, stream));
        cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
        if (e != cudaSuccess)
            return fail(TS_ERR_CUDA, "launch of decode_layers failed: %s (%d) %s", cudaGetErrorName(e), (int)e, cudaGetErrorString(e));
        return TS_OK;
    };
    switch (k->group) {
    case 1: return go(decode_layers_kernel<1>);
    case 2: return go(decode_layers_kernel<2>);
    default: return go(decode_layers_kernel<4>);
    }
}

int wait_runs_out(uint64_t wait_ns, cudaStream_t stream) {
    uint32_t *sync = nullptr;
    TS_CUDA(cudaMalloc((void **)&sync, 256));
    cudaError_t e = cudaMemsetAsync(sync, 0, 8, stream);
    int *status = nullptr;
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void **)&status, g_step_status);
    if (e == cudaSuccess) {
        wait_runs_out_kernel<<<1, 32, 0, stream>>>(sync, status, wait_ns);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    cudaFree(sync);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "wait_runs_out failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
