// The layer stack of a decode step as ONE persistent kernel: every SM holds one block for the whole step.
//
// A decode step at batch 64 is a chain of five dependent products per layer (q,k,v -> attention -> o ->
// gate/up -> down), each worth 1-2 microseconds of HBM time.  As separate launches each link of the chain
// pays a launch prologue (barrier set-up, TMEM allocation, tensor-map fetch), the first-byte latency of its
// weights and a cluster reduce: 9-12 microseconds a link.  Here the links are phases of one kernel:
//
//   * a producer warp streams the block's weight tiles of ALL phases and layers, in schedule order, through a
//     shared-memory ring by TMA.  Weights depend on nothing, so the stream never stops at a phase boundary:
//     while a block waits at a barrier or attends, the tiles of its next products are already landing;
//   * a control thread issues the tcgen05 MMAs of the block's (weight tile, k slice) units (weight rows on
//     the TMEM lanes, the batch on the columns) and runs the device-wide barrier that separates phases:
//     one release-add and an acquire-poll on a counter, bounded in time;
//   * four worker warps drain the accumulators into f32 partial sums in global memory (they stay in L2) and
//     do everything else: the embedding gather, decode attention (a warp per (row, kv head): per-head norm,
//     rotation, append, warp-MMA flash attention over TMA-fed 32-key tiles) and the fixed-order reduction of
//     the k-slice partials with the residual add, the next norm's scaled copy and sums of squares, or SwiGLU.
//
// Phases of layer l (a device-wide barrier after each):
//   QKV   partials of xs . Wqkv^T                      (xs = bf16(residual * ln1 gain), 1/rms applied later)
//   ATTN  q,k,v = bf16(sum of partials * 1/rms); norm, rotate, append k,v; attend  -> attn (bf16)
//   O     partials of attn . Wo^T
//   R1    x += sum of partials; xs = bf16(x * ln2 gain); sums of squares per 128 columns
//   GU    partials of xs . [Wgate; Wup]^T
//   R2    act = bf16(silu(g / rms) * (u / rms))
//   DOWN  partials of act . Wdown^T
//   R3    x += sum of partials; xs = bf16(x * next ln1 gain); sums of squares
// Every sum runs in a fixed order (k blocks inside a slice in the MMA, slices in ascending order): a re-run
// gives the same bits.  Every wait is bounded (two seconds); a block that gives up raises a device-wide flag,
// every role of every block leaves, waits for its own copies in flight, TMEM is freed and the host reads
// TS_ERR_TIMEOUT from the status word (the reference bounds its device spins the same way:
// engine/rules/device/include/tessera/status.h:9-39, grid.h:22-42).
//
// Stands in for the per-layer step list of engine/models/src/decoder.rs:281-389 at decode sizes (<= 64 rows,
// one row per slot, head width 128), i.e. for the `lanes`/`thin` matmul rules
// (engine/rules/linear/src/lanes.rs:20-65) and `attend_rows`/`flash_rows`
// (engine/rules/attention/src/attend.rs:124-167, flash.rs:505-580) with their fused stage chains.
#include <cstdlib>
#include <vector>

#include "head_prep.cuh"
#include "ts_common.cuh"
#include "ts_kernels.cuh"
#include "ts_ptx.cuh"

namespace ts {
namespace {

using namespace ptx;

constexpr uint32_t kRing = 5;                  // weight stages
constexpr uint32_t kInFlight = 2;              // weight tiles the producer keeps in flight
constexpr uint32_t kTile = 128 * 64 * 2;       // one stage: 128 weight rows x 64 k
constexpr uint32_t kXkb = 64 * 64 * 2;         // one k block of the batch operand: 64 rows x 64 k
constexpr uint32_t kWorkers = 4;
constexpr uint32_t kThreads = (2 + kWorkers) * 32;
constexpr uint32_t kKvStages = 2;              // per worker warp
constexpr uint32_t kKvStage = 2 * 32 * 128 * 2;  // a 32-key K tile and its V tile
constexpr uint32_t kUnion = kWorkers * kKvStages * kKvStage;  // x slice (linear phases) / K,V tiles (attention)
constexpr uint32_t kMaxKb = kUnion / kXkb;     // most k blocks a unit's x slice may hold
constexpr uint32_t kPrepHeads = 6;             // up to 4 query heads + k + v per item
constexpr uint32_t kBatch = 64;                // batch columns of the MMA; row stride of the partial buffers
constexpr uint32_t kAccStages = 2;
constexpr uint32_t kWarpStage = kKvStages * kKvStage;  // a worker warp's share of the union region

struct Smem {
    static constexpr uint32_t ring = 0;
    static constexpr uint32_t uni = ring + kRing * kTile;
    static constexpr uint32_t prep = uni + kUnion;                       // bf16 [kWorkers][kPrepHeads][128]
    static constexpr uint32_t bars = prep + kWorkers * kPrepHeads * 256;
    static constexpr uint32_t n_bars = 2 * kRing + 1 + 2 * kAccStages + 2 + kWorkers * kKvStages;
    static constexpr uint32_t misc = bars + ((n_bars * 8 + 63) / 64) * 64;   // tmem slot, abort flag
    static constexpr uint32_t bytes = misc + 64 + 1024;                  // slack for the 1024-byte alignment
};
static_assert(Smem::bytes <= 227 * 1024, "shared memory budget");

enum { LIN_QKV = 0, LIN_O = 1, LIN_GU = 2, LIN_DOWN = 3 };

struct LinPhase {
    uint32_t n;         // weight rows
    uint32_t kb_total;  // k / 64
    uint32_t tiles;     // 128-row tiles (gated: 64 gate rows + their 64 up rows)
    uint32_t splits;    // k slices
    uint32_t units;     // tiles * splits
    uint32_t cum;       // units of the layer's earlier phases (deals units round robin over the blocks)
    uint32_t gated;
    uint32_t x_map;     // which activation map feeds it
    float *part;        // [splits][kBatch][n] f32
};

struct LayerDev {
    const float *ln1, *ln2, *q_norm, *k_norm;
    uint16_t *k_rows, *v_rows;
};

struct StepParams {
    CUtensorMap x_maps[3];     // xs, attn, act: in the parameter space, where a copy need not fetch its map from global memory
    const CUtensorMap *maps;   // [4 L] weights, then [2 L] kept K and V
    const LayerDev *layers;
    LinPhase lin[4];
    uint32_t n_layers, blocks, rows, hidden, qw, ffn, heads, kv_heads, qkv_n, units_per_layer;
    uint32_t ss_parts;         // hidden / 128
    uint32_t vocab;
    uint32_t max_blk;          // 32-key blocks up to the furthest position of the launch
    float *x;                  // residual rows f32 [rows, hidden]
    uint16_t *xs, *attn, *act;
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
        const uint32_t c__ = blockIdx.x, i__ = (phase) * 8 + (k);                              \
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

__device__ __forceinline__ bool wait_bar(uint64_t *bar, uint32_t parity, const Bounds &b) {
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
__device__ __forceinline__ void drain_bar(uint64_t *bar, uint32_t parity, uint64_t wait_ns) {
    const uint64_t start = now_ns();
    for (uint32_t i = 0;; i++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 63u) == 63u && now_ns() - start > wait_ns) return;
    }
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Device-wide barrier, one thread per block.  Everything this block wrote (observed by this thread through
// the workers' arrivals) is released to the other blocks; what they wrote is acquired, for the async proxy
// (TMA) too.
__device__ __forceinline__ bool grid_sync(uint32_t *counter, uint32_t target, const Bounds &b) {
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

// ---- small helpers -----------------------------------------------------------------------------------------

// One thread.  Copies `bytes` (a multiple of 16, both addresses 16-byte aligned) from global to this block's shared
// memory and credits them to `bar`.  The copy reads through L2, so it sees what other blocks released before the
// barrier that preceded it.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// A worker warp's staging area (its share of the union region) and the barrier its copies complete on.
struct Stage {
    uint8_t *mem;       // kWarpStage bytes
    uint64_t *bar;
    uint32_t *parity;   // bit 0: parity of the barrier's next completion
    uint32_t *pending;  // bit 0: copies in flight
};

__device__ __forceinline__ void k_slice(const LinPhase &P, uint32_t split, uint32_t &kb0, uint32_t &kb1) {
    kb0 = (uint32_t)(((uint64_t)split * P.kb_total) / P.splits);
    kb1 = (uint32_t)(((uint64_t)(split + 1) * P.kb_total) / P.splits);
}

// First unit of phase `ph` of layer `l` that block `cta` owns; the block's units are that one and every
// `blocks`-th after it.  Units are dealt round robin over the blocks, carrying on across phases and layers.
__device__ __forceinline__ uint32_t first_unit(const StepParams &p, uint32_t l, uint32_t ph, uint32_t cta) {
    const uint32_t rot = (uint32_t)(((uint64_t)l * p.units_per_layer + p.lin[ph].cum) % p.blocks);
    return (cta + p.blocks - rot) % p.blocks;
}

// 1/rms of residual row `m` from the partial sums of squares the last reduction left (whole warp).
__device__ __forceinline__ float row_inv_rms(const StepParams &p, uint32_t m, uint32_t lane) {
    float ss = 0.0f;
    for (uint32_t i = lane; i < p.ss_parts; i += 32) ss += __ldcg(p.ss + (size_t)m * p.ss_parts + i);
    ss = warp_sum(ss);
    return 1.0f / sqrtf(ss / (float)p.hidden + p.eps);
}

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

// Asks L2 for the kept K and V rows this layer's attention will read (positions below each row's own), a 32-row
// block per lane: issued while the q,k,v product runs, so that the attention phase's tile copies hit L2 instead of
// paying HBM latency with two tiles in flight per warp.  The kept rows of earlier positions depend on nothing in
// this step.
__device__ __forceinline__ void prefetch_kept(const StepParams &p, const LayerDev &L, uint32_t wid, uint32_t lane) {
    const uint32_t units = p.rows * p.max_blk * 2, row_elems = p.kv_heads * 128;
    for (uint32_t u = wid * 32 + lane; u < units; u += kWorkers * p.blocks * 32) {
        const uint32_t t = u >> 1, blk = t % p.max_blk, row = t / p.max_blk;
        const uint32_t pos = p.positions[row];
        if (blk * 32 >= pos) continue;
        const uint32_t n = min(32u, pos - blk * 32);
        const uint16_t *at = ((u & 1) ? L.v_rows : L.k_rows) + (size_t)kept_row(p.kept, p.slots[row], blk * 32) * row_elems;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(at), "r"(n * row_elems * 2) : "memory");
    }
}

// Embedding rows: x = f32(row), xs = bf16(row * gain), sums of squares per 128 columns.
__device__ __forceinline__ void gather_phase(const StepParams &p, const float *gain, uint32_t wid, uint32_t lane) {
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

// x += sum over the k slices (ascending) of a residual-feeding product; xs = bf16(x * gain) and the sums of
// squares for the norm that follows (gain NULL: the last layer, nothing follows inside the kernel).  The slices'
// 128-column rows are staged in shared memory by bulk copies, all in flight at once: one L2 round trip a unit.
__device__ __forceinline__ bool residual_phase(const StepParams &p, const LinPhase &P, const float *gain, uint32_t wid,
                                               uint32_t lane, const Stage &st, const Bounds &bd) {
    const uint32_t nch = p.ss_parts, units = p.rows * nch, H = p.hidden, S = P.splits;
    constexpr uint32_t kMost = kWarpStage / 512 - 1;  // slices a pass can stage beside the residual row
    for (uint32_t u = wid; u < units; u += kWorkers * p.blocks) {
        const uint32_t m = u / nch, col0 = (u % nch) * 128;
        float *xo = p.x + (size_t)m * H + col0;
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t s0 = 0; s0 < S; s0 += kMost) {
            const uint32_t n = min(kMost, S - s0), copies = n + (s0 == 0 ? 1 : 0);
            if (lane == 0) {
                mbar_expect_tx(st.bar, copies * 512);
                *st.pending |= 1u;
            }
            __syncwarp();
            for (uint32_t c = lane; c < copies; c += 32) {
                const float *src = c < n ? P.part + ((size_t)(s0 + c) * kBatch + m) * H + col0 : xo;
                bulk_load(st.mem + c * 512, src, 512, st.bar);
            }
            if (!wait_bar(st.bar, *st.parity & 1, bd)) return false;
            *st.parity ^= 1u;
            *st.pending &= ~1u;
            if (s0 == 0) a = *reinterpret_cast<const float4 *>(st.mem + n * 512 + lane * 16);  // the residual row
            for (uint32_t c = 0; c < n; c++) {
                const float4 t = *reinterpret_cast<const float4 *>(st.mem + c * 512 + lane * 16);
                a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
            }
            __syncwarp();  // every lane has read the stage before the next pass overwrites it
        }
        const uint32_t col = col0 + lane * 4;
        *reinterpret_cast<float4 *>(xo + lane * 4) = a;
        if (gain) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gain + col));
            *reinterpret_cast<uint2 *>(p.xs + (size_t)m * H + col) =
                make_uint2(pack_bf16(a.x * g.x, a.y * g.y), pack_bf16(a.z * g.z, a.w * g.w));
            float ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, a.w * a.w)));
            ss = warp_sum(ss);
            if (lane == 0) p.ss[(size_t)m * nch + u % nch] = ss;
        }
    }
    return true;
}

// act = bf16(silu(g / rms) * (u / rms)), g and u the sums over the k slices of the gate and up halves; a unit is
// 512 columns of one row (or the row's last columns), staged like the residual rows.
__device__ __forceinline__ bool gated_phase(const StepParams &p, const LinPhase &P, uint32_t wid, uint32_t lane,
                                            const Stage &st, const Bounds &bd) {
    const uint32_t F = p.ffn, nch = (F + 511) / 512, units = p.rows * nch, N = P.n, S = P.splits;
    for (uint32_t u = wid; u < units; u += kWorkers * p.blocks) {
        const uint32_t m = u / nch, col0 = (u % nch) * 512;
        const uint32_t width = min(512u, F - col0), row_bytes = width * 4;      // multiples of 256 columns
        const uint32_t most = kWarpStage / (2 * row_bytes);
        float4 g[4], up[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) g[i] = up[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t s0 = 0; s0 < S; s0 += most) {
            const uint32_t n = min(most, S - s0), copies = 2 * n;
            if (lane == 0) {
                mbar_expect_tx(st.bar, copies * row_bytes);
                *st.pending |= 1u;
            }
            __syncwarp();
            for (uint32_t c = lane; c < copies; c += 32) {   // copy 2 j: gate columns of slice s0 + j; 2 j + 1: up columns
                const float *src = P.part + ((size_t)(s0 + (c >> 1)) * kBatch + m) * N + col0 + (c & 1) * F;
                bulk_load(st.mem + c * row_bytes, src, row_bytes, st.bar);
            }
            if (!wait_bar(st.bar, *st.parity & 1, bd)) return false;
            *st.parity ^= 1u;
            *st.pending &= ~1u;
            for (uint32_t c = 0; c < n; c++) {
#pragma unroll
                for (uint32_t i = 0; i < 4; i++)
                    if (i * 128 < width) {
                        const float4 a = *reinterpret_cast<const float4 *>(st.mem + (2 * c) * row_bytes + i * 512 + lane * 16);
                        const float4 b = *reinterpret_cast<const float4 *>(st.mem + (2 * c + 1) * row_bytes + i * 512 + lane * 16);
                        g[i].x += a.x; g[i].y += a.y; g[i].z += a.z; g[i].w += a.w;
                        up[i].x += b.x; up[i].y += b.y; up[i].z += b.z; up[i].w += b.w;
                    }
            }
            __syncwarp();
        }
        const float inv = row_inv_rms(p, m, lane);
#pragma unroll
        for (uint32_t i = 0; i < 4; i++)
            if (i * 128 < width) {
                const float r0 = silu(g[i].x * inv) * (up[i].x * inv), r1 = silu(g[i].y * inv) * (up[i].y * inv);
                const float r2 = silu(g[i].z * inv) * (up[i].z * inv), r3 = silu(g[i].w * inv) * (up[i].w * inv);
                *reinterpret_cast<uint2 *>(p.act + (size_t)m * F + col0 + i * 128 + lane * 4) =
                    make_uint2(pack_bf16(r0, r1), pack_bf16(r2, r3));
            }
    }
    return true;
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

// One (row, kv head) of the decode attention on one warp: q,k,v from the projection's partials, per-head
// norm and rotation (the stand-alone append kernel's code: same bits), append, then flash attention over the
// slot's kept rows in 32-key tiles the warp fetches for itself by TMA, two tiles ahead.  The products run on
// warp MMAs with the GRP query heads in rows 0..GRP-1 of the 16-row operand.
template <int GRP>
__device__ __forceinline__ bool attend_item(const StepParams &p, const LayerDev &L, const CUtensorMap *map_k,
                                            const CUtensorMap *map_v, const ItemCtx &c, const float (&qg)[4],
                                            const float (&kg)[4], bool normed, uint32_t lane, uint8_t *stages,
                                            uint16_t *prep, uint64_t *kv_full, uint32_t &kv_parity,
                                            uint32_t &kv_pending, const Bounds &bd, uint32_t stamp_phase) {
    constexpr int WIDTH = 128;
    (void)stamp_phase;
    const uint32_t row = c.row, kvh = c.kvh, slot = c.slot, pos = c.pos;
    const uint32_t head0 = kvh * GRP;
    const uint32_t hi = pos + 1, n_blk = (hi + 31) / 32;
    const int32_t x = (int32_t)(kvh * WIDTH);
    auto issue = [&](uint32_t blk) {  // whole warp
        const uint32_t s = blk % kKvStages;
        const uint32_t yl = __shfl_sync(0xFFFFFFFFu, c.y_lane, blk & 31);
        const int32_t y = (int32_t)(blk < 32 ? yl : kept_row(p.kept, slot, blk * 32));
        if (lane == 0) {
            uint8_t *dst = stages + s * kKvStage;
            mbar_expect_tx(&kv_full[s], kKvStage);
            tma_load_2d(dst, map_k, &kv_full[s], x, y);
            tma_load_2d(dst + 4096, map_k, &kv_full[s], x + 64, y);
            tma_load_2d(dst + kKvStage / 2, map_v, &kv_full[s], x, y);
            tma_load_2d(dst + kKvStage / 2 + 4096, map_v, &kv_full[s], x + 64, y);
        }
        kv_pending |= 1u << s;
    };
    // the row's sums of squares: asked for before anything is waited on
    float ss_part = 0.0f;
    for (uint32_t i = lane; i < p.ss_parts; i += 32) ss_part += __ldcg(p.ss + (size_t)row * p.ss_parts + i);
    if (lane == 0 && stamp_phase) STEP_STAMP(stamp_phase, 4);
    // ---- q heads, k, v of this row: the projection's partial sums, staged in the second tile stage by bulk
    // copies (all in flight at once), added in slice order, times 1/rms, as bf16 ----
    bool ok = true;
    {
        const LinPhase &P = p.lin[LIN_QKV];
        constexpr uint32_t kHeads = GRP + 2, kMost = 32 / kHeads < kKvStage / (kHeads * 512) ? 32 / kHeads : kKvStage / (kHeads * 512);
        uint8_t *stage = stages + kKvStage;
        uint64_t *bar = &kv_full[1];
        float4 acc[kHeads];
#pragma unroll
        for (uint32_t u = 0; u < kHeads; u++) acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t s0 = 0; s0 < P.splits; s0 += kMost) {
            const uint32_t n = min(kMost, P.splits - s0), copies = kHeads * n;   // <= 32: a lane a copy
            if (lane == 0) {
                mbar_expect_tx(bar, copies * 512);
                kv_pending |= 2u;
            }
            __syncwarp();
            if (lane < copies) {
                const uint32_t u = lane / n, j = lane % n;
                const bool is_q = u < (uint32_t)GRP, is_v = u == (uint32_t)GRP + 1;
                const uint32_t h = is_q ? head0 + u : (is_v ? p.heads + p.kv_heads + kvh : p.heads + kvh);
                bulk_load(stage + lane * 512, P.part + ((size_t)(s0 + j) * kBatch + row) * P.n + h * WIDTH, 512, bar);
            }
            if (s0 == 0) issue(0);  // the first key tile follows the small copies into the copy queue
            ok = wait_bar(bar, (kv_parity >> 1) & 1, bd);
            if (!ok) return false;
            kv_parity ^= 2u;
            kv_pending &= ~2u;
#pragma unroll
            for (uint32_t u = 0; u < kHeads; u++)
                for (uint32_t j = 0; j < n; j++) {
                    const float4 t = *reinterpret_cast<const float4 *>(stage + (u * n + j) * 512 + lane * 16);
                    acc[u].x += t.x; acc[u].y += t.y; acc[u].z += t.z; acc[u].w += t.w;
                }
            __syncwarp();
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss_part) / (float)p.hidden + p.eps);
#pragma unroll
        for (uint32_t u = 0; u < kHeads; u++)
            *reinterpret_cast<uint2 *>(prep + u * WIDTH + lane * 4) =
                make_uint2(pack_bf16(acc[u].x * inv, acc[u].y * inv), pack_bf16(acc[u].z * inv, acc[u].w * inv));
    }
    if (lane == 0 && stamp_phase) STEP_STAMP(stamp_phase, 5);
    if (n_blk > 1) issue(1);  // the staging area is a tile stage again
    __syncwarp();
#pragma unroll
    for (uint32_t u = 0; u < (uint32_t)GRP + 1; u++) norm_rotate(prep + u * WIDTH, u < (uint32_t)GRP ? qg : kg, normed, c, p.eps, lane);
    __syncwarp();
    {   // the new kept row, for later steps: lanes 0-15 the key, 16-31 the value
        const size_t at = ((size_t)kept_row(p.kept, slot, pos) * p.kv_heads + kvh) * WIDTH;
        const uint16_t *from = prep + (GRP + (lane >> 4)) * WIDTH;
        reinterpret_cast<uint4 *>((lane < 16 ? L.k_rows : L.v_rows) + at)[lane & 15] = reinterpret_cast<const uint4 *>(from)[lane & 15];
    }
    if (lane == 0 && stamp_phase) STEP_STAMP(stamp_phase, 6);
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

    for (uint32_t blk = 0; blk < n_blk; blk++) {
        const uint32_t s = blk % kKvStages;
        ok = wait_bar(&kv_full[s], (kv_parity >> s) & 1, bd);
        if (!ok) break;
        kv_parity ^= 1u << s;
        kv_pending &= ~(1u << s);
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
        if (blk + kKvStages < n_blk) issue(blk + kKvStages);
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
    unsigned char *ring = smem + Smem::ring;
    unsigned char *uni = smem + Smem::uni;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Smem::bars);
    uint64_t *ring_full = bars, *ring_empty = bars + kRing;
    uint64_t *x_full = ring_empty + kRing;
    uint64_t *acc_full = x_full + 1, *acc_empty = acc_full + kAccStages;
    uint64_t *workers_done = acc_empty + kAccStages, *phase_go = workers_done + 1;
    uint64_t *kv_full = phase_go + 1;  // [kWorkers][kKvStages]
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
        for (uint32_t s = 0; s < kWorkers * kKvStages; s++) mbar_init(&kv_full[s], 1);
        *abort_s = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kAccStages * kBatch);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t L = p.n_layers;

    if (warp == 0) {
        // ---- weight producer: the block's tiles of every phase and layer, in schedule order ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t l = 0; l < L && ok; l++) {
                for (uint32_t ph = 0; ph < 4 && ok; ph++) {
                    const LinPhase &P = p.lin[ph];
                    const CUtensorMap *mw = p.maps + l * 4 + ph;
                    for (uint32_t u = first_unit(p, l, ph, cta); u < P.units && ok; u += G) {
                        const uint32_t tile = u / P.splits;
                        uint32_t kb0, kb1;
                        k_slice(P, u % P.splits, kb0, kb1);
                        for (uint32_t kb = kb0; kb < kb1; kb++, it++) {
                            const uint32_t s = it % kRing;
                            ok = wait_bar(&ring_empty[s], ((it / kRing) & 1) ^ 1, bd);
                            if (!ok) break;
                            if (it >= kInFlight) {  // pace the stream: a burst of tiles would queue ahead of the small, urgent copies
                                const uint32_t j = it - kInFlight;
                                ok = wait_bar(&ring_full[j % kRing], (j / kRing) & 1, bd);
                                if (!ok) break;
                            }
                            unsigned char *dst = ring + s * kTile;
                            mbar_expect_tx(&ring_full[s], kTile);
                            const int32_t kx = (int32_t)(kb * 64);
                            if (P.gated) {
                                tma_load_2d(dst, mw, &ring_full[s], kx, (int32_t)(tile * 64));
                                tma_load_2d(dst + kTile / 2, mw, &ring_full[s], kx, (int32_t)(P.n / 2 + tile * 64));
                            } else {
                                tma_load_2d(dst, mw, &ring_full[s], kx, (int32_t)(tile * 128));
                            }
                        }
                    }
                }
            }
            if (!ok) {  // copies still in flight must land before the block leaves
                for (uint32_t back = 0; back < kRing && back < it; back++) {
                    const uint32_t j = it - 1 - back;
                    drain_bar(&ring_full[j % kRing], (j / kRing) & 1, p.wait_ns);
                }
            }
        }
    } else if (warp == 1) {
        // ---- control: the MMAs of the block's units and the barrier between phases ----
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
                const CUtensorMap *mx = &p.x_maps[P.x_map];
                bool first = true;
                for (uint32_t u = first_unit(p, l, ph, cta); u < P.units && ok; u += G) {
                    uint32_t kb0, kb1;
                    k_slice(P, u % P.splits, kb0, kb1);
                    const uint32_t nkb = kb1 - kb0;
                    if (!first) {  // the x slice is still being read by the previous unit's MMAs
                        const uint32_t prev = ai - 1;
                        ok = wait_bar(&acc_full[prev % kAccStages], (prev / kAccStages) & 1, bd);
                        if (!ok) break;
                    }
                    first = false;
                    mbar_expect_tx(x_full, nkb * kXkb);
                    for (uint32_t j = 0; j < nkb; j++) tma_load_2d(uni + j * kXkb, mx, x_full, (int32_t)((kb0 + j) * 64), 0);
                    x_pending = true;
                    const uint32_t as = ai % kAccStages;
                    ok = wait_bar(&acc_empty[as], ((ai / kAccStages) & 1) ^ 1, bd);
                    if (!ok) break;
                    ok = wait_bar(x_full, xi & 1, bd);
                    if (!ok) break;
                    x_pending = false;
                    xi++;
                    STEP_STAMP(bar, 4);
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + as * kBatch;
                    for (uint32_t kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t s = it % kRing;
                        ok = wait_bar(&ring_full[s], (it / kRing) & 1, bd);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint64_t da = umma_desc_k_sw128(smem_addr(ring + s * kTile));
                        const uint64_t db = umma_desc_k_sw128(smem_addr(uni + kb * kXkb));
#pragma unroll
                        for (uint32_t k16 = 0; k16 < 4; k16++) umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                        umma_commit(&ring_empty[s]);
                    }
                    if (!ok) break;
                    umma_commit(&acc_full[as]);
                    STEP_STAMP(bar, 5);
                    ai++;
                }
            };
            sync_phase();  // the gather
            for (uint32_t l = 0; l < L; l++) {
                linear(l, LIN_QKV);
                sync_phase();
                sync_phase();  // attention
                linear(l, LIN_O);
                sync_phase();
                sync_phase();  // residual
                linear(l, LIN_GU);
                sync_phase();
                sync_phase();  // gate
                linear(l, LIN_DOWN);
                sync_phase();
                if (l + 1 < L) sync_phase();  // residual; nothing follows the last one
            }
            if (x_pending) drain_bar(x_full, xi & 1, p.wait_ns);
        }
    } else {
        // ---- workers ----
        const uint32_t w = warp - 2, q = warp & 3;
        const uint32_t wid = w * G + cta;  // spreads consecutive units over the blocks first
        uint32_t ai = 0, bar = 0;
        uint32_t kv_parity = 0, kv_pending = 0;  // bit s: parity of the next completion of stage s / a copy in flight
        bool ok = true;
        uint8_t *stages = uni + w * kKvStages * kKvStage;
        uint16_t *prep = reinterpret_cast<uint16_t *>(smem + Smem::prep) + w * kPrepHeads * 128;
        uint64_t *my_kv_full = kv_full + w * kKvStages;
        const Stage st = {stages, my_kv_full, &kv_parity, &kv_pending};  // the residual and gate phases stage through tile stage 0
        auto begin = [&]() {  // the barrier that ended the previous phase
            if (ok && bar > 0) ok = wait_bar(phase_go, (bar - 1) & 1, bd);
            fence_proxy_async_all();  // this warp's bulk copies read what other blocks stored before the barrier
            if (w == 0 && lane == 0) STEP_STAMP(bar, 2);
        };
        auto done = [&]() {
            if (w == 0 && lane == 0) STEP_STAMP(bar, 3);
            fence_proxy_async_all();  // what this warp stored is read by other blocks' TMA loads
            __syncwarp();
            if (lane == 0) mbar_arrive(workers_done);
            bar++;
        };
        auto drain = [&](uint32_t l, uint32_t ph) {  // accumulators of the block's units -> partial sums
            const LinPhase &P = p.lin[ph];
            for (uint32_t u = first_unit(p, l, ph, cta); u < P.units && ok; u += G) {
                const uint32_t tile = u / P.splits, split = u % P.splits;
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
                if (w == 0 && lane == 0) STEP_STAMP(bar, 7);
                const uint32_t r = q * 32 + lane;
                const uint32_t n = P.gated ? (r < 64 ? tile * 64 + r : P.n / 2 + tile * 64 + (r - 64)) : tile * 128 + r;
                float *dst = P.part + (size_t)split * kBatch * P.n + n;
#pragma unroll
                for (uint32_t c = 0; c < kBatch; c++)
                    if (c < p.rows) dst[(size_t)c * P.n] = v[c];
            }
        };
        const uint32_t items = p.rows * p.kv_heads;
        ItemCtx first_item = {};
        if (wid < items) first_item = make_item(p, wid, lane);
        float qg[4] = {1.0f, 1.0f, 1.0f, 1.0f}, kg[4] = {1.0f, 1.0f, 1.0f, 1.0f};
        // phase 0: the gather
        gather_phase(p, p.layers[0].ln1, wid, lane);
        done();
        for (uint32_t l = 0; l < L; l++) {
            const LayerDev &Ly = p.layers[l];
            begin();
            const bool normed = Ly.q_norm != nullptr;
            if (ok && normed && wid < items) {  // the per-head gains of this layer, long before the attention phase wants them
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    qg[e] = __ldg(Ly.q_norm + lane * 2 + e);
                    qg[2 + e] = __ldg(Ly.q_norm + 64 + lane * 2 + e);
                    kg[e] = __ldg(Ly.k_norm + lane * 2 + e);
                    kg[2 + e] = __ldg(Ly.k_norm + 64 + lane * 2 + e);
                }
            }
            if (ok) prefetch_kept(p, Ly, wid, lane);
            drain(l, LIN_QKV);
            done();
            begin();
            if (ok) {
                const CUtensorMap *mk = p.maps + 4 * L + 2 * l, *mv = mk + 1;
                for (uint32_t item = wid; item < items && ok; item += kWorkers * G) {
                    const ItemCtx c = item == wid ? first_item : make_item(p, item, lane);
                    ok = attend_item<GRP>(p, Ly, mk, mv, c, qg, kg, normed, lane, stages, prep, my_kv_full, kv_parity, kv_pending, bd,
                                          w == 0 ? bar : 0);
                }
            }
            done();
            begin();
            drain(l, LIN_O);
            done();
            begin();
            if (ok) ok = residual_phase(p, p.lin[LIN_O], Ly.ln2, wid, lane, st, bd);
            done();
            begin();
            drain(l, LIN_GU);
            done();
            begin();
            if (ok) ok = gated_phase(p, p.lin[LIN_GU], wid, lane, st, bd);
            done();
            begin();
            drain(l, LIN_DOWN);
            done();
            begin();
            if (ok) ok = residual_phase(p, p.lin[LIN_DOWN], l + 1 < L ? p.layers[l + 1].ln1 : nullptr, wid, lane, st, bd);
            done();
        }
        if (!ok && lane == 0) {
            for (uint32_t s = 0; s < kKvStages; s++)
                if ((kv_pending >> s) & 1) drain_bar(&my_kv_full[s], (kv_parity >> s) & 1, p.wait_ns);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
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
    void *maps = nullptr, *layers = nullptr, *sync = nullptr;
    float *parts[4] = {nullptr, nullptr, nullptr, nullptr};
    std::vector<void *> owned;
};

bool step_kernel_supports(const StepKernelShape &s) {
    if (!step_kernel_enabled()) return false;
    if (s.head_dim != 128 || s.heads % s.kv_heads != 0) return false;
    const uint32_t group = s.heads / s.kv_heads;
    if (group != 1 && group != 2 && group != 4) return false;
    if (s.hidden % 256 != 0 || s.ffn % 256 != 0 || (s.heads * s.head_dim) % 256 != 0 || s.hidden > 8192) return false;
    if (!(s.page == 0 || s.page >= 32)) return false;  // 32 aligned positions must be 32 consecutive kept rows
    if (s.kept_rows == 0) return false;
    return true;
}

static void plan_linear(LinPhase *P, uint32_t n, uint32_t k, bool gated, uint32_t x_map, uint32_t blocks) {
    P->n = n;
    P->kb_total = k / 64;
    P->gated = gated ? 1 : 0;
    P->tiles = gated ? (n / 2) / 64 : n / 128;
    P->x_map = x_map;
    // As many k slices as keep one wave of units, at least what the x slice's shared memory asks for; then the
    // fewest slices with the same longest slice (fewer partial sums to add up, same critical path).
    uint32_t most = std::max<uint32_t>(1, blocks / P->tiles);
    most = std::min<uint32_t>(std::min<uint32_t>(most, P->kb_total), 32);
    const uint32_t least = ceil_div(P->kb_total, kMaxKb);
    uint32_t s = std::max(most, least);
    const uint32_t longest = ceil_div(P->kb_total, s);
    while (s > least && s > 1 && ceil_div(P->kb_total, s - 1) == longest) s--;
    P->splits = s;
    P->units = P->tiles * s;
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
    p.blocks = (uint32_t)sm_count();
    p.n_layers = L;
    p.hidden = H;
    p.qw = QW;
    p.ffn = F;
    p.heads = s.heads;
    p.kv_heads = s.kv_heads;
    p.qkv_n = QW + 2 * KW;
    p.ss_parts = H / 128;
    p.vocab = s.vocab;
    plan_linear(&p.lin[LIN_QKV], p.qkv_n, H, false, 0, p.blocks);
    plan_linear(&p.lin[LIN_O], H, QW, false, 1, p.blocks);
    plan_linear(&p.lin[LIN_GU], 2 * F, H, true, 0, p.blocks);
    plan_linear(&p.lin[LIN_DOWN], H, F, false, 2, p.blocks);
    uint32_t cum = 0;
    for (int i = 0; i < 4; i++) {
        p.lin[i].cum = cum;
        cum += p.lin[i].units;
    }
    p.units_per_layer = cum;
    auto dev = [&](void **ptr, size_t bytes) -> int {
        TS_CUDA(cudaMalloc(ptr, bytes));
        k->owned.push_back(*ptr);
        TS_CUDA(cudaMemset(*ptr, 0, bytes));
        return TS_OK;
    };
    int rc;
    for (int i = 0; i < 4; i++) {
        if ((rc = dev((void **)&k->parts[i], (size_t)p.lin[i].splits * kBatch * p.lin[i].n * sizeof(float))) != TS_OK) return bail(rc);
        p.lin[i].part = k->parts[i];
    }
    if ((rc = dev(&k->sync, 256)) != TS_OK) return bail(rc);
    p.sync = (uint32_t *)k->sync;
    // tensor maps: weights of every layer, the three activations, kept K and V of every layer
    std::vector<CUtensorMap> maps(6 * (size_t)L);
    std::vector<LayerDev> layers(L);
    for (uint32_t l = 0; l < L; l++) {
        const StepKernelLayer &Y = b.layers[l];
        if ((rc = make_tensor_map_2d(&maps[l * 4 + LIN_QKV], Y.wqkv, p.qkv_n, H, H, 128, 64)) != TS_OK) return bail(rc);
        if ((rc = make_tensor_map_2d(&maps[l * 4 + LIN_O], Y.wo, H, QW, QW, 128, 64)) != TS_OK) return bail(rc);
        if ((rc = make_tensor_map_2d(&maps[l * 4 + LIN_GU], Y.wgu, 2 * F, H, H, 64, 64)) != TS_OK) return bail(rc);
        if ((rc = make_tensor_map_2d(&maps[l * 4 + LIN_DOWN], Y.wdown, H, F, F, 128, 64)) != TS_OK) return bail(rc);
        if ((rc = make_tensor_map_2d(&maps[4 * L + 2 * l], Y.k_rows, s.kept_rows, KW, KW, 32, 64)) != TS_OK) return bail(rc);
        if ((rc = make_tensor_map_2d(&maps[4 * L + 2 * l + 1], Y.v_rows, s.kept_rows, KW, KW, 32, 64)) != TS_OK) return bail(rc);
        layers[l] = {Y.ln1, Y.ln2, s.qk_norm ? Y.q_norm : nullptr, s.qk_norm ? Y.k_norm : nullptr, (uint16_t *)Y.k_rows,
                     (uint16_t *)Y.v_rows};
    }
    if ((rc = make_tensor_map_2d(&p.x_maps[0], b.xs, s.max_rows, H, H, kBatch, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.x_maps[1], b.attn, s.max_rows, QW, QW, kBatch, 64)) != TS_OK) return bail(rc);
    if ((rc = make_tensor_map_2d(&p.x_maps[2], b.act, s.max_rows, F, F, kBatch, 64)) != TS_OK) return bail(rc);
    if ((rc = dev(&k->maps, maps.size() * sizeof(CUtensorMap))) != TS_OK) return bail(rc);
    if ((rc = dev(&k->layers, layers.size() * sizeof(LayerDev))) != TS_OK) return bail(rc);
    cudaError_t e = cudaMemcpy(k->maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(k->layers, layers.data(), layers.size() * sizeof(LayerDev), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return bail(fail(TS_ERR_CUDA, "step kernel: uploads failed: %s", cudaGetErrorString(e)));
    p.maps = (const CUtensorMap *)k->maps;
    p.layers = (const LayerDev *)k->layers;
    p.x = b.x;
    p.xs = (uint16_t *)b.xs;
    p.attn = (uint16_t *)b.attn;
    p.act = (uint16_t *)b.act;
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
    StepParams p = k->p;
    p.rows = rows;
    p.kept = kept;
    p.max_blk = ceil_div(keys ? keys : 1, 32);
    auto go = [&](auto kernel) -> int {
        TS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem::bytes));
        int per_sm = 0;
        TS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, (int)kThreads, Smem::bytes));
        TS_REQUIRE(per_sm >= 1, "step kernel: a block does not fit an SM");
        TS_CUDA(cudaMemsetAsync(p.sync, 0, 8, stream));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(p.blocks);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = Smem::bytes;
        cfg.stream = stream;
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
