// Decode-sized linear on tcgen05: out[m, n] = sum_k x[m, k] * w[n, k] for m <= 128, with the
// epilogue stage fused and no second kernel.
//
// Weight rows sit on the 128 TMEM lanes (the MMA's M), batch rows on its columns (N = BN >= m).  A
// block loads its k slice of x once by TMA and keeps it in shared memory; 128-row weight tiles then
// stream HBM -> shared memory (TMA, 128-byte swizzle) -> tensor core exactly once.
//
// Small matrices do not have enough 128-row tiles to fill 148 SMs, so k is split over the S blocks of
// a thread-block cluster.  Each block ends with a 128 x BN f32 partial in TMEM; the cluster reduces
// it through distributed shared memory: block r owns batch columns [r BN/S, (r+1) BN/S), every block
// stages its partial of those columns and sends it into block r's receive buffer (one bulk copy per
// peer that credits r's mbarrier; its own share it stores there directly); block r then adds the S
// partials in rank order (a fixed order: a re-run gives the same bits), applies the epilogue (residual
// add, SwiGLU/GeGLU, scale) and stores.  No partial sums touch global memory and nothing is launched
// afterwards.  The exchange is bound by the bytes that cross the cluster, so its buffers carry no
// padding (a row's 4-column groups are swizzled by row for the bank spread instead).
//
// A decode-sized launch is a chain of latencies, not of bandwidth: what is on the path between the
// upstream launch ending and this one's store is kept short.  The weights of a block's one tile are
// all asked for in its first instructions and credit one barrier (a poll of a complete mbarrier still
// costs about 300 clocks); what the epilogue adds to the sums is loaded before the exchange; in gated
// tiles the threads of the up rows share the gate rows' columns.
//
// Gated epilogues pair gate row j with up row j + n/2: a gated tile is 64 gate rows and their 64 up
// rows, so both meet in the owner's receive buffer.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2..9 = epilogue (lane quarter = warp % 4,
// column half = (warp - 2) / 4).  With S == 1 blocks are persistent over tiles and two TMEM
// accumulator stages overlap a tile's epilogue with the next tile's MMAs.
//
// Stands in for the reference's `lanes` / `thin` / `tiled*` rules at decode sizes
// (engine/rules/linear/src/lanes.rs:20-65, tiled.rs:295-446) with their fused epilogue chain
// (engine/plan/lower/src/sites/matmul.rs:148-176).
#include "ts_common.cuh"
#include "ts_kernels.cuh"
#include "ts_ptx.cuh"

namespace ts {
namespace {

using namespace ptx;

constexpr uint32_t kRows = 128;    // weight rows per tile = TMEM lanes
constexpr uint32_t kBlockK = 64;   // bf16 per k block = one 128-byte swizzle row
constexpr uint32_t kEpiWarps = 8;
constexpr uint32_t kThreads = (2 + kEpiWarps) * 32;
constexpr uint32_t kAccStages = 2;
constexpr uint32_t kABytes = kRows * kBlockK * 2;

struct StreamParams {
    uint32_t m, n, k;        // out is [m, n] (or [m, n/2] when gated)
    uint32_t kb_total;       // k / 64
    uint32_t splits;         // S = cluster size along grid y
    uint32_t tiles;          // weight-row tiles
    uint32_t stages;
    uint32_t kb_max;         // most k blocks any split holds (sizes the resident x slice)
    uint32_t gated;
    uint32_t use_recv;       // reduce / pair through the receive buffer (S > 1 or gated)
    uint32_t use_bulk;       // S > 1: partials go out as one bulk copy per peer instead of 16-byte stores
    uint32_t chunk_shift;    // log2(BN / S): batch columns each block owns after the reduce
    uint32_t split_shift;    // log2(S)
    int epilogue, out_dtype;
    float scale;
    const float *a0;
    void *out;
    int *status;
    // Folded RMS norm (FUSED kernels; all NULL / 0 otherwise).
    // In: x holds bf16(row * gain) without the 1/rms factor; row_ss [m, row_parts] holds partial sums of
    // squares of the rows; every output row is multiplied by 1/sqrt(sum/k + row_eps) before the epilogue.
    const float *row_ss;
    uint32_t row_parts;
    float row_eps;
    // Out (f32 output, n % 128 == 0, split k): ss_out [m, tiles] = per-tile sums of squares of the finished
    // rows; xs_out [m, n] = bf16(out * xs_gain[n]), the next linear's x.
    float *ss_out;
    uint16_t *xs_out;
    const float *xs_gain;
};

struct StreamSmem {
    uint32_t a_off, b_off, recv_off, send_off, bar_off, total;
};

// recv: the block reduces / pairs through a receive buffer; send: it also stages its outgoing partials in a
// buffer of the same shape, for bulk copies into the peers' receive buffers.  With a split k every cluster owns
// exactly one tile, so by the time a block stages its partial the weight ring is drained (the MMAs that read it have
// completed and nothing more is copied into it): the send buffer then lies over the ring (send_over_ring) and the
// shared memory it would have taken holds more weight stages, which is what lets all of a block's k blocks be in
// flight before its x arrives (six for the down projection instead of four).
__host__ __device__ inline StreamSmem stream_smem(uint32_t bn, uint32_t stages, uint32_t kb_max, bool recv, bool send,
                                                  uint32_t splits, bool send_over_ring = false) {
    StreamSmem l;
    l.a_off = 0;
    l.b_off = stages * kABytes;
    l.recv_off = l.b_off + kb_max * bn * kBlockK * 2;
    const uint32_t buf = kRows * bn * 4;  // [sender][128 rows][chunk columns] f32, no padding (the 4-column groups of a row are swizzled)
    const bool over = send && send_over_ring && stages * kABytes >= buf;
    l.send_off = over ? l.a_off : l.recv_off + (recv ? buf : 0);
    l.bar_off = l.recv_off + (recv ? buf : 0) + ((send && !over) ? buf : 0);
    // barriers (256), per-warp partial sums of squares (4 x 128 floats) and 128 row factors, slack for the
    // 1024-byte alignment
    l.total = l.bar_off + 256 + 2560 + 1024;
    return l;
}

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag,
                                             bool cluster_scope = false) {
    uint64_t start = 0;
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        if (cluster_scope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > 2000000000ull) break;  // two seconds
        }
    }
    *abort_flag = 1;
    return false;
}

// CW consecutive f32 columns of this warp's TMEM lanes.
template <uint32_t CW>
__device__ __forceinline__ void load_columns(uint32_t taddr, float (&v)[CW]) {
    if constexpr (CW == 8) {
        uint32_t r[8];
        tmem_ld_32x8(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
    } else if constexpr (CW == 16) {
        uint32_t r[16];
        tmem_ld_32x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
    } else {
#pragma unroll
        for (uint32_t c0 = 0; c0 < CW; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) v[c0 + i] = __uint_as_float(r[i]);
        }
    }
}

__device__ __forceinline__ void store_out(void *out, int out_dtype, size_t at, float v) {
    if (out_dtype == TS_F32) reinterpret_cast<float *>(out)[at] = v;
    else reinterpret_cast<uint16_t *>(out)[at] = bf16_bits(v);
}

// FUSED compiles in the folded norm (row factors in, sums of squares and the scaled copy out); the plain instantiation carries
// neither (they cost registers and a few percent of a decode step even when unused).
template <uint32_t BN, bool FUSED>
// (144 registers: a block of the decode attention, 128 threads x 128 registers and 54 KB, then fits the same SM as a
// block of this kernel, so more of the next launch's blocks are resident and fetching key tiles while this one runs.)
__global__ void __maxnreg__(144)
linear_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                     const StreamParams p) {
    constexpr uint32_t CW = BN / 2;  // columns per epilogue warp
    constexpr uint32_t kBBytes = BN * kBlockK * 2;
    constexpr uint32_t kTmemCols = kAccStages * BN < 32 ? 32 : kAccStages * BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const StreamSmem L = stream_smem(BN, p.stages, p.kb_max, p.use_recv != 0, p.use_bulk != 0, p.splits, p.splits > 1);
    unsigned char *smem_a = smem + L.a_off;
    unsigned char *smem_b = smem + L.b_off;
    float *recv = reinterpret_cast<float *>(smem + L.recv_off);  // [S][128][BN / S]
    float *send = reinterpret_cast<float *>(smem + L.send_off);  // same shape, indexed by destination
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bar_off);  // [8]
    uint64_t *empty = full + 8;                                       // [8]
    uint64_t *acc_full = empty + 8;                                   // [2]
    uint64_t *acc_empty = acc_full + 2;                               // [2]
    uint64_t *b_full = acc_empty + 2;
    uint64_t *recv_full = b_full + 1;
    uint64_t *recv_free = recv_full + 1;
    uint64_t *red_full = recv_free + 1;
    uint64_t *inv_full = red_full + 1;
    uint64_t *send_full = inv_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(send_full + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    float *red = reinterpret_cast<float *>(smem + L.bar_off + 256);  // [4][128]
    float *inv_s = red + 512;                                       // [128] 1/rms of the batch rows

    const uint32_t S = p.splits;
    const uint32_t rank = blockIdx.y;  // == cluster rank: the cluster spans grid y
    // (The split is a power of two and a launch has a few thousand k blocks at most: shifts, not the 64-bit divisions
    // that stood between a block's first instruction and its first weight copy.)
    const uint32_t kb_begin = (rank * p.kb_total) >> p.split_shift;
    const uint32_t kb_end = ((rank + 1) * p.kb_total) >> p.split_shift;
    const uint32_t kbs = kb_end - kb_begin;
    const uint32_t chunk = BN / S;  // batch columns this block owns after the reduce

    const uint32_t half_n = p.n / 2;
    const uint32_t my_tiles = blockIdx.x >= p.tiles ? 0 : gridDim.x >= p.tiles ? 1 : (p.tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const uint32_t total_its = my_tiles * kbs;
    // One tile whose k blocks all fit the ring (every decode-sized launch with a split k): all of its weights are
    // asked for at once and credit ONE barrier, the MMA thread waits once and commits once.  A poll of a barrier
    // that is already complete still costs about 300 clocks, a commit about 90: per k block that was a third of a
    // microsecond on the path between x landing and the accumulator being ready.
    const bool whole = my_tiles == 1 && p.stages >= kbs;
    // Stage `it` of this block's stream of weight tiles: tile and k block.
    auto load_weights = [&](uint32_t it) {
        const uint32_t tile = blockIdx.x + (it / kbs) * gridDim.x, kb = it % kbs, s = it % p.stages;
        const int32_t kx = (int32_t)((kb_begin + kb) * kBlockK);
        uint64_t *bar = whole ? &full[0] : &full[s];
        if (!whole) mbar_expect_tx(bar, kABytes);
        unsigned char *dst = smem_a + s * kABytes;
        if (p.gated) {  // 64 gate rows, then their 64 up rows
            tma_load_2d(dst, &map_w, bar, kx, (int32_t)(tile * 64));
            tma_load_2d(dst + kABytes / 2, &map_w, bar, kx, (int32_t)(half_n + tile * 64));
        } else {
            tma_load_2d(dst, &map_w, bar, kx, (int32_t)(tile * kRows));
        }
    };
    const uint32_t early = min(p.stages, total_its);

    if (threadIdx.x == 0) STAMP(0);
    if (threadIdx.x == 0) {
        // Weights never depend on the upstream kernel, and this thread is the only one that touches the barriers
        // of the first stages before the block-wide sync: it sets up just those and the first stages go out at
        // once, while another thread sets up every other barrier and the other warps get ready.  (Behind two dozen
        // barrier initialisations the first copy left 0.8 us into the block; a block that could only start when
        // the launch before it had left waits for exactly these bytes.)
        const uint32_t n_first = whole ? 1 : early;
        for (uint32_t s = 0; s < n_first; s++) mbar_init(&full[s], 1);
        fence_barrier_init();
        if (whole) {  // the block's one tile, stage kb = k block kb: no index arithmetic on the way to the first copy
            mbar_expect_tx(&full[0], kbs * kABytes);
            for (uint32_t kb = 0; kb < kbs; kb++) {
                const int32_t kx = (int32_t)((kb_begin + kb) * kBlockK);
                unsigned char *dst = smem_a + kb * kABytes;
                if (p.gated) {
                    tma_load_2d(dst, &map_w, &full[0], kx, (int32_t)(blockIdx.x * 64));
                    tma_load_2d(dst + kABytes / 2, &map_w, &full[0], kx, (int32_t)(half_n + blockIdx.x * 64));
                } else {
                    tma_load_2d(dst, &map_w, &full[0], kx, (int32_t)(blockIdx.x * kRows));
                }
            }
        } else {
            for (uint32_t it = 0; it < early; it++) load_weights(it);
        }
        STAMP(1);
    } else if (threadIdx.x == 64) {
        const uint32_t n_first = whole ? 1 : early;
        for (uint32_t s = 0; s < p.stages; s++) {
            if (s >= n_first) mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (uint32_t s = 0; s < kAccStages; s++) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kEpiWarps);
        }
        mbar_init(b_full, 1);
        mbar_init(red_full, kEpiWarps);
        mbar_init(inv_full, kEpiWarps);
        mbar_init(send_full, kEpiWarps);
        // S > 1: one local arrival announces the bytes and the senders' asynchronous stores complete
        // them; S == 1: plain stores, one arrival per warp.
        // (with bulk copies a block's own share never leaves it: its eight warps store it straight into the receive
        // buffer and arrive here as well)
        mbar_init(recv_full, S > 1 ? (p.use_bulk ? 1 + kEpiWarps : 1) : kEpiWarps);
        mbar_init(recv_free, kEpiWarps);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    // Cluster barrier 1 (every block's barriers exist before anyone signals them remotely) is split: all
    // arrive here, the epilogue warps wait just before their first remote store, long after.  Barrier 2
    // (no block leaves while a peer may still write into it) likewise: a thread arrives once it will
    // send nothing more, and waits at the very end.
    if (S > 1) cluster_arrive();
    bool waited1 = false, arrived2 = false;
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) STAMP(2);

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            // x is what the upstream kernel wrote: wait for it, then fetch this block's k slice once.
            pdl_wait();
            mbar_expect_tx(b_full, kbs * kBBytes);
            for (uint32_t j = 0; j < kbs; j++)
                tma_load_2d(smem_b + j * kBBytes, &map_x, b_full, (int32_t)((kb_begin + j) * kBlockK), 0);
            uint32_t it = early;
            for (; it < total_its; it++) {
                ok = wait_bounded(&empty[it % p.stages], ((it / p.stages) & 1) ^ 1, abort_flag);
                if (!ok) break;
                load_weights(it);
            }
            STAMP(3);
            pdl_launch_dependents();
            if (ok && whole) {
                ok = wait_bounded(&full[0], 0, abort_flag);  // every copy this thread issued has landed
            } else if (ok) {  // every copy this thread issued has landed once its stage was released
                for (uint32_t back = 0; back < p.stages && back < total_its; back++) {
                    const uint32_t j = total_its - 1 - back;
                    if (!wait_bounded(&empty[j % p.stages], (j / p.stages) & 1, abort_flag)) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(kRows, BN);
            uint32_t it = 0;
            bool ok = wait_bounded(b_full, 0, abort_flag);
            STAMP(4);
            for (uint32_t acc_it = 0; acc_it < my_tiles && ok; acc_it++) {
                const uint32_t as = acc_it % kAccStages, aph = (acc_it / kAccStages) & 1;
                if (acc_it >= kAccStages) ok = wait_bounded(&acc_empty[as], aph ^ 1, abort_flag);  // a stage's first use waits for nobody
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * BN;
                if (whole) {
                    ok = wait_bounded(&full[0], 0, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    for (uint32_t kb = 0; kb < kbs; kb++) {
                        const uint64_t da = umma_desc_k_sw128(smem_addr(smem_a + kb * kABytes));
                        const uint64_t db = umma_desc_k_sw128(smem_addr(smem_b + kb * kBBytes));
#pragma unroll
                        for (uint32_t k16 = 0; k16 < kBlockK / 16; k16++)
                            umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                    }
                    umma_commit(&acc_full[as]);
                    STAMP(5);
                    continue;
                }
                for (uint32_t kb = 0; kb < kbs; kb++, it++) {
                    const uint32_t s = it % p.stages, ph = (it / p.stages) & 1;
                    ok = wait_bounded(&full[s], ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t da = umma_desc_k_sw128(smem_addr(smem_a + s * kABytes));
                    const uint64_t db = umma_desc_k_sw128(smem_addr(smem_b + kb * kBBytes));
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kBlockK / 16; k16++)
                        umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[as]);
                STAMP(5);
            }
        }
    } else {
        // ---- epilogue ----
        const uint32_t q = warp & 3, hcol = (warp - 2) >> 2;
        const uint32_t row = q * 32 + lane;           // tile row (TMEM lane) this thread owns
        const uint32_t col0 = hcol * CW;              // first batch column this thread owns
        const uint32_t out_n = p.gated ? half_n : p.n;
        const uint32_t shift = p.chunk_shift;         // chunk = 1 << shift batch columns per owner
        // Receive-buffer rows are `chunk` floats with no padding: what crosses the cluster is exactly the partial
        // sums (with 8 columns a row, 4 floats of padding were a third of the exchange, and the exchange is bound by
        // bytes).  Banks are spread by swizzling instead: the 4-column group g of row r sits at group g ^ f(r),
        // f(r) = (r >> sh) & mask, chosen so that eight consecutive rows reading the same group touch 32 banks.
        const uint32_t rs = chunk;
        const uint32_t groups = chunk >> 2;
        const uint32_t sw_mask = (groups < 8 ? groups : 8) - 1, sw_shift = groups == 2 ? 2 : groups == 4 ? 1 : 0;
        auto swz = [&](uint32_t r, uint32_t col) -> uint32_t {  // float offset of column `col` (a multiple of 4) in row r
            return (((col >> 2) ^ ((r >> sw_shift) & sw_mask)) << 2);
        };
        const uint32_t recv_base = smem_addr(recv);
        const uint32_t bar_local = smem_addr(recv_full);
        bool ok = true;
        if (FUSED && p.row_ss) {
            // 1/rms of every batch row from the partial sums the upstream linear left; runs under the
            // loads and the MMAs, the epilogue below multiplies by it.
            pdl_wait();
            constexpr uint32_t RPW = BN / kEpiWarps;
            const uint32_t e = warp - 2;
#pragma unroll
            for (uint32_t i = 0; i < RPW; i++) {
                const uint32_t r = e * RPW + i;
                float ss = (r < p.m && lane < p.row_parts) ? p.row_ss[(size_t)r * p.row_parts + lane] : 0.0f;
                ss = warp_sum(ss);
                if (lane == 0) inv_s[r] = 1.0f / sqrtf(ss / (float)p.k + p.row_eps);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(inv_full);
            ok = wait_bounded(inv_full, 0, abort_flag);
        }
        for (uint32_t acc_it = 0; acc_it < my_tiles && ok; acc_it++) {
            const uint32_t tile = blockIdx.x + acc_it * gridDim.x;
            const uint32_t as = acc_it % kAccStages, aph = (acc_it / kAccStages) & 1;
            ok = wait_bounded(&acc_full[as], aph, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            if (warp == 2 && lane == 0) STAMP(6);
            float v[CW];
            load_columns<CW>(tmem_base + ((q * 32u) << 16) + as * BN + col0, v);
            // The accumulator stage is free as soon as it sits in registers.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);

            if (!p.use_recv) {
                // One block holds the whole sum: store straight from registers.  Consecutive lanes
                // are consecutive output columns n; column c of the tile is batch row col0 + c.
                const uint32_t n_idx = tile * kRows + row;
                if (n_idx < p.n) {
                    size_t at = (size_t)col0 * p.n + n_idx;
#pragma unroll
                    for (uint32_t c = 0; c < CW; c++, at += p.n) {
                        if (col0 + c < p.m) {
                            float r = v[c];
                            if (FUSED && p.row_ss) r *= inv_s[col0 + c];
                            if (p.epilogue == TS_EPI_ADD) r += p.a0[at];
                            if (p.epilogue == TS_EPI_SCALE) r *= p.scale;
                            store_out(p.out, p.out_dtype, at, r);
                        }
                    }
                }
                continue;
            }

            // What the epilogue adds to the sums (the residual rows of this thread's outputs, the next norm's gain):
            // asked for now, so that it arrives under the exchange instead of after it.  Thread (row, hcol) takes
            // chunk / 2 consecutive batch columns of its row; with up to eight of them they wait in registers.
            // Gated tiles have 64 output rows for 128 lanes: with eight or more columns a thread, the threads of the up
            // rows take the second half of their gate row's columns instead of idling.
            const uint32_t per = chunk >> 1;
            const bool shared_rows = p.gated && per >= 8;
            const bool active = !p.gated || shared_rows || row < 64;
            const uint32_t orow = p.gated ? (row & 63) : row;  // the tile's output row this thread works on
            const uint32_t n_idx = p.gated ? tile * 64 + orow : tile * kRows + row;
            const bool early_adds = p.use_recv && p.epilogue == TS_EPI_ADD && per <= 8 && active && n_idx < out_n;
            float4 add_lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), add_hi = add_lo;
            float next_gain = 1.0f;
            if (early_adds) {
                const uint32_t m_first = rank * chunk + hcol * per;
                float a[8];
#pragma unroll
                for (uint32_t j = 0; j < 8; j++)
                    a[j] = (j < per && m_first + j < p.m) ? __ldcg(p.a0 + (size_t)(m_first + j) * out_n + n_idx) : 0.0f;
                add_lo = make_float4(a[0], a[1], a[2], a[3]);
                add_hi = make_float4(a[4], a[5], a[6], a[7]);
            }
            if (FUSED && p.xs_out && active && n_idx < out_n) next_gain = __ldg(p.xs_gain + n_idx);

            // The receive buffer of the previous tile must have been read by all of this block.
            if (acc_it > 0) {
                ok = wait_bounded(recv_free, (acc_it - 1) & 1, abort_flag);
                if (!ok) break;
            }
            if (S > 1) {
                if (!waited1) {
                    cluster_wait();
                    waited1 = true;
                }
                if (p.use_bulk) {
                    // Stage the partial in this block's send buffer, laid out like a peer's receive buffer
                    // (by destination, row, column), then one thread sends each destination its 128 x chunk
                    // block as a single bulk copy that credits the destination's barrier.  Eight 16-byte
                    // remote stores per thread took 2.3 us of a 7.7 us kernel; this takes a fraction.
#pragma unroll
                    for (uint32_t c = 0; c < CW; c += 4) {
                        const uint32_t col = col0 + c;
                        const uint32_t dest = col >> shift, within = col & (chunk - 1);
                        // the columns this block owns itself go straight where its reduce reads them
                        float *to = dest == rank ? recv + (rank * kRows + row) * rs : send + (dest * kRows + row) * rs;
                        *reinterpret_cast<float4 *>(to + swz(row, within)) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
                    }
                    fence_async_shared();  // the copy engine reads what these threads wrote
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(send_full);
                        mbar_arrive(recv_full);  // this warp's part of the block's own share is in place
                    }
                    if (warp == 2 && lane == 0) {
                        const uint32_t block_bytes = kRows * rs * 4;
                        mbar_expect_tx(recv_full, (S - 1) * block_bytes);
                        if (wait_bounded(send_full, acc_it & 1, abort_flag)) {
                            for (uint32_t d = 0; d < S; d++)
                                if (d != rank)
                                    bulk_copy_to_peer(map_to_rank(recv_base + rank * block_bytes, d),
                                                      smem_addr(send) + d * block_bytes, block_bytes, map_to_rank(bar_local, d));
                        }
                    }
                } else {
                    // This block will receive S x 128 rows x chunk columns of f32 for the tile.
                    if (warp == 2 && lane == 0) mbar_expect_tx(recv_full, S * kRows * chunk * 4);
                    // Send: columns [col0, col0 + CW) go to the blocks that own them as asynchronous
                    // 16-byte stores that credit the owner's barrier; the sender does not wait for them.
#pragma unroll
                    for (uint32_t c = 0; c < CW; c += 4) {
                        const uint32_t col = col0 + c;
                        const uint32_t dest = col >> shift, within = col & (chunk - 1);
                        const uint32_t local = recv_base + ((rank * kRows + row) * rs + swz(row, within)) * 4;
                        st_async_f32x4(map_to_rank(local, dest), map_to_rank(bar_local, dest), v[c], v[c + 1], v[c + 2],
                                       v[c + 3]);
                    }
                }
                // (With bulk copies the source buffer is still being read: that thread arrives after its own
                // receive, below, by when every peer has its data.)
                if (acc_it + 1 >= my_tiles && !arrived2 && !p.use_bulk) {  // nothing more goes to the peers from this thread
                    cluster_arrive();
                    arrived2 = true;
                }
            } else {
                // One block: the buffer only pairs gate rows with up rows.  Plain stores, then one
                // arrival per warp.
#pragma unroll
                for (uint32_t c = 0; c < CW; c += 4)
                    *reinterpret_cast<float4 *>(recv + row * rs + swz(row, col0 + c)) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
                __syncwarp();
                if (lane == 0) mbar_arrive(recv_full);
            }
            if (warp == 2 && lane == 0) STAMP(7);
            ok = wait_bounded(recv_full, acc_it & 1, abort_flag);
            if (!ok) break;
            if (S > 1 && p.use_bulk && acc_it + 1 >= my_tiles && !arrived2) {
                cluster_arrive();
                arrived2 = true;
            }
            if (warp == 2 && lane == 0) STAMP(8);

            // Reduce the S partials of this block's columns in rank order, finish, store.  Thread
            // (row, hcol) takes chunk / 2 consecutive columns of its row.
            if (active && n_idx < out_n) {
                const uint32_t cc_lo = hcol * per + ((shared_rows && row >= 64) ? per / 2 : 0);
                const uint32_t cc_hi = shared_rows ? cc_lo + per / 2 : cc_lo + per;
                for (uint32_t cc = cc_lo; cc < cc_hi; cc += 4) {
                    const float *src = recv + orow * rs + swz(orow, cc);
                    float4 sum = *reinterpret_cast<const float4 *>(src);
                    float4 up = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (p.gated) up = *reinterpret_cast<const float4 *>(src + 64 * rs);
                    for (uint32_t s = 1; s < S; s++) {
                        const float4 t = *reinterpret_cast<const float4 *>(src + (size_t)s * kRows * rs);
                        sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
                        if (p.gated) {
                            const float4 u = *reinterpret_cast<const float4 *>(src + ((size_t)s * kRows + 64) * rs);
                            up.x += u.x; up.y += u.y; up.z += u.z; up.w += u.w;
                        }
                    }
                    const float r4[4] = {sum.x, sum.y, sum.z, sum.w};
                    const float u4[4] = {up.x, up.y, up.z, up.w};
                    const float4 add4 = cc == hcol * per ? add_lo : add_hi;
                    const float e4[4] = {add4.x, add4.y, add4.z, add4.w};
                    const uint32_t m0 = rank * chunk + cc;
                    size_t at = (size_t)m0 * out_n + n_idx;
#pragma unroll
                    for (uint32_t j = 0; j < 4; j++, at += out_n) {
                        float r = 0.0f;
                        if (m0 + j < p.m) {
                            const float f = (FUSED && p.row_ss) ? inv_s[m0 + j] : 1.0f;
                            r = r4[j] * f;
                            if (p.gated) r = (p.epilogue == TS_EPI_SWIGLU ? silu(r) : gelu_tanh(r)) * (u4[j] * f);
                            if (p.epilogue == TS_EPI_ADD) r += early_adds ? e4[j] : p.a0[at];
                            if (p.epilogue == TS_EPI_SCALE) r *= p.scale;
                            store_out(p.out, p.out_dtype, at, r);
                            if (FUSED && p.xs_out) p.xs_out[at] = bf16_bits(r * next_gain);
                        }
                        if (FUSED && p.ss_out) {  // the host only asks for this when n is a multiple of 128: every lane is here
                            const float t = warp_sum(r * r);
                            if (lane == 0) red[q * 128 + cc + j] = t;
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(recv_free);
            if (FUSED && p.ss_out) {
                // The four lane quarters of a column meet in shared memory; one thread per batch column
                // adds them in a fixed order.
                __syncwarp();
                if (lane == 0) mbar_arrive(red_full);
                ok = wait_bounded(red_full, acc_it & 1, abort_flag);
                if (!ok) break;
                const uint32_t t = (warp - 2) * 32 + lane;
                if (t < chunk && rank * chunk + t < p.m)
                    p.ss_out[(size_t)(rank * chunk + t) * p.tiles + tile] =
                        ((red[t] + red[128 + t]) + red[256 + t]) + red[384 + t];
            }
            if (warp == 2 && lane == 0) STAMP(9);
        }
    }

    if (S > 1) {
        if (!waited1) cluster_wait();
        if (!arrived2) cluster_arrive();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) STAMP(10);
    if (S > 1) cluster_wait();  // no block leaves while a peer may still write to it
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TS_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

struct StreamPlan {
    uint32_t bn, splits, tiles, stages, kb_total, kb_max, blocks;
    bool gated, use_recv, use_bulk;
    StreamSmem layout;
};

constexpr uint32_t kSmemBudget = 225 * 1024;

// Clusters of `size` blocks of this kernel (one block an SM) that the device holds at once: GPCs whose SM count is
// not a multiple of the cluster size strand SMs, so 148 SMs hold fewer than 148 / size clusters.  Cached per
// device and size.
uint32_t resident_clusters(uint32_t size) {
    static std::atomic<uint32_t> cache[256][4] = {};
    const uint32_t slot = size == 2 ? 0 : size == 4 ? 1 : size == 8 ? 2 : 3;
    std::atomic<uint32_t> &c = cache[current_device() & 255][slot];
    if (const uint32_t have = c.load(std::memory_order_relaxed)) return have;
    auto kernel = linear_stream_kernel<64, false>;
    uint32_t found = (uint32_t)sm_count() / size;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, size * ((uint32_t)sm_count() / size));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBudget;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = size;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0) found = (uint32_t)n;
        else cudaGetLastError();
    } else {
        cudaGetLastError();
    }
    c.store(found, std::memory_order_relaxed);
    return found;
}

bool plan_stream(uint32_t m, uint32_t n, uint32_t k, int epilogue, StreamPlan *out) {
    StreamPlan s = {};
    s.gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    if (m == 0 || m > 128 || n == 0 || k == 0 || k % kBlockK != 0) return false;
    if (s.gated && (n % 2 != 0 || (n / 2) % 64 != 0)) return false;
    s.bn = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    s.kb_total = k / kBlockK;
    s.tiles = s.gated ? (n / 2) / 64 : ceil_div(n, kRows);
    const uint32_t sms = (uint32_t)sm_count();
    auto layout = [&](uint32_t splits, uint32_t stages, bool send = false) {
        const uint32_t kb_max = ceil_div(s.kb_total, splits);
        return stream_smem(s.bn, stages, kb_max, splits > 1 || s.gated, send, splits, splits > 1);
    };
    // The largest power-of-two split that still fits one wave; more if the resident x slice needs it.
    uint32_t splits = 1;
    const uint32_t max_splits = std::min<uint32_t>(std::min<uint32_t>(8, s.bn / 8), s.kb_total);
    while (splits * 2 <= max_splits && s.tiles * splits * 2 <= sms) splits *= 2;
    // ... and whose clusters are all resident at once: 16 clusters of 8 do not fit 148 SMs (a second wave doubles
    // the launch), 16 of 4 do.
    while (splits > 1 && s.tiles > resident_clusters(splits) && layout(splits / 2, 2).total <= kSmemBudget) splits /= 2;
    while (layout(splits, 2).total > kSmemBudget && splits * 2 <= max_splits) splits *= 2;
    if (layout(splits, 2).total > kSmemBudget) return false;
    s.splits = splits;
    s.kb_max = ceil_div(s.kb_total, splits);
    s.use_recv = splits > 1 || s.gated;
    // Bulk copies for the cluster reduce need a send buffer as large as the receive buffer: taken when at
    // least three weight stages (or all the block's k blocks) still fit beside it.
    const uint32_t want = std::min<uint32_t>(3, s.kb_max);
    s.use_bulk = splits > 1 && layout(splits, want, true).total <= kSmemBudget;
    // With a split k a block streams one tile: more stages than its k blocks would only hold shared memory that a
    // block of the next launch (the decode attention's are 54 KB) could use to become resident early.
    uint32_t stages = splits > 1 ? std::max<uint32_t>(2, std::min<uint32_t>(8, s.kb_max)) : 8;
    while (stages > 2 && layout(splits, stages, s.use_bulk).total > kSmemBudget) stages--;
    s.stages = stages;
    s.layout = layout(splits, stages, s.use_bulk);
    s.blocks = splits > 1 ? s.tiles : std::min(s.tiles, sms);
    *out = s;
    return true;
}

__device__ int g_stream_status = 0;

template <uint32_t BN, bool FUSED>
cudaError_t launch_stream(const CUtensorMap &mw, const CUtensorMap &mx, const StreamParams &p, const StreamPlan &s,
                          cudaStream_t stream) {
    auto kernel = linear_stream_kernel<BN, FUSED>;
    static OncePerDevice configured;
    if (configured.needs()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
        if (e != cudaSuccess) return e;
        configured.done();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(s.blocks, s.splits);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = s.layout.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (s.splits > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = s.splits;
        attr[n_attr].val.clusterDim.z = 1;
        n_attr++;
    }
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return cudaLaunchKernelEx(&cfg, kernel, mw, mx, p);
}

}  // namespace

#ifdef TS_DEBUG_STAMPS
extern "C" __attribute__((visibility("default"))) int ts_debug_stamps(unsigned long long *out) {
    return cudaMemcpyFromSymbol(out, g_stamps, sizeof(unsigned long long) * 16 * 32) == cudaSuccess ? 0 : 6;
}
#endif

bool stream_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    StreamPlan s;
    return plan_stream(m, n, k, epilogue, &s);
}

int stream_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
    return v;
}

uint32_t stream_sumsq_parts(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    StreamPlan s;
    if (!plan_stream(m, n, k, epilogue, &s)) return 0;
    return (!s.gated && s.splits > 1 && n % kRows == 0) ? s.tiles : 0;
}

int linear_stream(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                  int epilogue, float scale, int out_dtype, cudaStream_t stream, const StreamFused *fused) {
    // 65..128 rows against a large matrix: with 128 batch columns the resident x slice forces a k split over a
    // cluster on every one of thousands of tiles (469 us for the 151936 x 1024 unembedding against 65 us at 64
    // rows).  Two launches of at most 64 rows each read the weights twice and still finish in a third of the time.
    if (m > 64 && m <= 128 && (size_t)n * k >= ((size_t)16 << 20) && !fused) {
        const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
        const size_t out_n = gated ? n / 2 : n, esz = out_dtype == TS_F32 ? 4 : 2;
        int rc = linear_stream(x, w, a0, out, 64, n, k, epilogue, scale, out_dtype, stream, nullptr);
        if (rc != TS_OK) return rc;
        return linear_stream((const char *)x + (size_t)64 * k * 2, w, a0 ? (const char *)a0 + 64 * out_n * 4 : nullptr,
                             (char *)out + 64 * out_n * esz, m - 64, n, k, epilogue, scale, out_dtype, stream, nullptr);
    }
    StreamPlan s;
    if (!plan_stream(m, n, k, epilogue, &s))
        return fail(TS_ERR_BAD_INPUT, "linear (stream): unsupported shape m=%u n=%u k=%u epilogue=%d", m, n, k, epilogue);
    CUtensorMap map_w, map_x;
    int rc = make_tensor_map_2d(&map_w, w, n, k, k, s.gated ? 64 : kRows, kBlockK);
    if (rc != TS_OK) return rc;
    rc = make_tensor_map_2d(&map_x, x, m, k, k, s.bn, kBlockK);
    if (rc != TS_OK) return rc;
    if (fused && fused->row_ss)
        TS_REQUIRE(fused->row_parts >= 1 && fused->row_parts <= 32, "linear (stream): 1..32 partial sums per row, got %u",
                   fused->row_parts);
    if (fused && (fused->ss_out || fused->xs_out)) {
        TS_REQUIRE(stream_sumsq_parts(m, n, k, epilogue) != 0 && out_dtype == TS_F32,
                   "linear (stream): sums of squares need an f32 output, n %% 128 == 0 and a split k (m=%u n=%u k=%u)", m, n, k);
        TS_REQUIRE(!fused->xs_out || fused->xs_gain, "linear (stream): xs_out needs xs_gain");
    }
    StreamParams p = {};
    if (fused) {
        p.row_ss = fused->row_ss;
        p.row_parts = fused->row_parts;
        p.row_eps = fused->row_eps;
        p.ss_out = fused->ss_out;
        p.xs_out = (uint16_t *)fused->xs_out;
        p.xs_gain = fused->xs_gain;
    }
    p.m = m;
    p.n = n;
    p.k = k;
    p.kb_total = s.kb_total;
    p.splits = s.splits;
    p.tiles = s.tiles;
    p.stages = s.stages;
    p.kb_max = s.kb_max;
    p.gated = s.gated;
    p.use_recv = s.use_recv;
    p.use_bulk = s.use_bulk;
    {
        uint32_t chunk = s.bn / s.splits, sh = 0;
        while ((1u << sh) < chunk) sh++;
        p.chunk_shift = sh;
        uint32_t ssh = 0;
        while ((1u << ssh) < s.splits) ssh++;
        p.split_shift = ssh;
    }
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.scale = scale;
    p.a0 = (const float *)a0;
    p.out = out;
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_stream_status));
    p.status = status;
    cudaError_t e;
    const bool any_fused = p.row_ss || p.ss_out || p.xs_out;
    switch (s.bn) {
    case 16: e = any_fused ? launch_stream<16, true>(map_w, map_x, p, s, stream) : launch_stream<16, false>(map_w, map_x, p, s, stream); break;
    case 32: e = any_fused ? launch_stream<32, true>(map_w, map_x, p, s, stream) : launch_stream<32, false>(map_w, map_x, p, s, stream); break;
    case 64: e = any_fused ? launch_stream<64, true>(map_w, map_x, p, s, stream) : launch_stream<64, false>(map_w, map_x, p, s, stream); break;
    default: e = any_fused ? launch_stream<128, true>(map_w, map_x, p, s, stream) : launch_stream<128, false>(map_w, map_x, p, s, stream); break;
    }
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_stream failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
