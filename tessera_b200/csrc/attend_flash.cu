// Whole-sequence (prefill) attention on the 5th-generation tensor cores, head widths 128 and 256.
//
// One block owns 128 queries of one (sequence, head) and walks the visible keys BK at a time (128 keys
// at width 128, 64 at width 256):
//   S  = Q K^T   tcgen05.mma 128 x BK x 16, Q and K tiles K-major in shared memory (TMA, 128 B swizzle),
//                S (f32) in tensor memory, two buffers
//   P  = exp2(S * scale*log2e - m)   one softmax thread per query row reads its S row from TMEM (no
//                shuffles: the row is private to the thread), applies the mask window, and writes P as
//                bf16 pairs back into the same TMEM columns
//   O += P V     tcgen05.mma with A from TMEM (P) and V as an MN-major shared-memory operand (the V tile
//                is stored [key][dim] as TMA delivers it); O (f32, 128 x width) accumulates in TMEM over
//                all key blocks
// The maximum m the probabilities are taken against may lag the true running maximum by up to 8 (log2
// units): O and the running sum are rescaled (TMEM load, multiply, store) only when the maximum runs
// further ahead, which is rare after the first blocks, so the softmax thread's steady-state work is two
// passes over S.  The MMA thread runs one block ahead (S of block j+1 while block j is in softmax) and
// TMA keeps two K and two V tiles in flight.  Warp roles: 0 = TMA, 1 = MMA (owns TMEM), 2..5 = softmax
// and output.  Masks are the reference's per-query window [pos - back, pos + ahead] with query and key
// ends aligned (engine/ir/graph/src/node.rs:162-187; engine/ir/interp/src/cpu.rs:61-77).
//
// Stands in for the `flash*` rules (engine/rules/attention/src/flash.rs:415-502, launch 648-668).
#include <algorithm>
#include <cmath>

#include "ts_common.cuh"
#include "ts_ptx.cuh"

namespace ts {
namespace {

using namespace ptx;

constexpr uint32_t kTile = 128;     // queries per block = TMEM lanes
constexpr uint32_t kThreads = 192;
constexpr float kRescaleStep = 8.0f;  // log2 units the row maximum may run ahead of the one in use

struct FlashParams {
    uint16_t *out;
    const uint32_t *cu_seqlens;  // NULL: fixed lengths
    uint32_t seqs, queries, keys, heads, kv_heads;
    uint32_t back, ahead;
    float scale_log2;            // scale * log2(e)
    uint32_t q_tiles;
    int *status;
};

// D: head width (128 or 256).  BK keys per step: 128 at width 128, 64 at width 256, so that Q plus
// two K and two V tiles fit shared memory and S (2 buffers) plus O fit the 512 TMEM columns.
template <uint32_t D>
struct FlashShape {
    static constexpr uint32_t BK = D == 128 ? 128 : 64;
    static constexpr uint32_t chunks = D / 64;                 // 64-wide slices of the head width
    static constexpr uint32_t q_chunk = kTile * 128;           // bytes of one slice of the Q tile
    static constexpr uint32_t kv_chunk = BK * 128;             // bytes of one slice of a K or V tile
    static constexpr uint32_t q_bytes = chunks * q_chunk;
    static constexpr uint32_t kv_bytes = chunks * kv_chunk;
    static constexpr uint32_t q_off = 0;
    static constexpr uint32_t k_off = q_bytes;
    static constexpr uint32_t v_off = k_off + 2 * kv_bytes;
    static constexpr uint32_t bar_off = v_off + 2 * kv_bytes;
    static constexpr uint32_t total = bar_off + 256 + 1024;
    static constexpr uint32_t s_col = 0;                       // S / P buffers at 0 and BK
    static constexpr uint32_t o_col = 2 * BK;                  // O: D columns
};

__device__ __forceinline__ uint32_t sat_add(uint32_t a, uint32_t b) {
    uint32_t s = a + b;
    return s < a ? 0xFFFFFFFFu : s;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// What a work item (a 128-query tile of one sequence and head) covers; every role derives it from the item's
// index in the same way.
struct FlashItem {
    uint32_t head, kvh, q_begin, k_begin, k_len, past, t0, rows_here, jb0, nb;
};

template <uint32_t BK>
__device__ __forceinline__ FlashItem flash_item(const FlashParams &p, uint32_t item) {
    FlashItem it;
    const uint32_t per = p.heads * p.seqs;
    const uint32_t tile = p.q_tiles - 1 - item / per, rem = item % per;  // later tiles (more keys under a causal mask) first
    const uint32_t seq = rem / p.heads;
    it.head = rem % p.heads;
    it.kvh = it.head / (p.heads / p.kv_heads);
    uint32_t q_len;
    if (p.cu_seqlens) {
        it.q_begin = it.k_begin = p.cu_seqlens[seq];
        q_len = it.k_len = p.cu_seqlens[seq + 1] - it.q_begin;
    } else {
        it.q_begin = seq * p.queries;
        q_len = p.queries;
        it.k_begin = seq * p.keys;
        it.k_len = p.keys;
    }
    it.t0 = tile * kTile;
    it.past = it.k_len > q_len ? it.k_len - q_len : 0;
    it.rows_here = it.t0 < q_len ? min(kTile, q_len - it.t0) : 0;
    it.jb0 = it.nb = 0;
    if (it.rows_here) {
        // Keys any query of the tile can see: [lo, hi).
        const uint32_t pos_first = it.past + it.t0, pos_last = pos_first + it.rows_here - 1;
        const uint32_t lo = pos_first > p.back ? pos_first - p.back : 0;
        const uint32_t hi = min(it.k_len, sat_add(sat_add(pos_last, p.ahead), 1));
        it.jb0 = lo / BK;
        it.nb = hi > lo ? (hi + BK - 1) / BK - it.jb0 : 0;
    }
    return it;
}

// Blocks are persistent over items (item = blockIdx.x, + gridDim.x, ...): the block-level set-up (barriers,
// TMEM) is paid once, which matters for batches of short sequences where an item is a handful of key blocks.
// Barrier phases run on across items.
template <uint32_t D>
__global__ void __launch_bounds__(kThreads, 1)
attend_flash_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const FlashParams p, const uint32_t items) {
    using Sh = FlashShape<D>;
    constexpr uint32_t BK = Sh::BK;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *smem_q = smem + Sh::q_off;
    unsigned char *smem_k = smem + Sh::k_off;
    unsigned char *smem_v = smem + Sh::v_off;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Sh::bar_off);
    uint64_t *q_full = bars;          // [1]
    uint64_t *k_full = bars + 1;      // [2]
    uint64_t *v_full = bars + 3;      // [2]
    uint64_t *k_empty = bars + 5;     // [2]
    uint64_t *v_empty = bars + 7;     // [2]
    uint64_t *s_full = bars + 9;      // [2]
    uint64_t *p_full = bars + 11;     // [2]
    uint64_t *pv_done = bars + 13;    // [2]
    uint64_t *q_empty = bars + 15;    // [1]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 16);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 4);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            bool ok = true;
            uint32_t jr = 0, n_item = 0;  // key blocks and items (with keys) so far
            for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
                const FlashItem it = flash_item<BK>(p, item);
                if (it.nb == 0) continue;
                // Q of the previous item is free once its MMAs are done.
                if (n_item > 0) ok = mbar_wait_or_abort(q_empty, (n_item - 1) & 1, abort_flag);
                if (!ok) break;
                n_item++;
                mbar_expect_tx(q_full, Sh::q_bytes);
                for (uint32_t c = 0; c < Sh::chunks; c++)
                    tma_load_2d(smem_q + c * Sh::q_chunk, &map_q, q_full, (int32_t)(it.head * D + c * 64),
                                (int32_t)(it.q_begin + it.t0));
                for (uint32_t j = 0; j < it.nb && ok; j++, jr++) {
                    const uint32_t s = jr & 1, ph = (jr >> 1) & 1;
                    const int32_t krow = (int32_t)(it.k_begin + (it.jb0 + j) * BK);
                    ok = mbar_wait_or_abort(&k_empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&k_full[s], Sh::kv_bytes);
                    for (uint32_t c = 0; c < Sh::chunks; c++)
                        tma_load_2d(smem_k + s * Sh::kv_bytes + c * Sh::kv_chunk, &map_k, &k_full[s],
                                    (int32_t)(it.kvh * D + c * 64), krow);
                    ok = mbar_wait_or_abort(&v_empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&v_full[s], Sh::kv_bytes);
                    for (uint32_t c = 0; c < Sh::chunks; c++)
                        tma_load_2d(smem_v + s * Sh::kv_bytes + c * Sh::kv_chunk, &map_v, &v_full[s],
                                    (int32_t)(it.kvh * D + c * 64), krow);
                }
            }
            pdl_launch_dependents();
            // Copies in flight land before the MMAs that release their stages; wait for those releases.
            for (uint32_t back = 0; back < 2 && back < jr && ok; back++) {
                const uint32_t j = jr - 1 - back;
                ok = mbar_wait_or_abort(&k_empty[j & 1], (j >> 1) & 1, abort_flag) &&
                     mbar_wait_or_abort(&v_empty[j & 1], (j >> 1) & 1, abort_flag);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc_bf16(kTile, BK, false, false);
            const uint32_t idesc_pv = umma_idesc_bf16(kTile, D, false, true);  // V is MN-major
            bool ok = true;
            uint32_t jr = 0, n_item = 0;
            auto issue_qk = [&](uint32_t r) -> bool {  // r: running index of the key block
                const uint32_t s = r & 1, ph = (r >> 1) & 1;
                if (!mbar_wait_or_abort(&k_full[s], ph, abort_flag)) return false;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + Sh::s_col + s * BK;
#pragma unroll
                for (uint32_t c = 0; c < Sh::chunks; c++) {
                    const uint64_t da = umma_desc_k_sw128(smem_addr(smem_q + c * Sh::q_chunk));
                    const uint64_t db = umma_desc_k_sw128(smem_addr(smem_k + s * Sh::kv_bytes + c * Sh::kv_chunk));
#pragma unroll
                    for (uint32_t k16 = 0; k16 < 4; k16++)
                        umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc_qk, (c | k16) != 0);
                }
                umma_commit(&k_empty[s]);
                umma_commit(&s_full[s]);
                return true;
            };
            for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
                const FlashItem it = flash_item<BK>(p, item);
                if (it.nb == 0) continue;
                ok = mbar_wait_or_abort(q_full, n_item & 1, abort_flag);
                n_item++;
                if (ok) ok = issue_qk(jr);
                for (uint32_t j = 0; j < it.nb && ok; j++, jr++) {
                    const uint32_t s = jr & 1, ph = (jr >> 1) & 1;
                    if (j + 1 < it.nb) {
                        ok = issue_qk(jr + 1);
                        if (!ok) break;
                    }
                    ok = mbar_wait_or_abort(&p_full[s], ph, abort_flag) && mbar_wait_or_abort(&v_full[s], ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t p_tmem = tmem_base + Sh::s_col + s * BK;  // bf16 pairs: 16 keys = 8 columns
                    const uint32_t o_tmem = tmem_base + Sh::o_col;
                    const uint32_t v_addr = smem_addr(smem_v + s * Sh::kv_bytes);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < BK / 16; k16++) {
                        // 16 keys = 16 rows of 128 bytes further down the V tile; the 64-wide slices of the head
                        // width are kv_chunk bytes apart, 8-row groups 1024 bytes apart.
                        const uint64_t db = umma_desc_mn_sw128(v_addr + k16 * 2048, Sh::kv_chunk, 1024);
                        umma_bf16_ts(o_tmem, p_tmem + k16 * 8, db, idesc_pv, (j | k16) != 0);
                    }
                    umma_commit(&v_empty[s]);
                    umma_commit(&pv_done[s]);
                }
                if (ok) umma_commit(q_empty);
            }
        }
    } else {
        // ---- softmax + output: thread = query row ----
        const uint32_t q = warp & 3;
        const uint32_t row = q * 32 + lane;
        const uint32_t lane_base = (q * 32u) << 16;
        const uint32_t o_tmem = tmem_base + lane_base + Sh::o_col;
        bool ok = true;
        uint32_t jr = 0;
        for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const FlashItem it = flash_item<BK>(p, item);
        if (it.rows_here == 0) continue;
        const uint32_t nb = it.nb, jb0 = it.jb0, k_len = it.k_len;
        const bool row_ok = row < it.rows_here;
        const uint32_t pos = it.past + it.t0 + row;
        const uint32_t from = pos > p.back ? pos - p.back : 0;
        const uint32_t to = min(k_len, sat_add(sat_add(pos, p.ahead), 1));
        float m_use = -INFINITY;  // the maximum the probabilities are taken against (may lag the true one)
        float l_run = 0.0f;
        for (uint32_t j = 0; j < nb && ok; j++, jr++) {
            const uint32_t s = jr & 1, ph = (jr >> 1) & 1;
            ok = mbar_wait_or_abort(&s_full[s], ph, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t s_tmem = tmem_base + lane_base + Sh::s_col + s * BK;
            const uint32_t key0 = (jb0 + j) * BK;
            // Keys of this block the row sees: [c_from, c_to) in block columns.
            const uint32_t c_from = from > key0 ? min(from - key0, BK) : 0;
            const uint32_t c_to = to > key0 ? min(to - key0, BK) : 0;
            // The whole S row of the block in registers (one TMEM read); masked keys become -inf so that the
            // exponentials below need no selects.  Eight independent running maxima.
            uint32_t rr[BK / 32][32];
#pragma unroll
            for (uint32_t c = 0; c < BK / 32; c++) tmem_ld_32x32(s_tmem + c * 32, rr[c]);
            tmem_ld_wait();
            float mx[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; i++) mx[i] = -INFINITY;
            if (c_from == 0 && c_to == BK) {
#pragma unroll
                for (uint32_t c = 0; c < BK; c++) mx[c & 7] = fmaxf(mx[c & 7], __uint_as_float(rr[c >> 5][c & 31]));
            } else {
#pragma unroll
                for (uint32_t c = 0; c < BK; c++) {
                    const float v = (c >= c_from && c < c_to) ? __uint_as_float(rr[c >> 5][c & 31]) : -INFINITY;
                    rr[c >> 5][c & 31] = __float_as_uint(v);
                    mx[c & 7] = fmaxf(mx[c & 7], v);
                }
            }
            const float m_blk = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                      fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
            const float m_new = fmaxf(m_use, m_blk * p.scale_log2);
            // Rescale O and the running sum only when the maximum ran ahead by more than kRescaleStep:
            // probabilities stay below 2^kRescaleStep, and after the first blocks this is rare.
            float alpha = 1.0f;
            bool need = false;
            if (m_new > m_use + kRescaleStep || m_use == -INFINITY) {
                need = l_run > 0.0f;
                alpha = need ? ex2(m_use - m_new) : 1.0f;
                m_use = m_new;
            }
            if (__any_sync(0xFFFFFFFFu, need)) {
                // O is complete up to the previous block once its MMAs are done.
                const uint32_t sp = (jr - 1) & 1, php = ((jr - 1) >> 1) & 1;
                ok = mbar_wait_or_abort(&pv_done[sp], php, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
#pragma unroll
                for (uint32_t c0 = 0; c0 < D; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(o_tmem + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (uint32_t c = 0; c < 32; c++) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                    tmem_st_32x32(o_tmem + c0, r);
                }
                l_run *= alpha;
            }
            const float neg_m = m_use == -INFINITY ? 0.0f : -m_use;
            float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (uint32_t c0 = 0; c0 < BK / 32; c0++) {
                uint32_t packed[16];
#pragma unroll
                for (uint32_t c = 0; c < 32; c += 2) {
                    const float p0 = ex2(fmaf(__uint_as_float(rr[c0][c]), p.scale_log2, neg_m));
                    const float p1 = ex2(fmaf(__uint_as_float(rr[c0][c + 1]), p.scale_log2, neg_m));
                    ls[(c >> 1) & 1] += p0;
                    ls[2 + ((c >> 1) & 1)] += p1;
                    packed[c >> 1] = pack_bf16(p0, p1);
                }
                tmem_st_32x16(s_tmem + c0 * 16, packed);
            }
            const float l_blk = (ls[0] + ls[1]) + (ls[2] + ls[3]);
            l_run += l_blk;
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s]);
        }
        if (ok && nb > 0) {
            const uint32_t sp = (jr - 1) & 1, php = ((jr - 1) >> 1) & 1;
            ok = mbar_wait_or_abort(&pv_done[sp], php, abort_flag);
            if (ok) tc_fence_after_sync();
        }
        if (ok) {
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            uint16_t *dst = p.out + ((size_t)(it.q_begin + it.t0 + row) * p.heads + it.head) * D;
#pragma unroll
            for (uint32_t c0 = 0; c0 < D; c0 += 32) {
                uint32_t r[32];
                if (nb > 0) {
                    tmem_ld_32x32(o_tmem + c0, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (uint32_t c = 0; c < 32; c++) r[c] = 0;
                }
                if (row_ok) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; i += 8) {
                        float f[8];
#pragma unroll
                        for (uint32_t e = 0; e < 8; e++) f[e] = __uint_as_float(r[i + e]) * inv;
                        *reinterpret_cast<uint4 *>(dst + c0 + i) =
                            make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                                       pack_bf16(f[6], f[7]));
                    }
                }
            }
            tc_fence_before_sync();  // the reads of O above precede this thread's next arrival on p_full
        }
        }  // items
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TS_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- head width 128: two query tiles per block ----------------------------------------------
//
// The softmax of one tile needs about as long as the tensor core needs for both of a block's products,
// so a block with a single tile leaves the tensor core idle half the time.  Here a work item is 256
// queries of one (sequence, head) as two tiles A and B with a softmax warp group each (warps 0-3 and
// 4-7); the MMA thread alternates  O_A += P_A V_j, S_A = Q_A K_{j+1}^T, O_B += P_B V_j, S_B = Q_B K_{j+1}^T,
// so tile A's softmax of block j+1 runs under tile B's products and the other way round.  K and V tiles
// are loaded once for both.  TMEM: S_A, S_B, O_A, O_B, 128 columns each.  A softmax thread reads its
// whole S row into registers once (the TMA / MMA warp group hands its spare registers over), and a
// key block that every row of the tile sees in full skips the mask selects.
//
// Blocks are persistent, one per SM.  Items are ranked heaviest first (later queries see more keys
// under a causal mask) and dealt to the blocks back and forth (0..G-1, G-1..0, ...), so that every
// block ends up with about the same number of key blocks.  Barrier phases run on across items.
struct Flash2Shape {
    static constexpr uint32_t BK = 128;
    static constexpr uint32_t chunk = 128 * 128;               // bytes of a 64-wide slice of a 128-row tile
    static constexpr uint32_t tile_bytes = 2 * chunk;          // a Q, K or V tile
    static constexpr uint32_t q_off = 0;                       // Q_A, Q_B
    static constexpr uint32_t k_off = 2 * tile_bytes;          // two stages
    static constexpr uint32_t v_off = k_off + 2 * tile_bytes;  // two stages
    static constexpr uint32_t bar_off = v_off + 2 * tile_bytes;
    static constexpr uint32_t total = bar_off + 256 + 1024;
};

constexpr uint32_t kThreads2 = 384;  // softmax A, softmax B, and a group of TMA + MMA + two idle warps

// What a work item covers; every role derives it from the item's rank in the same way.
struct Flash2Item {
    uint32_t head, kvh, q_begin, k_begin, k_len, past;
    uint32_t t0[2], rows[2], b0[2], b1[2], m0[2], m1[2];  // per tile: first query, rows, key blocks seen, seen in full
    uint32_t u0, u1;                                      // key blocks either tile sees
    bool has[2];
};

__device__ __forceinline__ void flash2_item(const FlashParams &p, uint32_t rank, Flash2Item &it) {
    constexpr uint32_t BK = Flash2Shape::BK;
    const uint32_t per = p.heads * p.seqs, pairs = (p.q_tiles + 1) / 2;
    const uint32_t pair = pairs - 1 - rank / per, rem = rank % per;
    const uint32_t seq = rem / p.heads;
    it.head = rem % p.heads;
    it.kvh = it.head / (p.heads / p.kv_heads);
    uint32_t q_len;
    if (p.cu_seqlens) {
        it.q_begin = it.k_begin = p.cu_seqlens[seq];
        q_len = it.k_len = p.cu_seqlens[seq + 1] - it.q_begin;
    } else {
        it.q_begin = seq * p.queries;
        q_len = p.queries;
        it.k_begin = seq * p.keys;
        it.k_len = p.keys;
    }
    it.past = it.k_len > q_len ? it.k_len - q_len : 0;
#pragma unroll
    for (uint32_t t = 0; t < 2; t++) {
        it.t0[t] = (pair * 2 + t) * kTile;
        it.rows[t] = it.t0[t] < q_len ? min(kTile, q_len - it.t0[t]) : 0;
        it.b0[t] = it.b1[t] = it.m0[t] = it.m1[t] = 0;
        if (it.rows[t]) {
            const uint32_t pos_first = it.past + it.t0[t], pos_last = pos_first + it.rows[t] - 1;
            const uint32_t lo = pos_first > p.back ? pos_first - p.back : 0;
            const uint32_t hi = min(it.k_len, sat_add(sat_add(pos_last, p.ahead), 1));
            if (hi > lo) {
                it.b0[t] = lo / BK;
                it.b1[t] = (hi + BK - 1) / BK;
                const uint32_t from_max = pos_last > p.back ? pos_last - p.back : 0;
                const uint32_t to_min = min(it.k_len, sat_add(sat_add(pos_first, p.ahead), 1));
                it.m0[t] = (from_max + BK - 1) / BK;
                it.m1[t] = to_min / BK;
            }
        }
        it.has[t] = it.b1[t] > it.b0[t];
    }
    it.u0 = it.has[0] && it.has[1] ? min(it.b0[0], it.b0[1]) : it.has[0] ? it.b0[0] : it.b0[1];
    it.u1 = max(it.b1[0], it.b1[1]);
}

// Rank of the item a block takes in round r: forwards in even rounds, backwards in odd ones.
__device__ __forceinline__ uint32_t flash2_rank(uint32_t r) {
    return r * gridDim.x + ((r & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
}

__global__ void __launch_bounds__(kThreads2, 1)
attend_flash2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const FlashParams p, const uint32_t items) {
    using Sh = Flash2Shape;
    constexpr uint32_t BK = Sh::BK, D = 128;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *smem_q = smem + Sh::q_off;
    unsigned char *smem_k = smem + Sh::k_off;
    unsigned char *smem_v = smem + Sh::v_off;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Sh::bar_off);
    uint64_t *q_full = bars;          // [1]
    uint64_t *k_full = bars + 1;      // [2] stages
    uint64_t *v_full = bars + 3;      // [2]
    uint64_t *k_empty = bars + 5;     // [2]
    uint64_t *v_empty = bars + 7;     // [2]
    uint64_t *s_full = bars + 9;      // [2] tiles
    uint64_t *p_full = bars + 11;     // [2]
    uint64_t *pv_done = bars + 13;    // [2]
    uint64_t *q_empty = bars + 15;    // [1]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 16);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 4);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (warp == 9) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= 8) {
        // The block was given 384 x 168 registers at launch; what this group gives back (88 each) is all
        // the softmax groups can take (40 each): asking for more would wait forever.
        setmaxnreg_dec<80>();
        if (warp == 8 && lane == 0) {
            // ---- TMA ----
            pdl_wait();
            bool ok = true;
            uint32_t kv_i = 0, n_item = 0;  // K/V tiles and items so far (phases run on across items)
            for (uint32_t r = 0; ok; r++) {
                const uint32_t rank = flash2_rank(r);
                if (rank >= items) break;
                Flash2Item it;
                flash2_item(p, rank, it);
                if (!(it.has[0] || it.has[1])) continue;
                // Q of the previous item is free once its MMAs are done.
                if (n_item > 0) ok = mbar_wait_or_abort(q_empty, (n_item - 1) & 1, abort_flag);
                if (!ok) break;
                mbar_expect_tx(q_full, (it.has[0] ? Sh::tile_bytes : 0) + (it.has[1] ? Sh::tile_bytes : 0));
#pragma unroll
                for (uint32_t t = 0; t < 2; t++)
                    if (it.has[t])
                        for (uint32_t c = 0; c < 2; c++)
                            tma_load_2d(smem_q + t * Sh::tile_bytes + c * Sh::chunk, &map_q, q_full,
                                        (int32_t)(it.head * D + c * 64), (int32_t)(it.q_begin + it.t0[t]));
                n_item++;
                for (uint32_t j = it.u0; j < it.u1 && ok; j++, kv_i++) {
                    const uint32_t s = kv_i & 1, ph = (kv_i >> 1) & 1;
                    const int32_t krow = (int32_t)(it.k_begin + j * BK);
                    ok = mbar_wait_or_abort(&k_empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&k_full[s], Sh::tile_bytes);
                    for (uint32_t c = 0; c < 2; c++)
                        tma_load_2d(smem_k + s * Sh::tile_bytes + c * Sh::chunk, &map_k, &k_full[s],
                                    (int32_t)(it.kvh * D + c * 64), krow);
                    ok = mbar_wait_or_abort(&v_empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&v_full[s], Sh::tile_bytes);
                    for (uint32_t c = 0; c < 2; c++)
                        tma_load_2d(smem_v + s * Sh::tile_bytes + c * Sh::chunk, &map_v, &v_full[s],
                                    (int32_t)(it.kvh * D + c * 64), krow);
                }
            }
            pdl_launch_dependents();
            // Copies in flight land before the MMAs that release their stages; wait for those releases.
            for (uint32_t back = 0; back < 2 && back < kv_i && ok; back++) {
                const uint32_t i = kv_i - 1 - back;
                ok = mbar_wait_or_abort(&k_empty[i & 1], (i >> 1) & 1, abort_flag) &&
                     mbar_wait_or_abort(&v_empty[i & 1], (i >> 1) & 1, abort_flag);
            }
        } else if (warp == 9 && lane == 0) {
            // ---- MMA ----
            const uint32_t idesc_qk = umma_idesc_bf16(kTile, BK, false, false);
            const uint32_t idesc_pv = umma_idesc_bf16(kTile, D, false, true);  // V is MN-major
            bool ok = true;
            uint32_t kv_i = 0, n_item = 0;
            uint32_t done[2] = {0, 0};  // products P V issued per tile, over all items
            for (uint32_t r = 0; ok; r++) {
                const uint32_t rank = flash2_rank(r);
                if (rank >= items) break;
                Flash2Item it;
                flash2_item(p, rank, it);
                if (!(it.has[0] || it.has[1])) continue;
                ok = mbar_wait_or_abort(q_full, n_item & 1, abort_flag);
                n_item++;
                bool fresh[2] = {true, true};  // O of the tile has not been written in this item yet
                auto uses = [&](uint32_t t, uint32_t j) { return j >= it.b0[t] && j < it.b1[t]; };
                auto qk = [&](uint32_t t, uint32_t s) {
                    const uint32_t d_tmem = tmem_base + t * BK;
#pragma unroll
                    for (uint32_t c = 0; c < 2; c++) {
                        const uint64_t da = umma_desc_k_sw128(smem_addr(smem_q + t * Sh::tile_bytes + c * Sh::chunk));
                        const uint64_t db = umma_desc_k_sw128(smem_addr(smem_k + s * Sh::tile_bytes + c * Sh::chunk));
#pragma unroll
                        for (uint32_t k16 = 0; k16 < 4; k16++)
                            umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc_qk, (c | k16) != 0);
                    }
                    umma_commit(&s_full[t]);
                };
                auto pv = [&](uint32_t t, uint32_t s) -> bool {
                    if (!mbar_wait_or_abort(&p_full[t], done[t] & 1, abort_flag)) return false;
                    tc_fence_after_sync();
                    const uint32_t p_tmem = tmem_base + t * BK;  // bf16 pairs: 16 keys = 8 columns
                    const uint32_t o_tmem = tmem_base + 2 * BK + t * D;
                    const uint32_t v_addr = smem_addr(smem_v + s * Sh::tile_bytes);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < BK / 16; k16++) {
                        const uint64_t db = umma_desc_mn_sw128(v_addr + k16 * 2048, Sh::chunk, 1024);
                        umma_bf16_ts(o_tmem, p_tmem + k16 * 8, db, idesc_pv, !fresh[t] || k16 != 0);
                    }
                    umma_commit(&pv_done[t]);
                    fresh[t] = false;
                    done[t]++;
                    return true;
                };
                if (ok) ok = mbar_wait_or_abort(&k_full[kv_i & 1], (kv_i >> 1) & 1, abort_flag);
                if (ok) {
                    tc_fence_after_sync();
                    if (uses(0, it.u0)) qk(0, kv_i & 1);
                    if (uses(1, it.u0)) qk(1, kv_i & 1);
                    umma_commit(&k_empty[kv_i & 1]);
                }
                for (uint32_t j = it.u0; j < it.u1 && ok; j++, kv_i++) {
                    const uint32_t s = kv_i & 1, ph = (kv_i >> 1) & 1, sn = (kv_i + 1) & 1;
                    const bool more = j + 1 < it.u1;
                    ok = mbar_wait_or_abort(&v_full[s], ph, abort_flag);
                    if (ok && more) ok = mbar_wait_or_abort(&k_full[sn], ((kv_i + 1) >> 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (uint32_t t = 0; t < 2; t++) {
                        if (uses(t, j)) {
                            ok = pv(t, s);
                            if (!ok) break;
                        }
                        if (more && uses(t, j + 1)) qk(t, sn);
                    }
                    if (!ok) break;
                    umma_commit(&v_empty[s]);
                    if (more) umma_commit(&k_empty[sn]);
                }
                if (ok) umma_commit(q_empty);
            }
        }
    } else {
        setmaxnreg_inc<208>();
        // ---- softmax + output: warp group = tile, thread = query row ----
        const uint32_t t = warp >> 2;
        const uint32_t q = warp & 3;
        const uint32_t row = q * 32 + lane;
        const uint32_t lane_base = (q * 32u) << 16;
        const uint32_t s_tmem = tmem_base + lane_base + t * BK;
        const uint32_t o_tmem = tmem_base + lane_base + 2 * BK + t * D;
        uint64_t *my_s_full = &s_full[t], *my_p_full = &p_full[t], *my_pv_done = &pv_done[t];
        uint32_t n_blk = 0;  // key blocks of this tile so far, over all items
        bool ok = true;
        for (uint32_t r = 0; ok; r++) {
            const uint32_t rank = flash2_rank(r);
            if (rank >= items) break;
            Flash2Item it;
            flash2_item(p, rank, it);
            // this tile's figures as scalars (indexing the arrays by t would put them in local memory)
            const uint32_t my_t0 = t ? it.t0[1] : it.t0[0], my_rows = t ? it.rows[1] : it.rows[0];
            const uint32_t my_b0 = t ? it.b0[1] : it.b0[0], my_b1 = t ? it.b1[1] : it.b1[0];
            const uint32_t my_m0 = t ? it.m0[1] : it.m0[0], my_m1 = t ? it.m1[1] : it.m1[0];
            if (my_rows == 0) continue;
            const bool row_ok = row < my_rows;
            const uint32_t pos = it.past + my_t0 + row;
            const uint32_t from = pos > p.back ? pos - p.back : 0;
            const uint32_t to = min(it.k_len, sat_add(sat_add(pos, p.ahead), 1));
            const uint32_t nb = my_b1 - my_b0;
            float m_use = -INFINITY;  // the maximum the probabilities are taken against (may lag the true one)
            float l_run = 0.0f;
            for (uint32_t b = 0; b < nb && ok; b++, n_blk++) {
                const uint32_t j = my_b0 + b;
                ok = mbar_wait_or_abort(my_s_full, n_blk & 1, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t rr[4][32];
#pragma unroll
                for (uint32_t c = 0; c < 4; c++) tmem_ld_32x32(s_tmem + c * 32, rr[c]);
                tmem_ld_wait();
                const bool solid = j >= my_m0 && j < my_m1;
                const uint32_t key0 = j * BK;
                const uint32_t c_from = from > key0 ? min(from - key0, BK) : 0;
                const uint32_t c_to = to > key0 ? min(to - key0, BK) : 0;
                // Eight independent running maxima: a single chain of 128 dependent fmax would cost more
                // than the exponentials.
                float mx[8];
#pragma unroll
                for (uint32_t i = 0; i < 8; i++) mx[i] = -INFINITY;
                if (solid) {
#pragma unroll
                    for (uint32_t c = 0; c < 128; c++) mx[c & 7] = fmaxf(mx[c & 7], __uint_as_float(rr[c >> 5][c & 31]));
                } else {
#pragma unroll
                    for (uint32_t c = 0; c < 128; c++) {
                        const float v = (c >= c_from && c < c_to) ? __uint_as_float(rr[c >> 5][c & 31]) : -INFINITY;
                        rr[c >> 5][c & 31] = __float_as_uint(v);  // masked keys: exp2(-inf) = 0 below
                        mx[c & 7] = fmaxf(mx[c & 7], v);
                    }
                }
                const float m_blk = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                          fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
                const float m_new = fmaxf(m_use, m_blk * p.scale_log2);
                // Rescale O and the running sum only when the maximum ran ahead by more than kRescaleStep:
                // probabilities stay below 2^kRescaleStep, and after the first blocks this is rare.
                float alpha = 1.0f;
                bool need = false;
                if (m_new > m_use + kRescaleStep || m_use == -INFINITY) {
                    need = l_run > 0.0f;
                    alpha = need ? ex2(m_use - m_new) : 1.0f;
                    m_use = m_new;
                }
                if (__any_sync(0xFFFFFFFFu, need)) {
                    // O is complete up to the previous block once its MMAs are done.
                    ok = mbar_wait_or_abort(my_pv_done, (n_blk - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (uint32_t c0 = 0; c0 < D; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld_32x32(o_tmem + c0, o);
                        tmem_ld_wait();
#pragma unroll
                        for (uint32_t c = 0; c < 32; c++) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                        tmem_st_32x32(o_tmem + c0, o);
                    }
                    l_run *= alpha;
                }
                const float neg_m = m_use == -INFINITY ? 0.0f : -m_use;
                float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (uint32_t c0 = 0; c0 < 4; c0++) {
                    uint32_t packed[16];
#pragma unroll
                    for (uint32_t c = 0; c < 32; c += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(rr[c0][c]), p.scale_log2, neg_m));
                        const float p1 = ex2(fmaf(__uint_as_float(rr[c0][c + 1]), p.scale_log2, neg_m));
                        ls[(c >> 1) & 1] += p0;
                        ls[2 + ((c >> 1) & 1)] += p1;
                        packed[c >> 1] = pack_bf16(p0, p1);
                    }
                    tmem_st_32x16(s_tmem + c0 * 16, packed);
                }
                l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(my_p_full);
            }
            if (ok && nb > 0) {
                ok = mbar_wait_or_abort(my_pv_done, (n_blk - 1) & 1, abort_flag);
                if (ok) tc_fence_after_sync();
            }
            if (!ok) break;
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            uint16_t *dst = p.out + ((size_t)(it.q_begin + my_t0 + row) * p.heads + it.head) * D;
#pragma unroll
            for (uint32_t c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                if (nb > 0) {
                    tmem_ld_32x32(o_tmem + c0, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (uint32_t c = 0; c < 32; c++) o[c] = 0;
                }
                if (row_ok) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; i += 8) {
                        float f[8];
#pragma unroll
                        for (uint32_t e = 0; e < 8; e++) f[e] = __uint_as_float(o[i + e]) * inv;
                        *reinterpret_cast<uint4 *>(dst + c0 + i) =
                            make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                                       pack_bf16(f[6], f[7]));
                    }
                }
            }
            // The reads of O above are ordered before this thread's next arrival on p_full, which is what
            // lets the tensor core overwrite O for the next item.
            tc_fence_before_sync();
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TS_ERR_TIMEOUT);
    if (warp == 9) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

__device__ int g_flash_status = 0;

}  // namespace

int flash_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_flash_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_flash_status, &zero, sizeof(int));
    return v;
}

bool flash_supports(uint32_t width) { return width == 128 || width == 256; }

template <uint32_t D>
static int launch_flash(const void *q, const void *k, const void *v, const FlashParams &p, uint32_t total_q,
                        uint32_t total_k, cudaStream_t stream) {
    using Sh = FlashShape<D>;
    CUtensorMap map_q, map_k, map_v;
    int rc = make_tensor_map_2d(&map_q, q, total_q, (uint64_t)p.heads * D, (uint64_t)p.heads * D, kTile, 64);
    if (rc != TS_OK) return rc;
    rc = make_tensor_map_2d(&map_k, k, total_k, (uint64_t)p.kv_heads * D, (uint64_t)p.kv_heads * D, Sh::BK, 64);
    if (rc != TS_OK) return rc;
    rc = make_tensor_map_2d(&map_v, v, total_k, (uint64_t)p.kv_heads * D, (uint64_t)p.kv_heads * D, Sh::BK, 64);
    if (rc != TS_OK) return rc;
    static OncePerDevice configured;
    if (configured.needs()) {
        TS_CUDA(cudaFuncSetAttribute(attend_flash_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Sh::total));
        TS_CUDA(cudaFuncSetAttribute(attend_flash2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Flash2Shape::total));
        configured.done();
    }
    cudaError_t e;
    const uint64_t items = (uint64_t)((p.q_tiles + 1) / 2) * p.heads * p.seqs;
    if (D == 128 && p.q_tiles > 1 && items < 0x7FFFFFFFull)  // two query tiles per item, persistent blocks
        e = launch(attend_flash2_kernel, dim3((uint32_t)std::min<uint64_t>(items, (uint64_t)sm_count())), dim3(kThreads2),
                   Flash2Shape::total, stream, pdl_enabled(), map_q, map_k, map_v, p, (uint32_t)items);
    else
    {
        const uint64_t tiles = (uint64_t)p.q_tiles * p.heads * p.seqs;
        if (tiles >= 0x7FFFFFFFull) return fail(TS_ERR_BAD_INPUT, "attend: %llu query tiles are too many", (unsigned long long)tiles);
        e = launch(attend_flash_kernel<D>, dim3((uint32_t)std::min<uint64_t>(tiles, (uint64_t)sm_count())), dim3(kThreads),
                   Sh::total, stream, pdl_enabled(), map_q, map_k, map_v, p, (uint32_t)tiles);
    }
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of attend_flash failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

// q [total_q, heads, width], k/v [total_k, kv_heads, width], out like q (rows packed sequence after sequence).
int attend_flash(const void *q, const void *k, const void *v, void *out, const uint32_t *cu_seqlens, uint32_t seqs,
                 uint32_t queries, uint32_t keys, uint32_t total_q, uint32_t total_k, uint32_t heads, uint32_t kv_heads,
                 uint32_t width, uint32_t back, uint32_t ahead, float scale, cudaStream_t stream) {
    FlashParams p = {};
    p.out = (uint16_t *)out;
    p.cu_seqlens = cu_seqlens;
    p.seqs = seqs;
    p.queries = queries;
    p.keys = keys;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.back = back;
    p.ahead = ahead;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.q_tiles = ceil_div(queries, kTile);
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_flash_status));
    p.status = status;
    if (width == 128) return launch_flash<128>(q, k, v, p, total_q, total_k, stream);
    return launch_flash<256>(q, k, v, p, total_q, total_k, stream);
}

}  // namespace ts
