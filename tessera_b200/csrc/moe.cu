// Routed experts: the reference's per-row `picked` matmuls (engine/rules/linear/src/picked.rs:28-60;
// engine/ir/interp/src/cpu.rs:89-105) and the gate-weighted `mix` (cpu.rs:449-473) of its MoE block
// (engine/models/src/decoder.rs:70-84), regrouped by expert so that each expert's weights stream from
// HBM once per batch tile instead of once per row.
//
//   1. moe_plan_kernel     integer work, bit-exact on every run: counts picks per local expert, orders
//                          the picks by expert (stable in pick index), records each pick's place, and
//                          lays out the batch tiles (BN rows) every expert needs.
//   2. moe_gather_kernel   x rows into expert order (pick i reads row i / repeat, the `repeat` of
//                          `picked`).
//   3. moe_grouped_kernel  tcgen05 grouped linear over work items (expert, batch tile, weight tile):
//                          weights on the 128 TMEM lanes, the expert's batch tile on BN columns, both
//                          operands streamed by TMA; blocks are persistent over an item list whose
//                          length lives on the device (no host read of the routing).  Epilogue SwiGLU
//                          (64 gate rows + their 64 up rows per tile) for the first linear, plain f32
//                          for the second.
//   4. moe_scatter_mix     out[pick] rows back in pick order, or the gate-weighted sum over a row's
//                          picks in pick order p = 0..top-1 (the checker's order).
#include "ts_common.cuh"
#include "ts_ptx.cuh"

namespace ts {
namespace {

using namespace ptx;

constexpr uint32_t kBN = 32;        // batch rows per tile
constexpr uint32_t kRows = 128;     // weight rows per tile
constexpr uint32_t kBlockK = 64;
constexpr uint32_t kABytes = kRows * kBlockK * 2;
constexpr uint32_t kBBytes = kBN * kBlockK * 2;
constexpr uint32_t kStages = 8;
constexpr uint32_t kEpiWarps = 4;
constexpr uint32_t kThreads = (2 + kEpiWarps) * 32;
constexpr uint32_t kNone = 0xFFFFFFFFu;

// ---- 1. plan ------------------------------------------------------------------------------------
// One block.  ids [picks]; outputs: order [picks] (pick indices by expert, stable), place [picks]
// (where pick i sits in `order`, or kNone for an expert outside [first, first + experts)), offsets
// [experts + 1], btiles [experts + 1] (prefix sum of ceil(count / kBN)).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const uint32_t *ids, uint32_t *order, uint32_t *place,
                                                        uint32_t *offsets, uint32_t *btiles, uint32_t picks,
                                                        uint32_t experts, uint32_t first) {
    extern __shared__ uint32_t sm[];
    uint32_t *count = sm;                 // [experts]
    uint32_t *start = sm + experts;       // [experts + 1]
    pdl_wait();
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < picks; i += blockDim.x) {
        const uint32_t id = ids[i];
        if (id >= first && id - first < experts) atomicAdd(&count[id - first], 1u);  // integer: order-free
        else place[i] = kNone;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0, tiles = 0;
        for (uint32_t e = 0; e < experts; e++) {
            start[e] = run;
            offsets[e] = run;
            btiles[e] = tiles;
            run += count[e];
            tiles += (count[e] + kBN - 1) / kBN;
        }
        start[experts] = run;
        offsets[experts] = run;
        btiles[experts] = tiles;
    }
    __syncthreads();
    // Stable placement: a warp per expert walks the picks in order.
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (uint32_t e = warp; e < experts; e += warps) {
        uint32_t at = start[e];
        if (count[e] == 0) continue;
        for (uint32_t i0 = 0; i0 < picks; i0 += 32) {
            const uint32_t i = i0 + lane;
            const bool mine = i < picks && ids[i] == first + e;
            const uint32_t mask = __ballot_sync(0xFFFFFFFFu, mine);
            if (mine) {
                const uint32_t pos = at + __popc(mask & ((1u << lane) - 1u));
                order[pos] = i;
                place[i] = pos;
            }
            at += __popc(mask);
        }
    }
    pdl_launch_dependents();
}

// ---- 2. gather ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) moe_gather_kernel(const uint16_t *x, const uint32_t *order,
                                                         const uint32_t *offsets, uint16_t *xp, uint32_t experts,
                                                         uint32_t width, uint32_t repeat) {
    pdl_wait();
    const uint32_t i = blockIdx.x;
    if (i >= offsets[experts]) return;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)(order[i] / repeat) * width);
    uint4 *dst = reinterpret_cast<uint4 *>(xp + (size_t)i * width);
    for (uint32_t j = threadIdx.x; j < width / 8; j += blockDim.x) dst[j] = src[j];
    pdl_launch_dependents();
}

// ---- 3. grouped linear ----------------------------------------------------------------------------
struct GroupedParams {
    const uint32_t *offsets, *btiles;  // [experts + 1]
    uint32_t experts, n, k;            // per expert: weight [n, k]
    uint32_t w_stride;                 // weight rows from one expert to the next (n, or more inside a wider table)
    uint32_t tiles;                    // weight tiles per expert: n / 128, or (n / 2) / 64 when gated
    uint32_t gated;
    void *out;                         // gated: bf16 [picks, n / 2]; plain: f32 [picks, n]
    int *status;
};

struct GroupedSmem {
    static constexpr uint32_t a_off = 0;
    static constexpr uint32_t b_off = kStages * kABytes;
    static constexpr uint32_t recv_off = b_off + kStages * kBBytes;
    static constexpr uint32_t bar_off = recv_off + kRows * (kBN + 4) * 4;
    static constexpr uint32_t total = bar_off + 256 + 1024;
};

// Item i of the launch: batch tile gb = i / tiles (over all experts), weight tile t = i % tiles.
struct Item {
    uint32_t expert, row0, rows, tile;
};

__device__ __forceinline__ Item decode_item(const GroupedParams &p, uint32_t i) {
    const uint32_t gb = i / p.tiles;
    uint32_t lo = 0, hi = p.experts;  // last expert with btiles[e] <= gb
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (p.btiles[mid] <= gb) lo = mid;
        else hi = mid;
    }
    Item it;
    it.expert = lo;
    const uint32_t b = gb - p.btiles[lo];
    it.row0 = p.offsets[lo] + b * kBN;
    it.rows = min(kBN, p.offsets[lo + 1] - it.row0);
    it.tile = i % p.tiles;
    return it;
}

__global__ void __launch_bounds__(kThreads, 1)
moe_grouped_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const GroupedParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *smem_a = smem + GroupedSmem::a_off;
    unsigned char *smem_b = smem + GroupedSmem::b_off;
    float *recv = reinterpret_cast<float *>(smem + GroupedSmem::recv_off);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + GroupedSmem::bar_off);
    uint64_t *empty = full + 8;
    uint64_t *acc_full = empty + 8;   // [2]
    uint64_t *acc_empty = acc_full + 2;
    uint64_t *recv_full = acc_empty + 2;
    uint64_t *recv_free = recv_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(recv_free + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    constexpr uint32_t kTmemCols = 2 * kBN;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (uint32_t s = 0; s < 2; s++) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kEpiWarps);
        }
        mbar_init(recv_full, kEpiWarps);
        mbar_init(recv_free, kEpiWarps);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // the plan and the gathered rows come from the upstream kernels
    const uint32_t items = p.btiles[p.experts] * p.tiles;
    const uint32_t kbs = p.k / kBlockK;
    const uint32_t half_n = p.n / 2;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t i = blockIdx.x; i < items && ok; i += gridDim.x) {
                const Item item = decode_item(p, i);
                const uint32_t wrow = item.expert * p.w_stride;  // the expert's first weight row
                for (uint32_t kb = 0; kb < kbs; kb++, it++) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    ok = mbar_wait_or_abort(&empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    const int32_t kx = (int32_t)(kb * kBlockK);
                    mbar_expect_tx(&full[s], kABytes + kBBytes);
                    unsigned char *dst = smem_a + s * kABytes;
                    if (p.gated) {
                        tma_load_2d(dst, &map_w, &full[s], kx, (int32_t)(wrow + item.tile * 64));
                        tma_load_2d(dst + kABytes / 2, &map_w, &full[s], kx, (int32_t)(wrow + half_n + item.tile * 64));
                    } else {
                        tma_load_2d(dst, &map_w, &full[s], kx, (int32_t)(wrow + item.tile * kRows));
                    }
                    tma_load_2d(smem_b + s * kBBytes, &map_x, &full[s], kx, (int32_t)item.row0);
                }
            }
            pdl_launch_dependents();
            if (ok)
                for (uint32_t back = 0; back < kStages && back < it; back++) {
                    const uint32_t j = it - 1 - back;
                    if (!mbar_wait_or_abort(&empty[j % kStages], (j / kStages) & 1, abort_flag)) break;
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(kRows, kBN);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (uint32_t i = blockIdx.x; i < items && ok; i += gridDim.x, acc_it++) {
                const uint32_t as = acc_it & 1, aph = (acc_it >> 1) & 1;
                ok = mbar_wait_or_abort(&acc_empty[as], aph ^ 1, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * kBN;
                for (uint32_t kb = 0; kb < kbs; kb++, it++) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    ok = mbar_wait_or_abort(&full[s], ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t da = umma_desc_k_sw128(smem_addr(smem_a + s * kABytes));
                    const uint64_t db = umma_desc_k_sw128(smem_addr(smem_b + s * kBBytes));
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kBlockK / 16; k16++)
                        umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[as]);
            }
        }
    } else {
        const uint32_t q = warp & 3;
        const uint32_t row = q * 32 + lane;  // weight row of the tile = TMEM lane
        constexpr uint32_t rs = kBN + 4;
        uint32_t acc_it = 0;
        bool ok = true;
        for (uint32_t i = blockIdx.x; i < items && ok; i += gridDim.x, acc_it++) {
            const Item item = decode_item(p, i);
            const uint32_t as = acc_it & 1, aph = (acc_it >> 1) & 1;
            ok = mbar_wait_or_abort(&acc_full[as], aph, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + as * kBN, r);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
            if (!p.gated) {
                // Column c of the tile is pick row0 + c; consecutive lanes are consecutive outputs n.
                const uint32_t n_idx = item.tile * kRows + row;
                float *out = reinterpret_cast<float *>(p.out) + (size_t)item.row0 * p.n + n_idx;
#pragma unroll
                for (uint32_t c = 0; c < kBN; c++, out += p.n)
                    if (c < item.rows) *out = __uint_as_float(r[c]);
                continue;
            }
            // Gated: lanes 0-63 hold gate rows, 64-127 the matching up rows; pair them through smem.
            if (acc_it > 0) {
                ok = mbar_wait_or_abort(recv_free, (acc_it - 1) & 1, abort_flag);
                if (!ok) break;
            }
#pragma unroll
            for (uint32_t c = 0; c < kBN; c += 4)
                *reinterpret_cast<float4 *>(recv + row * rs + c) =
                    make_float4(__uint_as_float(r[c]), __uint_as_float(r[c + 1]), __uint_as_float(r[c + 2]),
                                __uint_as_float(r[c + 3]));
            __syncwarp();
            if (lane == 0) mbar_arrive(recv_full);
            ok = mbar_wait_or_abort(recv_full, acc_it & 1, abort_flag);
            if (!ok) break;
            // 128 threads finish 64 outputs x kBN picks: thread (j = row % 64, half = row / 64) takes
            // every second pick.
            {
                const uint32_t j = row & 63, half = row >> 6;
                const uint32_t n_idx = item.tile * 64 + j;
                uint16_t *out = reinterpret_cast<uint16_t *>(p.out);
                for (uint32_t c = half; c < item.rows; c += 2) {
                    const float g = recv[j * rs + c], u = recv[(j + 64) * rs + c];
                    out[(size_t)(item.row0 + c) * half_n + n_idx] = bf16_bits(silu(g) * u);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(recv_free);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TS_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- 4. back to pick order, or the gate-weighted sum -------------------------------------------
// mix == 0: out[i, :] = y[place[i], :] (zeros for picks of experts held elsewhere), i over picks.
// mix == 1: out[r, :] = sum_p gates[r, p] * y[place[r * top + p], :] in pick order (+ add[r, :]).
__global__ void __launch_bounds__(256) moe_scatter_mix_kernel(const float *y, const uint32_t *place, const float *gates,
                                                              const float *add, float *out, uint32_t width,
                                                              uint32_t top, int mix) {
    __shared__ uint32_t s_at[32];
    __shared__ float s_gate[32];
    pdl_wait();
    const uint32_t r = blockIdx.x;
    const bool vec = (((uintptr_t)y | (uintptr_t)out | (uintptr_t)add) & 15) == 0 && width % 4 == 0;
    if (mix && top <= 32 && vec) {
        // The row's picks once into shared memory, then 16-byte columns: the same products and sums, in pick
        // order, as the scalar loop below.
        if (threadIdx.x < top) {
            s_at[threadIdx.x] = place ? place[r * top + threadIdx.x] : r * top + threadIdx.x;
            s_gate[threadIdx.x] = gates[r * top + threadIdx.x];
        }
        __syncthreads();
        for (uint32_t j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (uint32_t t = 0; t < top; t++) {
                const uint32_t at = s_at[t];
                const float g = s_gate[t];
                const float4 v = at == kNone ? make_float4(0.0f, 0.0f, 0.0f, 0.0f)
                                             : *reinterpret_cast<const float4 *>(y + (size_t)at * width + j);
                acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, g));
                acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, g));
                acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, g));
                acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, g));
            }
            if (add) {
                const float4 a = *reinterpret_cast<const float4 *>(add + (size_t)r * width + j);
                acc.x = __fadd_rn(acc.x, a.x);
                acc.y = __fadd_rn(acc.y, a.y);
                acc.z = __fadd_rn(acc.z, a.z);
                acc.w = __fadd_rn(acc.w, a.w);
            }
            *reinterpret_cast<float4 *>(out + (size_t)r * width + j) = acc;
        }
        pdl_launch_dependents();
        return;
    }
    for (uint32_t j = threadIdx.x; j < width; j += blockDim.x) {
        if (!mix) {
            const uint32_t at = place[r];
            out[(size_t)r * width + j] = at == kNone ? 0.0f : y[(size_t)at * width + j];
        } else {
            float acc = 0.0f;
            for (uint32_t t = 0; t < top; t++) {
                const uint32_t at = place ? place[r * top + t] : r * top + t;
                const float v = at == kNone ? 0.0f : y[(size_t)at * width + j];
                acc = __fadd_rn(acc, __fmul_rn(v, gates[r * top + t]));
            }
            if (add) acc = __fadd_rn(acc, add[(size_t)r * width + j]);
            out[(size_t)r * width + j] = acc;
        }
    }
    pdl_launch_dependents();
}

__device__ int g_moe_status = 0;

struct MoeWorkspace {
    uint32_t *order, *place, *offsets, *btiles;
    uint16_t *xp, *act;
    float *y;
    size_t total;
};

MoeWorkspace carve(void *base, uint32_t picks, uint32_t experts, uint32_t hidden, uint32_t ffn, uint32_t y_cols = 0) {
    MoeWorkspace w;
    size_t at = 0;
    auto take = [&](size_t bytes) {
        size_t here = at;
        at += align_up(bytes, 256);
        return (char *)base + here;
    };
    w.order = (uint32_t *)take((size_t)picks * 4);
    w.place = (uint32_t *)take((size_t)picks * 4);
    w.offsets = (uint32_t *)take((size_t)(experts + 1) * 4);
    w.btiles = (uint32_t *)take((size_t)(experts + 1) * 4);
    // TMA boxes of kBN rows may read past the last pick: pad the row buffers by one tile.
    w.xp = (uint16_t *)take((size_t)(picks + kBN) * hidden * 2);
    w.act = (uint16_t *)take((size_t)(picks + kBN) * ffn * 2);
    w.y = (float *)take((size_t)picks * (y_cols ? y_cols : hidden) * 4);
    w.total = at;
    return w;
}

int launch_grouped(const void *w, const void *x, void *out, const MoeWorkspace &ws, uint32_t picks, uint32_t experts,
                   uint32_t n, uint32_t k, bool gated, cudaStream_t stream, uint32_t w_stride = 0) {
    CUtensorMap map_w, map_x;
    if (w_stride == 0) w_stride = n;
    int rc = make_tensor_map_2d(&map_w, w, (uint64_t)(experts - 1) * w_stride + n, k, k, gated ? 64 : kRows, kBlockK);
    if (rc != TS_OK) return rc;
    rc = make_tensor_map_2d(&map_x, x, (uint64_t)picks + kBN, k, k, kBN, kBlockK);
    if (rc != TS_OK) return rc;
    GroupedParams p = {};
    p.offsets = ws.offsets;
    p.btiles = ws.btiles;
    p.experts = experts;
    p.n = n;
    p.k = k;
    p.w_stride = w_stride;
    p.tiles = gated ? (n / 2) / 64 : n / kRows;
    p.gated = gated;
    p.out = out;
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_moe_status));
    p.status = status;
    static OncePerDevice configured;
    if (configured.needs()) {
        TS_CUDA(cudaFuncSetAttribute(moe_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GroupedSmem::total));
        configured.done();
    }
    cudaError_t e = launch(moe_grouped_kernel, dim3(sm_count()), dim3(kThreads), GroupedSmem::total, stream,
                           pdl_enabled(), map_w, map_x, p);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of moe_grouped failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace

int moe_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_moe_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_moe_status, &zero, sizeof(int));
    return v;
}

size_t moe_workspace_bytes(uint32_t picks, uint32_t experts, uint32_t hidden, uint32_t ffn) {
    return carve(nullptr, picks, experts, hidden, ffn).total;
}

int moe_permutation(const uint32_t *ids, uint32_t *order, uint32_t *place, uint32_t *offsets, uint32_t *btiles,
                    uint32_t picks, uint32_t experts, uint32_t first, cudaStream_t stream) {
    const size_t smem = (size_t)(2 * experts + 1) * 4;
    cudaError_t e = launch(moe_plan_kernel, dim3(1), dim3(1024), smem, stream, pdl_enabled(), ids, order, place, offsets,
                           btiles, picks, experts, first);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of moe_plan failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

// out [picks, hidden] f32 (mix == 0) or [picks / top, hidden] f32 (mix == 1).
int moe_experts(const void *x, const uint32_t *ids, const float *gates, const float *add, const void *w_in,
                const void *w_out, float *out, uint32_t picks, uint32_t repeat, uint32_t top, int mix, uint32_t experts,
                uint32_t first, uint32_t hidden, uint32_t ffn, void *workspace, size_t workspace_bytes,
                cudaStream_t stream) {
    const size_t need = moe_workspace_bytes(picks, experts, hidden, ffn);
    TS_REQUIRE(workspace && workspace_bytes >= need, "moe: workspace of %zu bytes is smaller than the %zu needed",
               workspace_bytes, need);
    MoeWorkspace ws = carve(workspace, picks, experts, hidden, ffn);
    int rc = moe_permutation(ids, ws.order, ws.place, ws.offsets, ws.btiles, picks, experts, first, stream);
    if (rc != TS_OK) return rc;
    cudaError_t e = launch(moe_gather_kernel, dim3(picks), dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)x,
                           (const uint32_t *)ws.order, (const uint32_t *)ws.offsets, ws.xp, experts, hidden, repeat);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of moe_gather failed: %s", cudaGetErrorString(e));
    rc = launch_grouped(w_in, ws.xp, ws.act, ws, picks, experts, 2 * ffn, hidden, true, stream);
    if (rc != TS_OK) return rc;
    rc = launch_grouped(w_out, ws.act, ws.y, ws, picks, experts, hidden, ffn, false, stream);
    if (rc != TS_OK) return rc;
    const uint32_t out_rows = mix ? picks / top : picks;
    e = launch(moe_scatter_mix_kernel, dim3(out_rows), dim3(256), 0, stream, pdl_enabled(), (const float *)ws.y,
               (const uint32_t *)ws.place, gates, add, out, hidden, top, mix);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of moe_scatter_mix failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

// `picked` for sizes the grouped kernel's tiles do not take (n off the 128 grid, k off the 64 grid: the reference's
// own case runs 4 matrices of 64 x 32, engine/rules/linear/tests/lanes_test.rs:112-149).  A warp per output
// element, lanes stride k in ascending order, a fixed butterfly: the same bits on every run and in any batch.
__global__ void __launch_bounds__(256) picked_plain_kernel(const uint16_t *x, const uint16_t *w, const uint32_t *ids,
                                                           float *out, uint32_t rows, uint32_t n, uint32_t k,
                                                           uint32_t count, uint32_t stride, uint32_t offset,
                                                           uint32_t repeat, uint32_t first) {
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const size_t total = (size_t)rows * n, warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t i = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < total; i += warps) {
        const uint32_t row = (uint32_t)(i / n), col = (uint32_t)(i % n);
        const uint32_t id = ids[row];
        float sum = 0.0f;
        if (id >= first && id - first < count) {   // this rank's matrices start at `first`
            const uint16_t *xr = x + (size_t)(row / repeat) * k;
            const uint16_t *wr = w + ((size_t)(id - first) * stride + offset + col) * k;
            for (uint32_t j = lane; j < k; j += 32)
                sum = fmaf(__uint_as_float((uint32_t)xr[j] << 16), __uint_as_float((uint32_t)wr[j] << 16), sum);
            sum = warp_sum(sum);
        }
        if (lane == 0) out[i] = sum;
    }
    pdl_launch_dependents();
}

// The reference's `picked` launch on its own: out[i, :] = x[i / repeat, :] . w[(ids[i] - first) * stride + offset + col, :],
// zeros where ids[i] falls outside [first, first + count).  Rows are grouped by matrix so that each matrix
// streams once per 32 rows that picked it.
size_t picked_workspace_bytes(uint32_t rows, uint32_t n, uint32_t k, uint32_t count) {
    if (n % kRows != 0 || k % kBlockK != 0) return 0;  // the plain kernel needs none
    return carve(nullptr, rows, count, k, 0, n).total;
}

int picked(const void *x, const void *w, const uint32_t *ids, float *out, uint32_t rows, uint32_t n, uint32_t k,
           uint32_t count, uint32_t stride, uint32_t offset, uint32_t repeat, uint32_t first, void *workspace,
           size_t workspace_bytes, cudaStream_t stream) {
    TS_REQUIRE(count >= 1 && repeat >= 1 && stride >= offset + n, "picked: stride %u does not hold offset %u + n %u",
               stride, offset, n);
    if (rows == 0 || n == 0) return TS_OK;
    if (n % kRows != 0 || k % kBlockK != 0) {
        TS_REQUIRE(k > 0, "picked: k is zero");
        const size_t total = (size_t)rows * n;
        const uint32_t blocks = (uint32_t)std::min<size_t>((total + 7) / 8, (size_t)sm_count() * 16);
        cudaError_t pe = launch(picked_plain_kernel, dim3(blocks ? blocks : 1), dim3(256), 0, stream, pdl_enabled(),
                                (const uint16_t *)x, (const uint16_t *)w, ids, out, rows, n, k, count, stride, offset, repeat,
                                first);
        if (pe != cudaSuccess) return fail(TS_ERR_CUDA, "launch of picked (plain) failed: %s", cudaGetErrorString(pe));
        return TS_OK;
    }
    const size_t need = picked_workspace_bytes(rows, n, k, count);
    TS_REQUIRE(workspace && workspace_bytes >= need, "picked: workspace of %zu bytes is smaller than the %zu needed",
               workspace_bytes, need);
    MoeWorkspace ws = carve(workspace, rows, count, k, 0, n);  // no inner rows; y holds n columns
    int rc = moe_permutation(ids, ws.order, ws.place, ws.offsets, ws.btiles, rows, count, first, stream);
    if (rc != TS_OK) return rc;
    cudaError_t e = launch(moe_gather_kernel, dim3(rows), dim3(128), 0, stream, pdl_enabled(), (const uint16_t *)x,
                           (const uint32_t *)ws.order, (const uint32_t *)ws.offsets, ws.xp, count, k, repeat);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of moe_gather failed: %s", cudaGetErrorString(e));
    const uint16_t *w0 = (const uint16_t *)w + (size_t)offset * k;
    rc = launch_grouped(w0, ws.xp, ws.y, ws, rows, count, n, k, false, stream, stride);
    if (rc != TS_OK) return rc;
    e = launch(moe_scatter_mix_kernel, dim3(rows), dim3(256), 0, stream, pdl_enabled(), (const float *)ws.y,
               (const uint32_t *)ws.place, (const float *)nullptr, (const float *)nullptr, out, n, 1u, 0);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of moe_scatter_mix failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

// y_picks [rows * top, width] already in pick order: out[r] = sum_p gates[r, p] * y_picks[r * top + p] (+ add).
int moe_mix(const float *y_picks, const float *gates, const float *add, float *out, uint32_t rows, uint32_t top,
            uint32_t width, cudaStream_t stream) {
    if (rows == 0) return TS_OK;
    cudaError_t e = launch(moe_scatter_mix_kernel, dim3(rows), dim3(256), 0, stream, pdl_enabled(), y_picks,
                           (const uint32_t *)nullptr, gates, add, out, width, top, 1);
    if (e != cudaSuccess) return fail(TS_ERR_CUDA, "launch of moe_mix failed: %s", cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
