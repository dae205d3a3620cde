// Prefill-sized linear on two-SM tensor-core pairs: out[m, n] = sum_k x[m, k] * w[n, k] (+ epilogue).
//
// A 128 x 256 tile per SM needs (128 + 256) x 64 x 2 bytes of operands per 64-deep k block, 85 flop
// per byte of shared-memory fill, and at the tensor rate that is more than the L2 can feed 148 SMs.
// Here two blocks of a cluster (two SMs) share one 256 x 256 tile: block r loads rows
// [128 r, 128 r + 128) of x and rows [128 r, 128 r + 128) of the tile's w (half of B each), the leader's
// single MMA thread issues tcgen05.mma.cta_group::2 (M = 256, N = 256) that reads both halves of both
// operands out of the two shared memories, and each block ends up with its 128 rows of the
// accumulator in its own TMEM: 128 flop per byte, one and a half times less traffic per SM.  No
// multicast copies: each block fetches what it holds.
//
// Per block: warp 0 = TMA producer (both blocks; the bytes of both are credited to the leader's
// barrier), warp 1 = MMA (leader issues; both allocate TMEM as a pair), warps 2-5 = epilogue out of
// the block's own TMEM.  The tensor core reports finished stages and accumulators to the barriers of
// both blocks (tcgen05.commit to the pair).  Six
// 32 KB stages, two 256-column accumulator stages.  Pairs are persistent over tiles.  Gated epilogues:
// the leader's B half holds 128 gate rows, the partner's their up rows.
//
// Stands in for the reference's `tiled*` rules at prefill sizes (engine/rules/linear/src/tiled.rs:295-446)
// with their fused epilogue chain (engine/plan/lower/src/sites/matmul.rs:148-176).
#include <algorithm>

#include "ts_common.cuh"
#include "ts_kernels.cuh"
#include "ts_ptx.cuh"

namespace ts {
namespace {

using namespace ptx;

constexpr uint32_t kRowsPerBlock = 128;  // x rows per block = TMEM lanes
constexpr uint32_t kTileM = 256;         // per pair
constexpr uint32_t kTileN = 256;
constexpr uint32_t kBlockK = 64;
constexpr uint32_t kStages = 6;
constexpr uint32_t kAccStages = 2;
constexpr uint32_t kThreads = 192;
constexpr uint32_t kHalfBytes = 128 * kBlockK * 2;  // a 128-row operand half of one k block
constexpr uint32_t kStageBytes = 2 * kHalfBytes;
constexpr uint32_t kSmemTotal = kStages * kStageBytes + 256 + 1024;

struct PairParams {
    uint32_t m, n, k, kb_total, tiles_i, tiles_j;
    uint32_t gated;
    int epilogue, out_dtype;
    float scale;
    const float *a0;
    void *out;
    int *status;
    // The residual stream's RMS norms folded into the linears on either side (NULL / 0: off), as in the
    // streamed linear: in, x holds bf16(row * gain) and row_ss [m, row_parts] partial sums of squares of the rows,
    // and the output rows get the factor 1/sqrt(sum/k + row_eps); out (f32 output), ss_out [m, tiles_j] takes the
    // sum of squares of each finished row over the tile's columns and xs_out [m, n] = bf16(out * xs_gain[n]).
    const float *row_ss;
    uint32_t row_parts;
    float row_eps;
    float *ss_out;
    uint16_t *xs_out;
    const float *xs_gain;
};

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag) {
    uint64_t start = 0;
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
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

__global__ void __launch_bounds__(kThreads, 1)
linear_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   const PairParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);  // [kStages]  (the leader's are used)
    uint64_t *empty = full + kStages;                                            // [kStages]  per block
    uint64_t *acc_full = empty + kStages;                                        // [2]        per block
    uint64_t *acc_empty = acc_full + kAccStages;                                 // [2]        (the leader's are used)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + kAccStages);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint32_t tiles = p.tiles_i * p.tiles_j;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);   // the leader's producer announces the bytes of both blocks
            mbar_init(&empty[s], 1);  // one commit per use
        }
        for (uint32_t s = 0; s < kAccStages; s++) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 8);  // four epilogue warps in each block
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();  // both blocks' barriers exist before either signals the other
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer (both blocks) ----
        if (lane == 0) {
            pdl_wait();
            bool ok = true;
            uint32_t it = 0;
            for (uint32_t tile = pair; tile < tiles && ok; tile += pairs) {
                const uint32_t ti = tile / p.tiles_j, tj = tile % p.tiles_j;
                const int32_t x_row = (int32_t)(ti * kTileM + rank * kRowsPerBlock);
                const int32_t w_row = p.gated ? (int32_t)((rank ? p.n / 2 : 0) + tj * 128)
                                              : (int32_t)(tj * kTileN + rank * 128);
                for (uint32_t kb = 0; kb < p.kb_total; kb++, it++) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    ok = wait_bounded(&empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * kStageBytes);
                    const uint32_t leader_full = map_to_rank(smem_addr(&full[s]), 0);
                    unsigned char *dst = smem + s * kStageBytes;
                    tma_load_2d_pair(dst, &map_x, leader_full, (int32_t)(kb * kBlockK), x_row);
                    tma_load_2d_pair(dst + kHalfBytes, &map_w, leader_full, (int32_t)(kb * kBlockK), w_row);
                }
            }
            pdl_launch_dependents();
            // every copy this thread issued has landed once the MMAs that read it are done
            for (uint32_t back = 0; back < kStages && back < it && ok; back++) {
                const uint32_t j = it - 1 - back;
                ok = wait_bounded(&empty[j % kStages], (j / kStages) & 1, abort_flag);
            }
        }
    } else if (warp == 1) {
        // ---- MMA: the leader issues for the pair ----
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(kTileM, kTileN);
            bool ok = true;
            uint32_t it = 0, acc_it = 0;
            for (uint32_t tile = pair; tile < tiles && ok; tile += pairs, acc_it++) {
                const uint32_t as = acc_it % kAccStages, aph = (acc_it / kAccStages) & 1;
                ok = wait_bounded(&acc_empty[as], aph ^ 1, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * kTileN;
                for (uint32_t kb = 0; kb < p.kb_total; kb++, it++) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    ok = wait_bounded(&full[s], ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t da = umma_desc_k_sw128(smem_addr(smem + s * kStageBytes));
                    const uint64_t db = umma_desc_k_sw128(smem_addr(smem + s * kStageBytes + kHalfBytes));
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kBlockK / 16; k16++)
                        umma_bf16_pair(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                    umma_commit_pair(&empty[s]);  // the stage is free in both blocks once these MMAs are done
                }
                if (ok) umma_commit_pair(&acc_full[as]);
            }
        }
    } else {
        // ---- epilogue: warp w reads lanes (w % 4) * 32 .. + 31 of this block's TMEM ----
        const uint32_t q = warp & 3;
        const uint32_t row = q * 32 + lane;
        const uint32_t out_n = p.gated ? p.n / 2 : p.n;
        bool ok = true;
        uint32_t acc_it = 0;
        for (uint32_t tile = pair; tile < tiles && ok; tile += pairs, acc_it++) {
            const uint32_t ti = tile / p.tiles_j, tj = tile % p.tiles_j;
            const uint32_t as = acc_it % kAccStages, aph = (acc_it / kAccStages) & 1;
            ok = wait_bounded(&acc_full[as], aph, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t gi = ti * kTileM + rank * kRowsPerBlock + row;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + as * kTileN;
            float inv = 1.0f;  // this thread's row: 1/rms from the partial sums the upstream linear left
            if (p.row_ss && gi < p.m) {
                float ss = 0.0f;
                for (uint32_t i = 0; i < p.row_parts; i++) ss += p.row_ss[(size_t)gi * p.row_parts + i];
                inv = 1.0f / sqrtf(ss / (float)p.k + p.row_eps);
            }
            float sq = 0.0f;   // sum of squares of the row's finished values over this tile's columns
            if (p.gated) {
                // columns [0, 128) are gate rows of w (the leader's half of B), [128, 256) the matching up rows
                for (uint32_t c0 = 0; c0 < 128; c0 += 16) {
                    uint32_t rg[16], ru[16];
                    tmem_ld_32x16(taddr + c0, rg);
                    tmem_ld_32x16(taddr + 128 + c0, ru);
                    tmem_ld_wait();
                    if (gi < p.m) {
                        const uint32_t gj0 = tj * 128 + c0;
                        const size_t at0 = (size_t)gi * out_n + gj0;
                        float v[16];
#pragma unroll
                        for (uint32_t c = 0; c < 16; c++) {
                            const float gv = __uint_as_float(rg[c]) * inv, uv = __uint_as_float(ru[c]) * inv;
                            v[c] = (p.epilogue == TS_EPI_SWIGLU ? silu(gv) : gelu_tanh(gv)) * uv;
                        }
                        if (out_n % 8 == 0 && gj0 + 16 <= out_n && p.out_dtype == TS_BF16) {
                            uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + at0;
#pragma unroll
                            for (uint32_t c = 0; c < 16; c += 8)
                                *reinterpret_cast<uint4 *>(o + c) =
                                    make_uint4(pack_bf16(v[c], v[c + 1]), pack_bf16(v[c + 2], v[c + 3]),
                                               pack_bf16(v[c + 4], v[c + 5]), pack_bf16(v[c + 6], v[c + 7]));
                        } else {
#pragma unroll
                            for (uint32_t c = 0; c < 16; c++)
                                if (gj0 + c < out_n) {
                                    if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[at0 + c] = v[c];
                                    else reinterpret_cast<uint16_t *>(p.out)[at0 + c] = bf16_bits(v[c]);
                                }
                        }
                    }
                }
            } else {
                for (uint32_t c0 = 0; c0 < kTileN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c0, r);
                    tmem_ld_wait();
                    if (gi >= p.m) continue;
                    const uint32_t gj0 = tj * kTileN + c0;
                    if (gj0 >= p.n) continue;
                    const size_t at0 = (size_t)gi * p.n + gj0;
                    const bool vec = (p.n % 8 == 0) && gj0 + 32 <= p.n;
                    if (vec && p.out_dtype == TS_BF16) {
                        uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + at0;
#pragma unroll
                        for (uint32_t c = 0; c < 32; c += 8) {
                            float v[8];
#pragma unroll
                            for (uint32_t e = 0; e < 8; e++) {
                                v[e] = __uint_as_float(r[c + e]) * inv;
                                if (p.epilogue == TS_EPI_ADD) v[e] += p.a0[at0 + c + e];
                                if (p.epilogue == TS_EPI_SCALE) v[e] *= p.scale;
                            }
                            *reinterpret_cast<uint4 *>(o + c) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]),
                                                                           pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                        }
                    } else if (vec) {
                        float *o = reinterpret_cast<float *>(p.out) + at0;
#pragma unroll
                        for (uint32_t c = 0; c < 32; c += 4) {
                            float4 v = make_float4(__uint_as_float(r[c]) * inv, __uint_as_float(r[c + 1]) * inv,
                                                   __uint_as_float(r[c + 2]) * inv, __uint_as_float(r[c + 3]) * inv);
                            if (p.epilogue == TS_EPI_ADD) {
                                const float4 a = *reinterpret_cast<const float4 *>(p.a0 + at0 + c);
                                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                            }
                            if (p.epilogue == TS_EPI_SCALE) {
                                v.x *= p.scale; v.y *= p.scale; v.z *= p.scale; v.w *= p.scale;
                            }
                            *reinterpret_cast<float4 *>(o + c) = v;
                            if (p.ss_out) {  // the host asks for these only with n % 8 == 0 and an f32 output: this path
                                sq = fmaf(v.x, v.x, sq); sq = fmaf(v.y, v.y, sq); sq = fmaf(v.z, v.z, sq); sq = fmaf(v.w, v.w, sq);
                                const float4 g = *reinterpret_cast<const float4 *>(p.xs_gain + gj0 + c);
                                *reinterpret_cast<uint2 *>(p.xs_out + at0 + c) =
                                    make_uint2(pack_bf16(v.x * g.x, v.y * g.y), pack_bf16(v.z * g.z, v.w * g.w));
                            }
                        }
                    } else {
#pragma unroll
                        for (uint32_t c = 0; c < 32; c++)
                            if (gj0 + c < p.n) {
                                float v = __uint_as_float(r[c]) * inv;
                                if (p.epilogue == TS_EPI_ADD) v += p.a0[at0 + c];
                                if (p.epilogue == TS_EPI_SCALE) v *= p.scale;
                                if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[at0 + c] = v;
                                else reinterpret_cast<uint16_t *>(p.out)[at0 + c] = bf16_bits(v);
                                if (p.ss_out) {
                                    sq = fmaf(v, v, sq);
                                    p.xs_out[at0 + c] = bf16_bits(v * p.xs_gain[gj0 + c]);
                                }
                            }
                    }
                }
            }
            if (p.ss_out && gi < p.m) p.ss_out[(size_t)gi * p.tiles_j + tj] = sq;
            // Release the accumulator stage to the leader's MMA thread: one arrival per epilogue warp of
            // either block.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_rank(smem_addr(&acc_empty[as]), 0));
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TS_ERR_TIMEOUT);
    cluster_sync();  // neither block frees the pair's TMEM, or leaves, while the other may still use it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

__device__ int g_pair_status = 0;

}  // namespace

int pair_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_pair_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_pair_status, &zero, sizeof(int));
    return v;
}

// Pairs of SMs that can hold a cluster of two of these blocks at the same time (not every SM has a partner
// on a part with disabled SMs); persistent pairs beyond that number would only queue behind the others.
uint32_t pair_slots() {
    static std::atomic<uint32_t> per_device[256] = {};
    std::atomic<uint32_t> &cached = per_device[current_device() & 255];
    if (const uint32_t have = cached.load(std::memory_order_relaxed)) return have;
    cudaFuncSetAttribute(linear_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((uint32_t)sm_count() / 2 * 2);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemTotal;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, linear_pair_kernel, &cfg) != cudaSuccess || clusters <= 0)
        clusters = sm_count() / 2;
    cached.store((uint32_t)clusters, std::memory_order_relaxed);
    return (uint32_t)clusters;
}

// Worth it from a few hundred rows on: below that the 256-row tile wastes more than the pairing saves.
bool pair_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    if (m < 512 || k == 0 || k % kBlockK != 0) return false;
    if (gated) return n % 2 == 0 && (n / 2) % 128 == 0;
    return n >= 256;
}

uint32_t pair_sumsq_parts(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    return (!gated && pair_supports(m, n, k, epilogue) && n % 8 == 0) ? ceil_div(n, kTileN) : 0;
}

int linear_pair(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k, int epilogue,
                float scale, int out_dtype, cudaStream_t stream, const StreamFused *fused) {
    if (!pair_supports(m, n, k, epilogue))
        return fail(TS_ERR_BAD_INPUT, "linear (pair): unsupported shape m=%u n=%u k=%u epilogue=%d", m, n, k, epilogue);
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    CUtensorMap map_x, map_w;
    int rc = make_tensor_map_2d(&map_x, x, m, k, k, 128, kBlockK);
    if (rc != TS_OK) return rc;
    rc = make_tensor_map_2d(&map_w, w, n, k, k, 128, kBlockK);
    if (rc != TS_OK) return rc;
    PairParams p = {};
    p.m = m;
    p.n = n;
    p.k = k;
    p.kb_total = k / kBlockK;
    p.tiles_i = ceil_div(m, kTileM);
    p.tiles_j = gated ? (n / 2) / 128 : ceil_div(n, kTileN);
    p.gated = gated;
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.scale = scale;
    p.a0 = (const float *)a0;
    p.out = out;
    if (fused) {
        if (fused->row_ss)
            TS_REQUIRE(fused->row_parts >= 1 && fused->row_parts <= 64, "linear (pair): 1..64 partial sums per row, got %u",
                       fused->row_parts);
        if (fused->ss_out || fused->xs_out)
            TS_REQUIRE(fused->ss_out && fused->xs_out && fused->xs_gain && out_dtype == TS_F32 &&
                           pair_sumsq_parts(m, n, k, epilogue) != 0,
                       "linear (pair): sums of squares and the scaled copy come together, with an f32 output and n %% 8 == 0");
        p.row_ss = fused->row_ss;
        p.row_parts = fused->row_parts;
        p.row_eps = fused->row_eps;
        p.ss_out = fused->ss_out;
        p.xs_out = (uint16_t *)fused->xs_out;
        p.xs_gain = fused->xs_gain;
    }
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_pair_status));
    p.status = status;
    static OncePerDevice configured;
    if (configured.needs()) {
        TS_CUDA(cudaFuncSetAttribute(linear_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
        configured.done();
    }
    const uint32_t tiles = p.tiles_i * p.tiles_j;
    const uint32_t pairs = std::min<uint32_t>(tiles, pair_slots());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pairs * 2);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    unsigned n_attr = 1;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, linear_pair_kernel, map_x, map_w, p);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_pair failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
