// Linear on the 5th-generation tensor cores: D[i, j] = sum_k A[i, k] * B[j, k] with both
// operands K-major bf16, fetched by TMA into 128-byte-swizzled shared-memory tiles, multiplied by
// tcgen05.mma (one issuing thread, 128 x BN x 16 per instruction) into f32 accumulators that live
// in tensor memory, and read back with tcgen05.ld by four epilogue warps.
//
// Two uses of the same kernel:
//   * prefill-sized m: A = x (rows on TMEM lanes), B = w; both stream through the stage ring.
//   * decode-sized m (<= 128): A = w, B = x ("swapped"): the whole k slice of x is loaded once and
//     stays resident in shared memory while the block walks over 128-row weight tiles, so weights
//     cross HBM -> shared memory exactly once and nothing else moves.
//
// Blocks are persistent: each walks tiles blockIdx.x, + gridDim.x, ...; two accumulator stages in
// TMEM let the epilogue of one tile overlap the MMAs of the next.  Warp roles: 0 = TMA producer,
// 1 = MMA issuer (also owns the TMEM allocation), 2..5 = epilogue.
//
// Stands in for the reference's `tiled*` / `parts_*` rules (engine/rules/linear/src/tiled.rs:295-446).
#include "ts_common.cuh"
#include "ts_ptx.cuh"

namespace ts {

// Shared with the skinny path: adds k slices in ascending order and applies the epilogue.
int launch_linear_reduce(const float *partial, uint32_t splits, const float *a0, void *out, uint32_t m,
                         uint32_t n, int epilogue, float scale, int out_dtype, cudaStream_t stream);

namespace {

using namespace ptx;

constexpr uint32_t kBlockA = 128;  // rows of A per tile = TMEM lanes
constexpr uint32_t kBlockK = 64;   // bf16 per k block = one 128-byte swizzle row
constexpr uint32_t kThreads = 192;
constexpr uint32_t kAccStages = 2;

struct UmmaParams {
    uint32_t ia, jb, k;      // D is [ia, jb]
    uint32_t kb_per_split;   // k blocks per split
    uint32_t splits;
    uint32_t tiles_i, tiles_j;
    uint32_t stages;
    uint32_t b_resident;     // B's k slice loaded once per block (tiles_j must be 1)
    uint32_t swapped;        // output element (i, j) is out[j, i]
    uint32_t gated;          // not swapped only: B tiles pair gate rows with their up rows
    uint32_t to_partial;     // write f32 sums of each k slice to `partial`; a second kernel finishes
    uint32_t m, n;           // output matrix [m, n] (before gating)
    int epilogue, out_dtype;
    float scale;
    const float *a0;
    void *out;
    float *partial;
    int *status;             // device word: 0, or TS_ERR_TIMEOUT once any wait gave up
};

struct SmemLayout {
    uint32_t a_off, b_off, bar_off, total;
};

// Offsets from a 1024-byte-aligned base; `total` includes the slack for aligning that base.
__host__ __device__ inline SmemLayout smem_layout(uint32_t bn, uint32_t stages, uint32_t b_blocks) {
    SmemLayout l;
    l.a_off = 0;
    l.b_off = stages * kBlockA * kBlockK * 2;
    l.bar_off = l.b_off + b_blocks * bn * kBlockK * 2;
    l.total = l.bar_off + 256 + 1024;
    return l;
}

// Bounded wait that also leaves when another role has already given up.
// Gives up after two seconds of wall time (or kSpinLimit polls, whichever comes first).
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag) {
    uint64_t start = 0;
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > 2000000000ull) break;
        }
    }
    *abort_flag = 1;
    return false;
}

template <uint32_t BN>
__global__ void __launch_bounds__(kThreads, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const UmmaParams p) {
    extern __shared__ unsigned char smem_raw[];
    // The swizzled tiles need a 1024-byte-aligned base.
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b_blocks = p.b_resident ? p.kb_per_split : p.stages;
    const SmemLayout L = smem_layout(BN, p.stages, b_blocks);
    unsigned char *smem_a = smem + L.a_off;
    unsigned char *smem_b = smem + L.b_off;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bar_off);   // [stages]
    uint64_t *empty = full + 8;                                        // [stages]
    uint64_t *acc_full = empty + 8;                                    // [2]
    uint64_t *acc_empty = acc_full + 2;                                // [2]
    uint64_t *b_full = acc_empty + 2;                                  // [1]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(b_full + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    constexpr uint32_t kTmemCols = (kAccStages * BN) < 32 ? 32 : kAccStages * BN;
    const uint32_t split = blockIdx.y;
    const uint32_t kb0 = split * p.kb_per_split;
    const uint32_t tiles = p.tiles_i * p.tiles_j;
    constexpr uint32_t kABytes = kBlockA * kBlockK * 2;
    constexpr uint32_t kBBytes = BN * kBlockK * 2;

    if (threadIdx.x == 0) STAMP(0);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (uint32_t s = 0; s < kAccStages; s++) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        mbar_init(b_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) STAMP(1);

    // Row of w where the up half of a gated tile starts.
    const uint32_t gate_rows_b = p.n / 2;

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            // Weights never depend on the upstream kernel; x does.  In the swapped layout A is the
            // weight, so only B has to wait.
            if (!p.swapped) pdl_wait();
            STAMP(2);
            uint32_t it = 0;
            bool ok = true;
            if (p.b_resident) {
                if (p.swapped) pdl_wait();
                mbar_expect_tx(b_full, p.kb_per_split * kBBytes);
                for (uint32_t kb = 0; kb < p.kb_per_split; kb++)
                    tma_load_2d(smem_b + kb * kBBytes, &map_b, b_full, (int32_t)((kb0 + kb) * kBlockK), 0);
            }
            for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const uint32_t ti = tile / p.tiles_j, tj = tile % p.tiles_j;
                for (uint32_t kb = 0; kb < p.kb_per_split; kb++, it++) {
                    const uint32_t s = it % p.stages, ph = (it / p.stages) & 1;
                    ok = wait_or_abort(&empty[s], ph ^ 1, abort_flag);
                    if (!ok) break;
                    const int32_t kx = (int32_t)((kb0 + kb) * kBlockK);
                    const uint32_t bytes = kABytes + (p.b_resident ? 0 : kBBytes);
                    mbar_expect_tx(&full[s], bytes);
                    unsigned char *dst_a = smem_a + s * kABytes;
                    tma_load_2d(dst_a, &map_a, &full[s], kx, (int32_t)(ti * kBlockA));
                    if (!p.b_resident) {
                        unsigned char *dst_b = smem_b + s * kBBytes;
                        if (p.gated) {
                            tma_load_2d(dst_b, &map_b, &full[s], kx, (int32_t)(tj * (BN / 2)));
                            tma_load_2d(dst_b + kBBytes / 2, &map_b, &full[s], kx,
                                        (int32_t)(gate_rows_b + tj * (BN / 2)));
                        } else {
                            tma_load_2d(dst_b, &map_b, &full[s], kx, (int32_t)(tj * BN));
                        }
                    }
                }
            }
            STAMP(3);
            pdl_launch_dependents();
            // Copies still in flight must land before the block's shared memory goes away: wait for
            // the consumer to release every stage this thread filled (bounded).
            if (ok) {
                const uint32_t last = it;
                for (uint32_t back = 0; back < p.stages && back < last; back++) {
                    const uint32_t j = last - 1 - back;
                    const uint32_t s = j % p.stages, ph = (j / p.stages) & 1;
                    if (!wait_or_abort(&empty[s], ph, abort_flag)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(kBlockA, BN);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            if (p.b_resident) ok = wait_or_abort(b_full, 0, abort_flag);
            STAMP(4);
            for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, acc_it++) {
                const uint32_t as = acc_it % kAccStages, aph = (acc_it / kAccStages) & 1;
                ok = wait_or_abort(&acc_empty[as], aph ^ 1, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (uint32_t kb = 0; kb < p.kb_per_split; kb++, it++) {
                    const uint32_t s = it % p.stages, ph = (it / p.stages) & 1;
                    ok = wait_or_abort(&full[s], ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_addr(smem_a + s * kABytes);
                    const uint32_t b_addr = smem_addr(smem_b + (p.b_resident ? kb : s) * kBBytes);
                    const uint64_t da = umma_desc_k_sw128(a_addr), db = umma_desc_k_sw128(b_addr);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kBlockK / 16; k16++) {
                        // 16 bf16 = 32 bytes further along the swizzled row: +2 in the address field
                        umma_bf16(d_tmem, da + 2 * k16, db + 2 * k16, idesc, (kb | k16) != 0);
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[as]);
                STAMP(5);
            }
        }
    } else {
        // ---- epilogue: warp w reads TMEM lanes (w % 4) * 32 .. + 31 ----
        const uint32_t q = warp & 3;
        uint32_t acc_it = 0;
        bool ok = true;
        const uint32_t out_n = p.gated ? p.n / 2 : p.n;
        constexpr uint32_t kChunk = BN < 32 ? BN : 32;
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, acc_it++) {
            const uint32_t ti = tile / p.tiles_j, tj = tile % p.tiles_j;
            const uint32_t as = acc_it % kAccStages, aph = (acc_it / kAccStages) & 1;
            ok = wait_or_abort(&acc_full[as], aph, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            if (warp == 2 && lane == 0) STAMP(6);
            const uint32_t row = q * 32 + lane;  // row of the 128 x BN tile this thread owns
            const uint32_t gi = ti * kBlockA + row;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + as * BN;

            if (p.to_partial) {
                // f32 sums of this k slice; the reduce kernel adds the slices and applies the epilogue.
                float *part = p.partial + (size_t)split * p.m * p.n;
                for (uint32_t c0 = 0; c0 < BN; c0 += kChunk) {
                    uint32_t r[32];
                    if constexpr (BN >= 32) tmem_ld_32x32(taddr + c0, r);
                    else {
                        uint32_t r16[16];
                        tmem_ld_32x16(taddr + c0, r16);
#pragma unroll
                        for (int c = 0; c < 16; c++) r[c] = r16[c];
                    }
                    tmem_ld_wait();
                    if (gi < p.ia) {
#pragma unroll
                        for (uint32_t c = 0; c < kChunk; c++) {
                            const uint32_t gj = tj * BN + c0 + c;
                            if (gj < p.jb) {
                                const size_t at = p.swapped ? (size_t)gj * p.n + gi : (size_t)gi * p.n + gj;
                                part[at] = __uint_as_float(r[c]);
                            }
                        }
                    }
                }
            } else if (p.gated) {
                // Not swapped: columns [0, BN/2) are gate rows of w, [BN/2, BN) the matching up rows.
                constexpr uint32_t kHalf = BN / 2;
                if constexpr (kHalf >= 16) {
                    for (uint32_t c0 = 0; c0 < kHalf; c0 += 16) {
                        uint32_t rg[16], ru[16];
                        tmem_ld_32x16(taddr + c0, rg);
                        tmem_ld_32x16(taddr + kHalf + c0, ru);
                        tmem_ld_wait();
                        if (gi < p.ia) {
                            const uint32_t gj0 = tj * kHalf + c0;
                            const size_t at0 = (size_t)gi * out_n + gj0;
                            const bool vec = (out_n % 8 == 0) && gj0 + 16 <= out_n;
                            float v[16];
#pragma unroll
                            for (uint32_t c = 0; c < 16; c++) {
                                float gv = __uint_as_float(rg[c]), uv = __uint_as_float(ru[c]);
                                v[c] = (p.epilogue == TS_EPI_SWIGLU ? silu(gv) : gelu_tanh(gv)) * uv;
                            }
                            if (vec && p.out_dtype == TS_BF16) {
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
                }
            } else {
                for (uint32_t c0 = 0; c0 < BN; c0 += kChunk) {
                    uint32_t r[32];
                    if constexpr (BN >= 32) tmem_ld_32x32(taddr + c0, r);
                    else {
                        uint32_t r16[16];
                        tmem_ld_32x16(taddr + c0, r16);
#pragma unroll
                        for (int c = 0; c < 16; c++) r[c] = r16[c];
                    }
                    tmem_ld_wait();
                    if (gi >= p.ia) continue;
                    const uint32_t gj0 = tj * BN + c0;
                    if (!p.swapped) {
                        // This thread owns kChunk consecutive columns of output row gi.
                        const size_t at0 = (size_t)gi * p.n + gj0;
                        const bool vec = (p.n % 8 == 0) && gj0 + kChunk <= p.jb;
                        if (vec && p.out_dtype == TS_BF16) {
                            uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + at0;
#pragma unroll
                            for (uint32_t c = 0; c < kChunk; c += 8) {
                                float v[8];
#pragma unroll
                                for (uint32_t e = 0; e < 8; e++) {
                                    v[e] = __uint_as_float(r[c + e]);
                                    if (p.epilogue == TS_EPI_ADD) v[e] += p.a0[at0 + c + e];
                                    if (p.epilogue == TS_EPI_SCALE) v[e] *= p.scale;
                                }
                                *reinterpret_cast<uint4 *>(o + c) =
                                    make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]),
                                               pack_bf16(v[6], v[7]));
                            }
                        } else if (vec) {
                            float *o = reinterpret_cast<float *>(p.out) + at0;
#pragma unroll
                            for (uint32_t c = 0; c < kChunk; c += 4) {
                                float4 v = make_float4(__uint_as_float(r[c]), __uint_as_float(r[c + 1]),
                                                       __uint_as_float(r[c + 2]), __uint_as_float(r[c + 3]));
                                if (p.epilogue == TS_EPI_ADD) {
                                    const float4 a = *reinterpret_cast<const float4 *>(p.a0 + at0 + c);
                                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                                }
                                if (p.epilogue == TS_EPI_SCALE) {
                                    v.x *= p.scale; v.y *= p.scale; v.z *= p.scale; v.w *= p.scale;
                                }
                                *reinterpret_cast<float4 *>(o + c) = v;
                            }
                        } else {
#pragma unroll
                            for (uint32_t c = 0; c < kChunk; c++)
                                if (gj0 + c < p.jb) {
                                    float v = __uint_as_float(r[c]);
                                    if (p.epilogue == TS_EPI_ADD) v += p.a0[at0 + c];
                                    if (p.epilogue == TS_EPI_SCALE) v *= p.scale;
                                    if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[at0 + c] = v;
                                    else reinterpret_cast<uint16_t *>(p.out)[at0 + c] = bf16_bits(v);
                                }
                        }
                    } else {
                        // Swapped: this thread owns output column gi; consecutive lanes write consecutive
                        // columns of one output row.
#pragma unroll
                        for (uint32_t c = 0; c < kChunk; c++) {
                            const uint32_t gj = gj0 + c;
                            if (gj < p.jb) {
                                const size_t at = (size_t)gj * p.n + gi;
                                float v = __uint_as_float(r[c]);
                                if (p.epilogue == TS_EPI_ADD) v += p.a0[at];
                                if (p.epilogue == TS_EPI_SCALE) v *= p.scale;
                                if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[at] = v;
                                else reinterpret_cast<uint16_t *>(p.out)[at] = bf16_bits(v);
                            }
                        }
                    }
                }
            }
            if (warp == 2 && lane == 0) STAMP(7);
            // Release the accumulator stage: one arrival per epilogue warp.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) STAMP(8);
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TS_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

struct UmmaPlan {
    uint32_t bn, stages, splits, kb_per_split, tiles_i, tiles_j, blocks;
    bool swapped, b_resident, gated, to_partial;
    SmemLayout layout;
};

constexpr uint32_t kSmemBudget = 224 * 1024;

bool plan_umma(uint32_t m, uint32_t n, uint32_t k, int epilogue, UmmaPlan *out) {
    UmmaPlan s = {};
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    if (k == 0 || k % kBlockK != 0 || m == 0 || n == 0) return false;
    if (gated && n % 2 != 0) return false;
    const uint32_t kb = k / kBlockK;
    const uint32_t sms = (uint32_t)sm_count();
    s.swapped = m <= 128;
    if (s.swapped) {
        // A = w (n rows on TMEM lanes), B = x (m rows, one column tile, resident).
        s.bn = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
        s.tiles_i = ceil_div(n, kBlockA);
        s.tiles_j = 1;
        s.b_resident = true;
        s.gated = false;  // gating happens in the reduce kernel
        auto fits = [&](uint32_t sp) { return smem_layout(s.bn, 3, kb / sp).total <= kSmemBudget; };
        // Split k until the resident x slice fits and the machine has about a tile per SM, keeping
        // at least two k blocks per slice.
        uint32_t splits = 1;
        while (kb % (splits * 2) == 0 && kb / (splits * 2) >= 2 && (!fits(splits) || s.tiles_i * splits < sms))
            splits *= 2;
        if (!fits(splits)) return false;
        s.splits = splits;
        s.kb_per_split = kb / splits;
        s.to_partial = splits > 1 || gated;
        uint32_t stages = 8;
        while (stages > 3 && smem_layout(s.bn, stages, s.kb_per_split).total > kSmemBudget) stages--;
        s.stages = stages;
        s.layout = smem_layout(s.bn, s.stages, s.kb_per_split);
    } else {
        s.gated = gated;
        s.bn = gated ? 128 : (n >= 256 ? 256 : 128);
        if (gated && (n / 2) % (s.bn / 2) != 0) return false;
        s.tiles_i = ceil_div(m, kBlockA);
        s.tiles_j = gated ? (n / 2) / (s.bn / 2) : ceil_div(n, s.bn);
        s.b_resident = false;
        // A handful of output tiles (a router: a few hundred rows against a hundred experts) would run their
        // whole k loop on as many SMs: split k over blocks until about half the machine is busy, at least four
        // k blocks a slice; the slices meet in the reduce kernel, in ascending order.
        uint32_t splits = 1;
        if (!gated)
            while (kb % (splits * 2) == 0 && kb / (splits * 2) >= 4 && s.tiles_i * s.tiles_j * splits * 2 <= sms / 2)
                splits *= 2;
        s.splits = splits;
        s.kb_per_split = kb / splits;
        s.to_partial = splits > 1;
        uint32_t stages = 8;
        while (stages > 2 && smem_layout(s.bn, stages, stages).total > kSmemBudget) stages--;
        s.stages = stages;
        s.layout = smem_layout(s.bn, s.stages, s.stages);
    }
    s.blocks = std::min<uint32_t>(s.tiles_i * s.tiles_j, sms);
    *out = s;
    return true;
}

__device__ int g_umma_status = 0;

template <uint32_t BN>
cudaError_t launch_umma(const CUtensorMap &ma, const CUtensorMap &mb, const UmmaParams &p, const UmmaPlan &s,
                        cudaStream_t stream) {
    auto kernel = linear_umma_kernel<BN>;
    static OncePerDevice configured;
    if (configured.needs()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
        if (e != cudaSuccess) return e;
        configured.done();
    }
    return launch(kernel, dim3(s.blocks, s.splits), dim3(kThreads), s.layout.total, stream, pdl_enabled(), ma,
                  mb, p);
}

}  // namespace

bool umma_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    UmmaPlan s;
    return plan_umma(m, n, k, epilogue, &s);
}

size_t umma_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    UmmaPlan s;
    if (!plan_umma(m, n, k, epilogue, &s)) return 0;
    return s.to_partial ? (size_t)s.splits * m * n * sizeof(float) : 0;
}

// Reads (and clears) the device word that a timed-out wait sets.  Synchronises the device.
int umma_take_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int));
    return v;
}

int linear_umma(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                int epilogue, float scale, int out_dtype, void *workspace, size_t workspace_bytes,
                cudaStream_t stream) {
    UmmaPlan s;
    if (!plan_umma(m, n, k, epilogue, &s))
        return fail(TS_ERR_BAD_INPUT, "linear (umma): unsupported shape m=%u n=%u k=%u epilogue=%d", m, n, k, epilogue);
    size_t need = s.to_partial ? (size_t)s.splits * m * n * sizeof(float) : 0;
    TS_REQUIRE(workspace_bytes >= need && (need == 0 || workspace != nullptr),
               "linear (umma): workspace of %zu bytes is smaller than the %zu needed", workspace_bytes, need);
    CUtensorMap map_a, map_b;
    const void *a_ptr = s.swapped ? w : x;
    const void *b_ptr = s.swapped ? x : w;
    const uint32_t ia = s.swapped ? n : m, jb = s.swapped ? m : n;
    uint32_t box_a = kBlockA;
    uint32_t box_b = s.gated ? s.bn / 2 : s.bn;
    int rc = make_tensor_map_2d(&map_a, a_ptr, ia, k, k, box_a, kBlockK);
    if (rc != TS_OK) return rc;
    rc = make_tensor_map_2d(&map_b, b_ptr, jb, k, k, box_b, kBlockK);
    if (rc != TS_OK) return rc;

    UmmaParams p = {};
    p.ia = ia;
    p.jb = jb;
    p.k = k;
    p.kb_per_split = s.kb_per_split;
    p.splits = s.splits;
    p.tiles_i = s.tiles_i;
    p.tiles_j = s.tiles_j;
    p.stages = s.stages;
    p.b_resident = s.b_resident;
    p.swapped = s.swapped;
    p.gated = s.gated;
    p.to_partial = s.to_partial;
    p.m = m;
    p.n = n;
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.scale = scale;
    p.a0 = (const float *)a0;
    p.out = out;
    p.partial = (float *)workspace;
    int *status = nullptr;
    TS_CUDA(cudaGetSymbolAddress((void **)&status, g_umma_status));
    p.status = status;

    cudaError_t e;
    switch (s.bn) {
    case 16: e = launch_umma<16>(map_a, map_b, p, s, stream); break;
    case 32: e = launch_umma<32>(map_a, map_b, p, s, stream); break;
    case 64: e = launch_umma<64>(map_a, map_b, p, s, stream); break;
    case 128: e = launch_umma<128>(map_a, map_b, p, s, stream); break;
    default: e = launch_umma<256>(map_a, map_b, p, s, stream); break;
    }
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_umma failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    if (s.to_partial)
        return launch_linear_reduce((const float *)workspace, s.splits, (const float *)a0, out, m, n, epilogue, scale,
                                    out_dtype, stream);
    return TS_OK;
}

}  // namespace ts
