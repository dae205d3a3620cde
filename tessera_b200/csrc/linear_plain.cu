// The linear for shapes the tensor-core kernels do not take: any m, n, k (k off the 64 grid, rows that start
// off a 16-byte boundary, a handful of outputs).  The reference's `tiled` rule takes every size
// (engine/rules/linear/tests/tiled_test.rs:61-67 runs 1 x 3 x 4 and 37 x 50 x 72 beside the block-sized cases);
// this kernel keeps that promise, the others keep the speed.  A warp per output element: lane l sums
// k = l, l + 32, ... in ascending order, the 32 partial sums meet in a fixed butterfly, so a re-run gives the
// same bits.  Gated epilogues take the gate row n and the up row n + n_out of w side by side.
#include "ts_common.cuh"
#include "ts_kernels.cuh"

namespace ts {
namespace {

struct PlainParams {
    const uint16_t *x, *w;
    const float *a0;
    void *out;
    uint32_t m, n, k;
    int epilogue, out_dtype;
    float scale;
};

__device__ __forceinline__ float widen(uint16_t bits) { return __uint_as_float((uint32_t)bits << 16); }

__global__ void __launch_bounds__(256) linear_plain_kernel(const PlainParams p) {
    pdl_wait();
    const bool gated = p.epilogue == TS_EPI_SWIGLU || p.epilogue == TS_EPI_GEGLU;
    const uint32_t out_n = gated ? p.n / 2 : p.n;
    const size_t total = (size_t)p.m * out_n;
    const uint32_t lane = threadIdx.x & 31;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t i = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < total; i += warps) {
        const uint32_t row = (uint32_t)(i / out_n), col = (uint32_t)(i % out_n);
        const uint16_t *xr = p.x + (size_t)row * p.k;
        const uint16_t *wr = p.w + (size_t)col * p.k;
        const uint16_t *ur = wr + (size_t)out_n * p.k;  // the up row of a gated pair
        float sum = 0.0f, up = 0.0f;
        for (uint32_t j = lane; j < p.k; j += 32) {
            const float xv = widen(xr[j]);
            sum = fmaf(xv, widen(wr[j]), sum);
            if (gated) up = fmaf(xv, widen(ur[j]), up);
        }
        sum = warp_sum(sum);
        if (gated) up = warp_sum(up);
        if (lane == 0) {
            float v = sum;
            if (gated) v = (p.epilogue == TS_EPI_SWIGLU ? silu(sum) : gelu_tanh(sum)) * up;
            else if (p.epilogue == TS_EPI_ADD) v += p.a0[i];
            else if (p.epilogue == TS_EPI_SCALE) v *= p.scale;
            if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[i] = v;
            else reinterpret_cast<uint16_t *>(p.out)[i] = bf16_bits(v);
        }
    }
    pdl_launch_dependents();
}

// The same product with every output summed over k in ascending order, one multiply and one add at a time
// (no fused multiply-add, no tree): the order of the reference's interpreter (engine/ir/interp/src/cpu.rs
// matmul, sequential f32 sums), so the f32 outputs carry its bits.  For the few outputs whose *ranking* matters:
// a MoE router's scores feed top-k, and an index must not flip on a near tie because the sums met in another
// order.  A block owns 8 rows x 32 columns and walks k in chunks staged in shared memory (coalesced loads); a
// thread owns one output.
constexpr uint32_t kOrdRows = 8, kOrdCols = 32, kOrdChunk = 128, kOrdThreads = kOrdRows * kOrdCols;

__device__ __forceinline__ void widen8(const uint4 &v, float *to) {
    to[0] = bf16_lo(v.x); to[1] = bf16_hi(v.x); to[2] = bf16_lo(v.y); to[3] = bf16_hi(v.y);
    to[4] = bf16_lo(v.z); to[5] = bf16_hi(v.z); to[6] = bf16_lo(v.w); to[7] = bf16_hi(v.w);
}

// VEC: k is a multiple of 8 and both operands start on 16-byte boundaries, so a chunk arrives as 16-byte loads,
// asked for one chunk ahead of the sums that use it; otherwise element by element.
template <bool VEC>
__global__ void __launch_bounds__(kOrdThreads) linear_ordered_kernel(const PlainParams p) {
    // Rows of w are 132 floats apart: the 16-byte reads of eight consecutive lanes (eight rows, the same k) then fall on
    // 32 different banks.  The shared-memory pipe is what bounds this kernel, so both operands move 16 bytes at a time.
    __shared__ __align__(16) float xs[kOrdRows][kOrdChunk];
    __shared__ __align__(16) float ws[kOrdCols][kOrdChunk + 4];
    pdl_wait();
    const uint32_t tid = threadIdx.x, tx = tid % kOrdCols, ty = tid / kOrdCols;
    const uint32_t row0 = blockIdx.y * kOrdRows, col0 = blockIdx.x * kOrdCols;
    float sum = 0.0f;
    if constexpr (VEC) {
        // piece i of a chunk: 8 consecutive k of one row; pieces 0..127 are x (8 rows x 16), 128..639 are w (32 x 16)
        constexpr uint32_t kPer = (kOrdRows + kOrdCols) * (kOrdChunk / 8) / kOrdThreads + 1;  // 3
        uint4 held[kPer];
        auto ask = [&](uint32_t k0) {
#pragma unroll
            for (uint32_t u = 0; u < kPer; u++) {
                const uint32_t i = tid + u * kOrdThreads;
                held[u] = make_uint4(0, 0, 0, 0);
                if (i >= (kOrdRows + kOrdCols) * (kOrdChunk / 8)) continue;
                const bool is_x = i < kOrdRows * (kOrdChunk / 8);
                const uint32_t j = is_x ? i : i - kOrdRows * (kOrdChunk / 8);
                const uint32_t r = j / (kOrdChunk / 8), kk = k0 + (j % (kOrdChunk / 8)) * 8;
                const uint32_t line = is_x ? row0 + r : col0 + r;
                if (kk < p.k && line < (is_x ? p.m : p.n))
                    held[u] = __ldg(reinterpret_cast<const uint4 *>((is_x ? p.x : p.w) + (size_t)line * p.k + kk));
            }
        };
        ask(0);
        for (uint32_t k0 = 0; k0 < p.k; k0 += kOrdChunk) {
#pragma unroll
            for (uint32_t u = 0; u < kPer; u++) {
                const uint32_t i = tid + u * kOrdThreads;
                if (i >= (kOrdRows + kOrdCols) * (kOrdChunk / 8)) continue;
                const bool is_x = i < kOrdRows * (kOrdChunk / 8);
                const uint32_t j = is_x ? i : i - kOrdRows * (kOrdChunk / 8);
                const uint32_t r = j / (kOrdChunk / 8), at = (j % (kOrdChunk / 8)) * 8;
                float f[8];
                widen8(held[u], f);
                float *to = is_x ? &xs[r][at] : &ws[r][at];
                *reinterpret_cast<float4 *>(to) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4 *>(to + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
            __syncthreads();
            if (k0 + kOrdChunk < p.k) ask(k0 + kOrdChunk);   // in flight under the sums below
            const uint32_t len = min(kOrdChunk, p.k - k0);
            if (len == kOrdChunk) {
#pragma unroll 8
                for (uint32_t j = 0; j < kOrdChunk; j += 4) {
                    const float4 a = *reinterpret_cast<const float4 *>(&xs[ty][j]);
                    const float4 b = *reinterpret_cast<const float4 *>(&ws[tx][j]);
                    sum = __fadd_rn(sum, __fmul_rn(a.x, b.x));
                    sum = __fadd_rn(sum, __fmul_rn(a.y, b.y));
                    sum = __fadd_rn(sum, __fmul_rn(a.z, b.z));
                    sum = __fadd_rn(sum, __fmul_rn(a.w, b.w));
                }
            } else {
                for (uint32_t j = 0; j < len; j++) sum = __fadd_rn(sum, __fmul_rn(xs[ty][j], ws[tx][j]));
            }
            __syncthreads();
        }
    } else {
        for (uint32_t k0 = 0; k0 < p.k; k0 += kOrdChunk) {
            const uint32_t len = min(kOrdChunk, p.k - k0);
            for (uint32_t i = tid; i < kOrdRows * kOrdChunk; i += kOrdThreads) {
                const uint32_t r = i / kOrdChunk, j = i % kOrdChunk;
                xs[r][j] = (row0 + r < p.m && j < len) ? widen(p.x[(size_t)(row0 + r) * p.k + k0 + j]) : 0.0f;
            }
            for (uint32_t i = tid; i < kOrdCols * kOrdChunk; i += kOrdThreads) {
                const uint32_t c = i / kOrdChunk, j = i % kOrdChunk;
                ws[c][j] = (col0 + c < p.n && j < len) ? widen(p.w[(size_t)(col0 + c) * p.k + k0 + j]) : 0.0f;
            }
            __syncthreads();
            for (uint32_t j = 0; j < len; j++) sum = __fadd_rn(sum, __fmul_rn(xs[ty][j], ws[tx][j]));
            __syncthreads();
        }
    }
    pdl_launch_dependents();
    const uint32_t row = row0 + ty, col = col0 + tx;
    if (row < p.m && col < p.n) {
        const size_t i = (size_t)row * p.n + col;
        float v = sum;
        if (p.epilogue == TS_EPI_ADD) v = __fadd_rn(v, p.a0[i]);
        else if (p.epilogue == TS_EPI_SCALE) v = __fmul_rn(v, p.scale);
        if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[i] = v;
        else reinterpret_cast<uint16_t *>(p.out)[i] = bf16_bits(v);
    }
}

}  // namespace

bool ordered_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    return m > 0 && n > 0 && k > 0 && epilogue != TS_EPI_SWIGLU && epilogue != TS_EPI_GEGLU;
}

int linear_ordered(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                   int epilogue, float scale, int out_dtype, cudaStream_t stream) {
    PlainParams p = {(const uint16_t *)x, (const uint16_t *)w, (const float *)a0, out, m, n, k, epilogue, out_dtype, scale};
    const dim3 grid(ceil_div(n, kOrdCols), ceil_div(m, kOrdRows));
    const bool vec = k % 8 == 0 && aligned16(x) && aligned16(w);
    cudaError_t e = vec ? launch(linear_ordered_kernel<true>, grid, dim3(kOrdThreads), 0, stream, pdl_enabled(), p)
                        : launch(linear_ordered_kernel<false>, grid, dim3(kOrdThreads), 0, stream, pdl_enabled(), p);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_ordered failed: %s (%d) %s", cudaGetErrorName(e), (int)e, cudaGetErrorString(e));
    return TS_OK;
}

bool plain_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    return m > 0 && n > 0 && k > 0 && (!gated || n % 2 == 0);
}

int linear_plain(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                 int epilogue, float scale, int out_dtype, cudaStream_t stream) {
    PlainParams p = {(const uint16_t *)x, (const uint16_t *)w, (const float *)a0, out, m, n, k, epilogue, out_dtype, scale};
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    const size_t total = (size_t)m * (gated ? n / 2 : n);
    uint32_t blocks = (uint32_t)std::min<size_t>((total + 7) / 8, (size_t)sm_count() * 16);
    if (blocks == 0) blocks = 1;
    cudaError_t e = launch(linear_plain_kernel, dim3(blocks), dim3(256), 0, stream, pdl_enabled(), p);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_plain failed: %s (%d) %s", cudaGetErrorName(e), (int)e, cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
