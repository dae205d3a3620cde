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

}  // namespace

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
