// Second pass of a split-k linear: adds the f32 partial sums of the k slices in ascending slice
// order (a fixed order, so a re-run gives the same bits) and applies the epilogue stage.
#include "ts_common.cuh"

namespace ts {
namespace {

struct ReduceParams {
    const float *partial;  // [splits, m, n]
    const float *a0;
    void *out;
    uint32_t splits, m, n;
    int epilogue, out_dtype;
    float scale;
};

__global__ void __launch_bounds__(256) linear_reduce_kernel(const ReduceParams p) {
    pdl_wait();
    const bool gated = p.epilogue == TS_EPI_SWIGLU || p.epilogue == TS_EPI_GEGLU;
    const uint32_t out_n = gated ? p.n / 2 : p.n;
    const size_t total = (size_t)p.m * out_n;
    const size_t plane = (size_t)p.m * p.n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t m = (uint32_t)(i / out_n), n = (uint32_t)(i % out_n);
        float v;
        if (gated) {
            float gsum = 0.0f, usum = 0.0f;
            for (uint32_t s = 0; s < p.splits; s++) {
                gsum += p.partial[s * plane + (size_t)m * p.n + n];
                usum += p.partial[s * plane + (size_t)m * p.n + out_n + n];
            }
            v = (p.epilogue == TS_EPI_SWIGLU ? silu(gsum) : gelu_tanh(gsum)) * usum;
        } else {
            float sum = 0.0f;
            for (uint32_t s = 0; s < p.splits; s++) sum += p.partial[s * plane + (size_t)m * p.n + n];
            v = sum;
            if (p.epilogue == TS_EPI_ADD) v += p.a0[i];
            if (p.epilogue == TS_EPI_SCALE) v *= p.scale;
        }
        if (p.out_dtype == TS_F32) reinterpret_cast<float *>(p.out)[i] = v;
        else reinterpret_cast<uint16_t *>(p.out)[i] = bf16_bits(v);
    }
    pdl_launch_dependents();
}

}  // namespace

int launch_linear_reduce(const float *partial, uint32_t splits, const float *a0, void *out, uint32_t m,
                         uint32_t n, int epilogue, float scale, int out_dtype, cudaStream_t stream) {
    ReduceParams p = {partial, a0, out, splits, m, n, epilogue, out_dtype, scale};
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    size_t total = (size_t)m * (gated ? n / 2 : n);
    uint32_t blocks = (uint32_t)std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 8);
    if (blocks == 0) blocks = 1;
    cudaError_t e = launch(linear_reduce_kernel, dim3(blocks), dim3(256), 0, stream, pdl_enabled(), p);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_reduce failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    return TS_OK;
}

}  // namespace ts
