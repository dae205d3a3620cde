// Decode-sized linear over Q8_0 weights: out[m, n] = sum_k x[m, k] * w[n, k], w in the reference's Q8_0 block form
// (engine/ir/mem/src/block.rs:259-260: per 32 elements an f16 scale, then 32 signed bytes; 34 bytes a block,
// blocks along k), x bf16, sums f32.  A decode step is bound by the weight bytes it streams: 34 bytes per 32
// weights instead of 64.
//
// The arithmetic follows the form's own dot product (block.rs:204-221): inside a block the plain sum of x times
// code, then the block's scale, blocks added in order.  The codes are small integers, exact in bf16, so a block's
// partial is two warp MMAs (m16n8k16, bf16 in, f32 out) on the raw codes - no weight is ever rounded - and the
// scale meets the partial in f32.  What differs from the checker is only the order of the f32 sums inside the MMA.
//
// A block of four warps owns 64 weight rows and a k slice; a warp owns 16 of the rows against all (up to 64)
// batch rows.  k is cut over blocks so that the launch covers the SMs; the slices' f32 partials meet in
// linear_reduce_kernel in ascending order, which also applies the epilogue stage (add, scale, SwiGLU / GeGLU) -
// the rules' fused stage chain (engine/plan/lower/src/sites/matmul.rs:148-176).
//
// Also here: the host-side packer and unpacker of the form (block.rs:223-258), for callers that hold f32 weights.
#include <cuda_fp16.h>

#include <cmath>
#include <cstring>

#include "ts_common.cuh"
#include "ts_kernels.cuh"

namespace ts {

int launch_linear_reduce(const float *partial, uint32_t splits, const float *a0, void *out, uint32_t m, uint32_t n,
                         int epilogue, float scale, int out_dtype, cudaStream_t stream);

namespace {

constexpr uint32_t kRowsPerBlock = 64;      // weight rows: 4 warps x 16
constexpr uint32_t kChunk = 256;            // k per staging round: 8 Q8_0 blocks = 272 bytes a row (a multiple of 16)
constexpr uint32_t kChunkBytes = kChunk / 32 * 34;
constexpr uint32_t kBatch = 64;
constexpr uint32_t kXStride = kChunk + 8;   // bf16 per staged x row: 528 bytes, so 8 rows land on 8 different banks
constexpr uint32_t kThreads = 128;
constexpr uint32_t kSmem = kRowsPerBlock * kChunkBytes + kBatch * kXStride * 2;

struct Q8Params {
    const uint16_t *x;
    const uint8_t *w;
    float *partial;  // [splits][m][n]
    uint32_t m, n, k, chunks, splits;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// two signed bytes (the low 16 bits of `pair`) as two bf16: both exact
__device__ __forceinline__ uint32_t codes_to_bf16x2(uint32_t pair) {
    const float lo = (float)(int8_t)(pair & 0xFF), hi = (float)(int8_t)((pair >> 8) & 0xFF);
    return pack_bf16(lo, hi);
}

__global__ void __launch_bounds__(kThreads) linear_q8_kernel(const Q8Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *ws = smem;                                                      // [64][272] raw blocks
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + kRowsPerBlock * kChunkBytes);  // [64][kXStride]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t row0 = blockIdx.x * kRowsPerBlock, split = blockIdx.y;
    const uint32_t c0 = (uint32_t)(((uint64_t)split * p.chunks) / p.splits), c1 = (uint32_t)(((uint64_t)(split + 1) * p.chunks) / p.splits);
    const size_t row_bytes = (size_t)(p.k / 32) * 34;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    pdl_wait();
    for (uint32_t c = c0; c < c1; c++) {
        // stage the chunk: 64 weight rows x 272 bytes and up to 64 batch rows x 256 bf16, 16 bytes a load
        for (uint32_t i = threadIdx.x; i < kRowsPerBlock * (kChunkBytes / 16); i += kThreads) {
            const uint32_t r = i / (kChunkBytes / 16), piece = i % (kChunkBytes / 16);
            *reinterpret_cast<uint4 *>(ws + r * kChunkBytes + piece * 16) =
                __ldg(reinterpret_cast<const uint4 *>(p.w + (size_t)(row0 + r) * row_bytes + (size_t)c * kChunkBytes + piece * 16));
        }
        for (uint32_t i = threadIdx.x; i < kBatch * (kChunk / 8); i += kThreads) {
            const uint32_t r = i / (kChunk / 8), piece = i % (kChunk / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < p.m) v = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)r * p.k + (size_t)c * kChunk + piece * 8));
            *reinterpret_cast<uint4 *>(xs + r * kXStride + piece * 8) = v;
        }
        __syncthreads();
        const unsigned char *wa = ws + (warp * 16 + g) * kChunkBytes, *wb = wa + 8 * kChunkBytes;  // rows g and g + 8
#pragma unroll 1
        for (uint32_t blk = 0; blk < kChunk / 32; blk++) {
            const float sa = __half2float(*reinterpret_cast<const __half *>(wa + blk * 34));
            const float sb = __half2float(*reinterpret_cast<const __half *>(wb + blk * 34));
            float part[8][4];
#pragma unroll
            for (int i = 0; i < 8; i++) part[i][0] = part[i][1] = part[i][2] = part[i][3] = 0.0f;
#pragma unroll
            for (uint32_t half = 0; half < 2; half++) {
                const uint32_t kk = half * 16 + 2 * t;   // within the block
                uint32_t a[4];
                a[0] = codes_to_bf16x2(*reinterpret_cast<const uint16_t *>(wa + blk * 34 + 2 + kk));
                a[1] = codes_to_bf16x2(*reinterpret_cast<const uint16_t *>(wb + blk * 34 + 2 + kk));
                a[2] = codes_to_bf16x2(*reinterpret_cast<const uint16_t *>(wa + blk * 34 + 2 + kk + 8));
                a[3] = codes_to_bf16x2(*reinterpret_cast<const uint16_t *>(wb + blk * 34 + 2 + kk + 8));
                const uint16_t *xb = xs + g * kXStride + blk * 32 + kk;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xb + i * 8 * kXStride);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xb + i * 8 * kXStride + 8);
                    mma_16816(part[i], a, b0, b1);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                acc[i][0] = fmaf(sa, part[i][0], acc[i][0]);
                acc[i][1] = fmaf(sa, part[i][1], acc[i][1]);
                acc[i][2] = fmaf(sb, part[i][2], acc[i][2]);
                acc[i][3] = fmaf(sb, part[i][3], acc[i][3]);
            }
        }
        __syncthreads();
    }
    pdl_launch_dependents();
    // acc[i][0,1]: weight row g, batch rows 8 i + 2 t, + 1; acc[i][2,3]: weight row g + 8
    float *out = p.partial + (size_t)split * p.m * p.n;
    const uint32_t na = row0 + warp * 16 + g, nb = na + 8;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t m0 = 8 * i + 2 * t;
        if (m0 < p.m) {
            out[(size_t)m0 * p.n + na] = acc[i][0];
            out[(size_t)m0 * p.n + nb] = acc[i][2];
        }
        if (m0 + 1 < p.m) {
            out[(size_t)(m0 + 1) * p.n + na] = acc[i][1];
            out[(size_t)(m0 + 1) * p.n + nb] = acc[i][3];
        }
    }
}

uint32_t q8_splits(uint32_t n, uint32_t k) {
    const uint32_t tiles = n / kRowsPerBlock, chunks = k / kChunk;
    uint32_t want = ceil_div(2 * (uint32_t)sm_count(), tiles ? tiles : 1);
    return std::max<uint32_t>(1, std::min<uint32_t>(want, chunks));
}

}  // namespace

bool q8_0_supports(uint32_t m, uint32_t n, uint32_t k) {
    return m >= 1 && m <= kBatch && n % kRowsPerBlock == 0 && n > 0 && k % kChunk == 0 && k > 0;
}

size_t q8_0_workspace_bytes(uint32_t m, uint32_t n, uint32_t k) {
    if (!q8_0_supports(m, n, k)) return 0;
    return (size_t)q8_splits(n, k) * m * n * sizeof(float);
}

int linear_q8_0(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k, int epilogue,
                float scale, int out_dtype, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    TS_REQUIRE(q8_0_supports(m, n, k), "linear (q8_0): needs 1..64 rows, n in multiples of 64 and k in multiples of 256 (m=%u n=%u k=%u)",
               m, n, k);
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    TS_REQUIRE(!gated || n % 2 == 0, "linear (q8_0): a gated epilogue needs an even n");
    const size_t need = q8_0_workspace_bytes(m, n, k);
    TS_REQUIRE(workspace && workspace_bytes >= need, "linear (q8_0): workspace of %zu bytes is smaller than the %zu needed",
               workspace_bytes, need);
    Q8Params p = {(const uint16_t *)x, (const uint8_t *)w, (float *)workspace, m, n, k, k / kChunk, q8_splits(n, k)};
    static OncePerDevice configured;
    if (configured.needs()) {
        TS_CUDA(cudaFuncSetAttribute(linear_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
        configured.done();
    }
    cudaError_t e = launch(linear_q8_kernel, dim3(n / kRowsPerBlock, p.splits), dim3(kThreads), kSmem, stream, pdl_enabled(), p);
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_q8 failed: %s (%d) %s", cudaGetErrorName(e), (int)e, cudaGetErrorString(e));
    return launch_linear_reduce(p.partial, p.splits, (const float *)a0, out, m, n, epilogue, scale, out_dtype, stream);
}

// ---- the form on the host: Block<F16, I8, 32>::pack / unpack (block.rs:223-258) --------------------------------

size_t q8_0_bytes(size_t elements) { return (elements + 31) / 32 * 34; }

void q8_0_pack(const float *data, size_t elements, uint8_t *out) {
    memset(out, 0, q8_0_bytes(elements));
    for (size_t b = 0; b * 32 < elements; b++) {
        const size_t n = std::min<size_t>(32, elements - b * 32);
        float top = 0.0f;
        for (size_t j = 0; j < n; j++) top = std::max(top, std::fabs(data[b * 32 + j]));
        const __half scale = __float2half_rn(top / 127.0f);
        uint8_t *at = out + b * 34;
        memcpy(at, &scale, 2);
        const float stored = __half2float(scale);  // the codes see the scale as it was stored
        for (size_t j = 0; j < n; j++) {
            const float scaled = stored == 0.0f ? 0.0f : data[b * 32 + j] / stored;
            const float r = std::min(127.0f, std::max(-128.0f, std::nearbyint(scaled)));  // ties to even
            at[2 + j] = (uint8_t)(int8_t)r;
        }
    }
}

void q8_0_unpack(const uint8_t *bytes, size_t elements, float *out) {
    for (size_t i = 0; i < elements; i++) {
        const uint8_t *at = bytes + i / 32 * 34;
        __half scale;
        memcpy(&scale, at, 2);
        out[i] = __half2float(scale) * (float)(int8_t)at[2 + i % 32];
    }
}

}  // namespace ts
