// Decode-sized linear: out[m, n] = sum_k x[m, k] * w[n, k] for m <= 64.
//
// The weight matrix is read exactly once, straight from HBM into registers with 16-byte
// loads, in the operand layout of the warp MMA (m16n8k16, bf16 in, f32 sums): a weight row
// is an MMA row, a batch row is an MMA column.  The k order inside one 32-wide step is
// permuted the same way for both operands (thread t of a quad owns k = 8t..8t+7), which
// leaves every dot product unchanged and lets each thread fetch 8 consecutive k with one
// load.  The activations x (a few KB to 128 KB) are staged once per block in shared memory.
//
// Work is cut into tasks of 32 weight rows x one k slice; the warps of all blocks take
// tasks round-robin and keep `DEPTH` steps of weight loads in flight across task
// boundaries.  With more than one k slice the f32 partial sums go to the caller's
// workspace and a second kernel adds the slices in ascending order (a fixed tree, so a
// re-run gives the same bits) and applies the epilogue.
//
// Stands in for the reference's `lanes` and `thin` rules
// (engine/rules/linear/src/lanes.rs:20-65, thin.rs:31-55).
#include "ts_common.cuh"

namespace ts {

int launch_linear_reduce(const float *partial, uint32_t splits, const float *a0, void *out, uint32_t m,
                         uint32_t n, int epilogue, float scale, int out_dtype, cudaStream_t stream);

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kXPad = 64;  // bytes; keeps the 8 rows of a 16-byte smem read phase on distinct banks

struct SkinnyParams {
    const uint16_t *x;
    const uint16_t *w;
    const float *a0;
    void *out;
    float *partial;  // [splits, m, n] when splits > 1
    uint32_t m, n, k;
    uint32_t ks;      // k per slice, a multiple of 32 * DEPTH
    uint32_t splits;
    uint32_t tiles;   // tasks along n
    uint32_t pair_stride;  // rows between the two 16-row halves of a task: 16, or n/2 for gated epilogues
    uint32_t rows;    // weight rows a task's first half may start at: n, or n/2 for gated epilogues
    int epilogue;
    int out_dtype;
    float scale;
};

__device__ __forceinline__ uint4 ldg_stream(const uint16_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float epilogue_value(const SkinnyParams &p, float acc, uint32_t m, uint32_t n) {
    if (p.epilogue == TS_EPI_ADD) return acc + p.a0[(size_t)m * p.n + n];
    if (p.epilogue == TS_EPI_SCALE) return acc * p.scale;
    return acc;
}

__device__ __forceinline__ void store_pair(const SkinnyParams &p, size_t at, float lo, float hi, bool both,
                                           bool aligned) {
    if (p.out_dtype == TS_F32) {
        float *o = reinterpret_cast<float *>(p.out) + at;
        if (both && aligned) {
            *reinterpret_cast<float2 *>(o) = make_float2(lo, hi);
        } else {
            o[0] = lo;
            if (both) o[1] = hi;
        }
    } else {
        uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + at;
        if (both && aligned) {
            *reinterpret_cast<uint32_t *>(o) = pack_bf16(lo, hi);
        } else {
            o[0] = bf16_bits(lo);
            if (both) o[1] = bf16_bits(hi);
        }
    }
}

// NT: batch columns / 8.  DEPTH: k steps of weight loads in flight per warp.
template <int NT, int DEPTH>
__global__ void __launch_bounds__(kThreads, 1) linear_skinny_kernel(const SkinnyParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t split = blockIdx.y;
    const uint32_t k0 = split * p.ks;
    const uint32_t steps = p.ks / 32;
    const uint32_t xs_stride = p.ks * 2 + kXPad;  // bytes
    const bool gated = p.epilogue == TS_EPI_SWIGLU || p.epilogue == TS_EPI_GEGLU;

    // Task order: every warp of the grid walks tasks first, first + stride, ...
    const uint32_t first = blockIdx.x * kWarps + warp;
    const uint32_t stride = gridDim.x * kWarps;

    // Weight rows this thread feeds into MMA rows g and g + 8 of each half: 2g and 2g + 1, so a
    // thread's two sums for one batch column are neighbours in the output row.
    auto row_of = [&](uint32_t task, int half) -> uint32_t {
        uint32_t base = gated ? task * 16 : task * 32;
        uint32_t r = base + half * p.pair_stride + 2 * g;
        return r;
    };

    uint4 a[DEPTH][2][2];
    uint32_t ld_task = first, ld_step = 0;
    auto issue = [&](uint4 (&dst)[2][2]) {
        if (ld_task < p.tiles) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t r0 = row_of(ld_task, half);
                uint32_t limit = p.n - 1;
                const uint16_t *at = p.w + (size_t)k0 + ld_step * 32 + t * 8;
                dst[half][0] = ldg_stream(at + (size_t)min(r0, limit) * p.k);
                dst[half][1] = ldg_stream(at + (size_t)min(r0 + 1, limit) * p.k);
            }
            if (++ld_step == steps) {
                ld_step = 0;
                ld_task += stride;
            }
        }
    };

    // Weights do not depend on the upstream kernel: start streaming before waiting on it.
#pragma unroll
    for (int d = 0; d < DEPTH; d++) issue(a[d]);

    pdl_wait();

    // Stage x[:, k0 .. k0 + ks) (rows past m read as zero).
    {
        const uint32_t vec_per_row = p.ks / 8;
        for (uint32_t i = threadIdx.x; i < NT * 8 * vec_per_row; i += kThreads) {
            uint32_t r = i / vec_per_row, c = i % vec_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < p.m) v = *reinterpret_cast<const uint4 *>(p.x + (size_t)r * p.k + k0 + c * 8);
            *reinterpret_cast<uint4 *>(smem + (size_t)r * xs_stride + c * 16) = v;
        }
    }
    __syncthreads();
    pdl_launch_dependents();

    const unsigned char *xs_thread = smem + (size_t)g * xs_stride + t * 16;

    for (uint32_t task = first; task < p.tiles; task += stride) {
        float acc[2][NT][4];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[h][j][c] = 0.0f;

        for (uint32_t s0 = 0; s0 < steps; s0 += DEPTH) {
#pragma unroll
            for (int d = 0; d < DEPTH; d++) {
                const unsigned char *xk = xs_thread + (s0 + d) * 64;
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    uint4 b = *reinterpret_cast<const uint4 *>(xk + (size_t)j * 8 * xs_stride);
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        mma_bf16(acc[h][j], a[d][h][0].x, a[d][h][1].x, a[d][h][0].y, a[d][h][1].y, b.x, b.y);
                        mma_bf16(acc[h][j], a[d][h][0].z, a[d][h][1].z, a[d][h][0].w, a[d][h][1].w, b.z, b.w);
                    }
                }
                issue(a[d]);
            }
        }

        // acc[h][j][0,1]: weight row 2g of half h, batch columns 8j + 2t, + 1; acc[h][j][2,3]: row 2g + 1.
        if (p.splits > 1) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t n0 = row_of(task, h);
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint32_t m = j * 8 + 2 * t + c;
                        if (m < p.m && n0 < p.n) {
                            float *o = p.partial + ((size_t)split * p.m + m) * p.n + n0;
                            if (n0 + 1 < p.n && (p.n & 1) == 0) {
                                *reinterpret_cast<float2 *>(o) = make_float2(acc[h][j][c], acc[h][j][2 + c]);
                            } else {
                                o[0] = acc[h][j][c];
                                if (n0 + 1 < p.n) o[1] = acc[h][j][2 + c];
                            }
                        }
                    }
            }
        } else if (gated) {
            const uint32_t half_n = p.n / 2;
            uint32_t n0 = row_of(task, 0);
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t m = j * 8 + 2 * t + c;
                    if (m < p.m && n0 < half_n) {
                        float g0 = acc[0][j][c], g1 = acc[0][j][2 + c];
                        float u0 = acc[1][j][c], u1 = acc[1][j][2 + c];
                        float lo = (p.epilogue == TS_EPI_SWIGLU ? silu(g0) : gelu_tanh(g0)) * u0;
                        float hi = (p.epilogue == TS_EPI_SWIGLU ? silu(g1) : gelu_tanh(g1)) * u1;
                        store_pair(p, (size_t)m * half_n + n0, lo, hi, n0 + 1 < half_n, (half_n & 1) == 0);
                    }
                }
        } else {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t n0 = row_of(task, h);
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint32_t m = j * 8 + 2 * t + c;
                        if (m < p.m && n0 < p.n) {
                            bool both = n0 + 1 < p.n;
                            float lo = epilogue_value(p, acc[h][j][c], m, n0);
                            float hi = both ? epilogue_value(p, acc[h][j][2 + c], m, n0 + 1) : 0.0f;
                            store_pair(p, (size_t)m * p.n + n0, lo, hi, both, (p.n & 1) == 0);
                        }
                    }
            }
        }
    }
}

struct SkinnyPlan {
    uint32_t nt, splits, ks, tiles, blocks;
    size_t smem;
};

// Picks the k split: enough tasks to give every warp of the machine a few, slices a multiple
// of 256 k, and an x slice that fits shared memory.
SkinnyPlan plan_skinny(uint32_t m, uint32_t n, uint32_t k, bool gated) {
    SkinnyPlan s;
    s.nt = m <= 8 ? 1 : m <= 16 ? 2 : m <= 32 ? 4 : 8;
    uint32_t rows = gated ? n / 2 : n;
    s.tiles = gated ? ceil_div(rows, 16) : ceil_div(rows, 32);
    const uint32_t unit = 256;  // k granule of a slice: 32 * the deepest DEPTH
    // Partial sums cost splits * m * n * 8 bytes of extra traffic; keep that under a quarter of
    // the weight bytes (n * k * 2).
    uint32_t max_splits = min(k / unit, max(1u, k / (16 * m)));
    uint32_t want = (uint32_t)sm_count() * kWarps;
    uint32_t splits = 1;
    while (splits < max_splits && s.tiles * splits < want && (k / unit) % (splits * 2) == 0) splits *= 2;
    // shared memory bound on the x slice
    const size_t limit = 200 * 1024;
    while ((size_t)s.nt * 8 * ((k / splits) * 2 + kXPad) > limit && (k / unit) % (splits * 2) == 0) splits *= 2;
    s.splits = splits;
    s.ks = k / splits;
    s.smem = (size_t)s.nt * 8 * (s.ks * 2 + kXPad);
    uint32_t per_split = ceil_div((uint32_t)sm_count(), 1);
    s.blocks = min(ceil_div(s.tiles, kWarps), per_split);
    if (s.blocks == 0) s.blocks = 1;
    return s;
}

}  // namespace

size_t skinny_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, bool gated) {
    if (m == 0 || m > 64 || k % 256 != 0) return 0;
    SkinnyPlan s = plan_skinny(m, n, k, gated);
    return s.splits > 1 ? (size_t)s.splits * m * n * sizeof(float) : 0;
}

bool skinny_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    if (m == 0 || m > 64 || k % 256 != 0 || k == 0) return false;
    if (gated && (n % 32 != 0)) return false;
    SkinnyPlan s = plan_skinny(m, n, k, gated);
    return s.smem <= 200 * 1024;
}

template <int NT, int DEPTH>
static cudaError_t launch_skinny(const SkinnyParams &p, const SkinnyPlan &s, cudaStream_t stream) {
    auto kernel = linear_skinny_kernel<NT, DEPTH>;
    static OncePerDevice configured;
    if (configured.needs()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured.done();
    }
    return launch(kernel, dim3(s.blocks, s.splits), dim3(kThreads), s.smem, stream, pdl_enabled(), p);
}

int linear_skinny(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                  int epilogue, float scale, int out_dtype, void *workspace, size_t workspace_bytes,
                  cudaStream_t stream) {
    bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    SkinnyPlan s = plan_skinny(m, n, k, gated);
    size_t need = s.splits > 1 ? (size_t)s.splits * m * n * sizeof(float) : 0;
    TS_REQUIRE(workspace_bytes >= need && (need == 0 || workspace != nullptr),
               "linear (skinny): workspace of %zu bytes is smaller than the %zu needed", workspace_bytes, need);
    SkinnyParams p;
    p.x = (const uint16_t *)x;
    p.w = (const uint16_t *)w;
    p.a0 = (const float *)a0;
    p.out = out;
    p.partial = (float *)workspace;
    p.m = m;
    p.n = n;
    p.k = k;
    p.ks = s.ks;
    p.splits = s.splits;
    p.tiles = s.tiles;
    p.pair_stride = gated ? n / 2 : 16;
    p.rows = gated ? n / 2 : n;
    p.epilogue = epilogue;
    p.out_dtype = out_dtype;
    p.scale = scale;
    cudaError_t e;
    switch (s.nt) {
    case 1: e = launch_skinny<1, 8>(p, s, stream); break;
    case 2: e = launch_skinny<2, 8>(p, s, stream); break;
    case 4: e = launch_skinny<4, 8>(p, s, stream); break;
    default: e = launch_skinny<8, 4>(p, s, stream); break;
    }
    if (e != cudaSuccess)
        return fail(TS_ERR_CUDA, "launch of linear_skinny failed: %s (%d) %s", cudaGetErrorName(e), (int)e,
                    cudaGetErrorString(e));
    if (s.splits > 1)
        return launch_linear_reduce((const float *)workspace, s.splits, (const float *)a0, out, m, n, epilogue, scale,
                                    out_dtype, stream);
    return TS_OK;
}

}  // namespace ts
