// The C ABI: argument checks on the host, then a launch.  Nothing here synchronises or allocates.
#include <cstdarg>
#include <cstring>
#include <cstdlib>
#include <mutex>

#include "ts_common.cuh"
#include "ts_kernels.cuh"
#include "ts_ptx.cuh"

namespace ts {

// ---- error text, device facts, switches ----
static thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
    return dev;
}

int sm_count() {
    static std::atomic<int> cached[256] = {};
    const int dev = current_device() & 255;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            return 148;  // B200; only reached without a device, where nothing launches anyway
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

static thread_local bool g_pdl = false;  // per host thread: a runner on another thread keeps its own setting
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool enabled) { g_pdl = enabled; }

int kept_to_dev(const ts_kept *kept, KeptDev *out) {
    TS_REQUIRE(kept != nullptr, "kept layout is NULL");
    TS_REQUIRE(kept->kind >= TS_KEPT_DENSE && kept->kind <= TS_KEPT_PAGED, "kept layout kind %d is unknown", kept->kind);
    out->kind = kept->kind;
    out->scalar = kept->kept_scalar;
    out->shift = 0;
    out->table = kept->table;
    if (kept->kind == TS_KEPT_PAGED) {
        TS_REQUIRE(kept->page >= 1 && (kept->page & (kept->page - 1)) == 0, "page of %u rows is not a power of two",
                   kept->page);
        TS_REQUIRE(kept->table != nullptr, "a paged layout needs its page table");
        uint32_t shift = 0;
        while ((1u << shift) < kept->page) shift++;
        out->shift = shift;
    }
    return TS_OK;
}

// ---- tensor maps ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int make_tensor_map_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                       uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a %llu x %llu tensor, box %u x %u", (int)r,
                    (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
    return TS_OK;
}

int make_tensor_map_2d_plain(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                             uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a plain %llu x %llu tensor, box %u x %u", (int)r,
                    (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
    return TS_OK;
}

int make_tensor_map_3d(CUtensorMap *map, const void *base, uint64_t outer, uint64_t rows, uint64_t cols,
                       uint64_t outer_stride, uint64_t row_stride, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {cols, rows, outer};
    cuuint64_t strides[2] = {row_stride * 2, outer_stride * 2};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed (%d)", (int)r);
    return TS_OK;
}

// TS_LINEAR_PAIR=0 keeps AUTO on the one-SM tiled kernel (for A/B timing).
static bool pair_auto() {
    static const bool off = [] {
        const char *v = getenv("TS_LINEAR_PAIR");
        return v && v[0] == '0';
    }();
    return !off;
}

int pick_linear_path(uint32_t m, uint32_t n, uint32_t k, int epilogue, int path) {
    if (path == TS_LINEAR_SKINNY || path == TS_LINEAR_UMMA || path == TS_LINEAR_STREAM || path == TS_LINEAR_PAIR ||
        path == TS_LINEAR_PLAIN || path == TS_LINEAR_ORDERED)
        return path;
    // m <= 16: the warp-MMA streamer; m <= 128: the weight-streaming tcgen05 kernel with its cluster
    // reduce; larger m: the tiled tcgen05 kernel.
    if (m <= 16 && skinny_supports(m, n, k, epilogue)) return TS_LINEAR_SKINNY;
    if (m <= 128 && stream_supports(m, n, k, epilogue)) return TS_LINEAR_STREAM;
    if (pair_auto() && pair_supports(m, n, k, epilogue)) return TS_LINEAR_PAIR;
    if (umma_supports(m, n, k, epilogue)) return TS_LINEAR_UMMA;
    if (skinny_supports(m, n, k, epilogue)) return TS_LINEAR_SKINNY;
    if (plain_supports(m, n, k, epilogue)) return TS_LINEAR_PLAIN;  // k off the 64 grid and the like
    return -1;
}

}  // namespace ts

using namespace ts;

#pragma GCC visibility push(default)
extern "C" {

const char *ts_last_error(void) { return g_error; }
int ts_abi_version(void) { return TS_ABI_VERSION; }

int ts_set_pdl(int enabled) {
    g_pdl = enabled != 0;
    return TS_OK;
}

int ts_device_status(void) {
    const int a = umma_take_status(), b = stream_take_status(), c = flash_take_status(), d = moe_take_status();
    const int e = rows_take_status(), f = pair_take_status(), g = step_take_status();
    return a ? a : b ? b : c ? c : d ? d : e ? e : f ? f : g;
}

size_t ts_q8_0_bytes(size_t elements) { return q8_0_bytes(elements); }

int ts_q8_0_pack(const float *data, size_t elements, void *out) {
    TS_REQUIRE(data && out, "q8_0 pack: NULL argument");
    q8_0_pack(data, elements, (uint8_t *)out);
    return TS_OK;
}

int ts_q8_0_unpack(const void *bytes, size_t elements, float *out) {
    TS_REQUIRE(bytes && out, "q8_0 unpack: NULL argument");
    q8_0_unpack((const uint8_t *)bytes, elements, out);
    return TS_OK;
}

size_t ts_linear_q8_0_workspace_bytes(uint32_t m, uint32_t n, uint32_t k) { return q8_0_workspace_bytes(m, n, k); }

int ts_linear_q8_0(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k, int epilogue,
                   float scale, int out_dtype, void *workspace, size_t workspace_bytes, void *stream) {
    TS_REQUIRE(x && w && out, "linear (q8_0): x, w and out must not be NULL");
    TS_REQUIRE(aligned16(x) && aligned16(w) && aligned16(out), "linear (q8_0): x, w and out must be 16-byte aligned");
    TS_REQUIRE(epilogue >= TS_EPI_NONE && epilogue <= TS_EPI_GEGLU, "linear (q8_0): epilogue %d is unknown", epilogue);
    TS_REQUIRE(out_dtype == TS_BF16 || out_dtype == TS_F32, "linear (q8_0): out dtype %d is unknown", out_dtype);
    TS_REQUIRE(epilogue != TS_EPI_ADD || a0 != nullptr, "linear (q8_0): the add epilogue needs its operand");
    return linear_q8_0(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, workspace, workspace_bytes, (cudaStream_t)stream);
}

int ts_wait_runs_out(uint64_t wait_ns, void *stream) {
    TS_REQUIRE(wait_ns > 0 && wait_ns <= 1000000000ull, "wait_runs_out: the bound must be within (0, 1 s]");
    return wait_runs_out(wait_ns, (cudaStream_t)stream);
}

size_t ts_linear_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, int epilogue, int path) {
    const bool gated = epilogue == TS_EPI_SWIGLU || epilogue == TS_EPI_GEGLU;
    size_t a = 0, b = 0;
    const bool any = path == TS_LINEAR_AUTO;
    if ((any || path == TS_LINEAR_SKINNY) && skinny_supports(m, n, k, epilogue)) a = skinny_workspace_bytes(m, n, k, gated);
    if ((any || path == TS_LINEAR_UMMA) && umma_supports(m, n, k, epilogue)) b = umma_workspace_bytes(m, n, k, epilogue);
    return a > b ? a : b;
}

uint32_t ts_linear_sumsq_parts(uint32_t m, uint32_t n, uint32_t k, int epilogue) {
    if (pick_linear_path(m, n, k, epilogue, TS_LINEAR_AUTO) == TS_LINEAR_PAIR) return pair_sumsq_parts(m, n, k, epilogue);
    return stream_sumsq_parts(m, n, k, epilogue);
}

int ts_linear_fused_bf16(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                         int epilogue, float scale, int out_dtype, const ts_linear_fused *fused, void *stream) {
    TS_REQUIRE(w && out, "linear: w and out must not be NULL");
    TS_REQUIRE(aligned16(w) && aligned16(out), "linear: w and out must be 16-byte aligned");
    TS_REQUIRE(out_dtype == TS_BF16 || out_dtype == TS_F32, "linear: out_dtype %d is neither bf16 nor f32", out_dtype);
    TS_REQUIRE(epilogue != TS_EPI_ADD || a0 != nullptr, "linear: the ADD epilogue needs a0");
    StreamFused f;
    if (fused) {
        f.row_ss = fused->row_ss;
        f.row_parts = fused->row_parts;
        f.row_eps = fused->row_eps;
        f.ss_out = fused->ss_out;
        f.xs_out = fused->xs_out;
        f.xs_gain = fused->xs_gain;
    }
    TS_REQUIRE(x && aligned16(x), "linear: x is NULL or not 16-byte aligned");
    if (m == 0 || n == 0) return TS_OK;
    if (pick_linear_path(m, n, k, epilogue, TS_LINEAR_AUTO) == TS_LINEAR_PAIR)
        return linear_pair(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, (cudaStream_t)stream, &f);
    TS_REQUIRE(stream_supports(m, n, k, epilogue),
               "linear (fused): m=%u n=%u k=%u epilogue=%d fits neither the decode-sized nor the paired kernel", m, n, k, epilogue);
    return linear_stream(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, (cudaStream_t)stream, &f);
}

int ts_linear_bf16(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                   int epilogue, float scale, int out_dtype, int path, void *workspace, size_t workspace_bytes,
                   void *stream) {
    TS_REQUIRE(x && w && out, "linear: x, w and out must not be NULL");
    TS_REQUIRE(aligned16(x) && aligned16(w) && aligned16(out), "linear: x, w and out must be 16-byte aligned");
    TS_REQUIRE(epilogue >= TS_EPI_NONE && epilogue <= TS_EPI_GEGLU, "linear: epilogue %d is unknown", epilogue);
    TS_REQUIRE(out_dtype == TS_BF16 || out_dtype == TS_F32, "linear: out dtype %d is unknown", out_dtype);
    TS_REQUIRE(epilogue != TS_EPI_ADD || a0 != nullptr, "linear: the add epilogue needs its operand");
    TS_REQUIRE(a0 == nullptr || aligned16(a0), "linear: the epilogue operand must be 16-byte aligned");
    TS_REQUIRE(k > 0, "linear: k is zero");
    TS_REQUIRE(path >= TS_LINEAR_AUTO && path <= TS_LINEAR_ORDERED, "linear: path %d is unknown", path);
    if (m == 0 || n == 0) return TS_OK;
    const int chosen = pick_linear_path(m, n, k, epilogue, path);
    TS_REQUIRE(chosen > 0, "linear: no kernel takes m=%u n=%u k=%u epilogue=%d", m, n, k, epilogue);
    cudaStream_t s = (cudaStream_t)stream;
    if (chosen == TS_LINEAR_SKINNY) {
        TS_REQUIRE(skinny_supports(m, n, k, epilogue), "linear (skinny): needs m <= 64 and k %% 256 == 0 (m=%u k=%u)", m,
                   k);
        return linear_skinny(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, workspace, workspace_bytes, s);
    }
    if (chosen == TS_LINEAR_STREAM) {
        TS_REQUIRE(stream_supports(m, n, k, epilogue), "linear (stream): needs m <= 128 (m=%u n=%u k=%u)", m, n, k);
        return linear_stream(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, s);
    }
    if (chosen == TS_LINEAR_PAIR) {
        TS_REQUIRE(pair_supports(m, n, k, epilogue), "linear (pair): needs m >= 512 and n >= 256 (m=%u n=%u k=%u)", m, n, k);
        return linear_pair(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, s);
    }
    if (chosen == TS_LINEAR_ORDERED) {
        TS_REQUIRE(ordered_supports(m, n, k, epilogue), "linear (ordered): gated epilogues are not offered in the fixed order");
        return linear_ordered(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, s);
    }
    if (chosen == TS_LINEAR_PLAIN) {
        TS_REQUIRE(plain_supports(m, n, k, epilogue), "linear (plain): a gated epilogue needs an even n (n=%u)", n);
        return linear_plain(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, s);
    }
    TS_REQUIRE(umma_supports(m, n, k, epilogue), "linear (umma): needs k in multiples of 64 (m=%u n=%u k=%u)", m, n, k);
    return linear_umma(x, w, a0, out, m, n, k, epilogue, scale, out_dtype, workspace, workspace_bytes, s);
}

static int check_kept(const ts_kept *kept, KeptDev *dev, bool *contiguous) {
    int rc = kept_to_dev(kept, dev);
    if (rc != TS_OK) return rc;
    *contiguous = kept->kind == TS_KEPT_DENSE || (kept->kind == TS_KEPT_PAGED && kept->page >= 32);
    return TS_OK;
}

size_t ts_attend_rows_workspace_bytes(uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads,
                                      uint32_t width) {
    return attend_rows_workspace_bytes(rows, keys, heads, kv_heads, width);
}

int ts_attend_rows_bf16(const void *q, const void *k, const void *v, void *out, const uint32_t *slots,
                        const uint32_t *positions, const ts_kept *kept, uint32_t rows, uint32_t keys,
                        uint32_t heads, uint32_t kv_heads, uint32_t width, uint32_t back, float scale,
                        void *workspace, size_t workspace_bytes, void *stream) {
    TS_REQUIRE(q && k && v && out && slots && positions, "attend_rows: a buffer is NULL");
    TS_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), "attend_rows: buffers must be 16-byte aligned");
    TS_REQUIRE(width == 16 || width == 32 || width == 64 || width == 128 || width == 256,
               "attend_rows: width %u is not 16, 32, 64, 128 or 256", width);
    TS_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attend_rows: %u heads do not split over %u kv heads", heads, kv_heads);
    KeptDev dev;
    bool contiguous;
    int rc = check_kept(kept, &dev, &contiguous);
    if (rc != TS_OK) return rc;
    if (rows == 0 || keys == 0) return TS_OK;
    return attend_rows(q, k, v, out, slots, positions, dev, contiguous, rows, keys, heads, kv_heads, width, back, scale,
                       workspace, workspace_bytes, (cudaStream_t)stream, 0, nullptr, kept->rows);
}

int ts_attend_rows_append_bf16(const void *qkv, const float *q_norm, const float *k_norm, const float *inv_freq, void *k_rows,
                               void *v_rows, void *out, const uint32_t *slots, const uint32_t *positions,
                               const ts_kept *kept, uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads,
                               uint32_t width, float eps, float scale, void *workspace, size_t workspace_bytes,
                               void *stream) {
    TS_REQUIRE(qkv && inv_freq && k_rows && v_rows && out && slots && positions, "attend_rows_append: a buffer is NULL");
    TS_REQUIRE(aligned16(qkv) && aligned16(k_rows) && aligned16(v_rows) && aligned16(out),
               "attend_rows_append: buffers must be 16-byte aligned");
    TS_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attend_rows_append: %u heads do not split over %u kv heads", heads, kv_heads);
    KeptDev dev;
    bool contiguous;
    int rc = check_kept(kept, &dev, &contiguous);
    if (rc != TS_OK) return rc;
    TS_REQUIRE(attend_rows_fused_supports(contiguous, width, kept->rows),
               "attend_rows_append: needs head width 128 (got %u) and a dense or >= 32-row paged layout with kept->rows set",
               width);
    if (rows == 0 || keys == 0) return TS_OK;
    RowsFused f;
    f.qkv = qkv;
    f.q_norm = q_norm;
    f.k_norm = k_norm;
    f.inv_freq = inv_freq;
    f.eps = eps;
    return attend_rows(nullptr, k_rows, v_rows, out, slots, positions, dev, contiguous, rows, keys, heads, kv_heads, width,
                       0xFFFFFFFFu, scale, workspace, workspace_bytes, (cudaStream_t)stream, 0, nullptr, kept->rows, &f);
}

size_t ts_attend_workspace_bytes(uint32_t seqs, uint32_t queries, uint32_t keys, uint32_t heads, uint32_t kv_heads,
                                 uint32_t width) {
    if (flash_supports(width)) return 0;
    // fallback: slot and position of every query row, then the rows kernel's own scratch
    const size_t rows = (size_t)seqs * queries;
    return align_up(rows * 8, 256) + attend_rows_workspace_bytes((uint32_t)rows, keys, heads, kv_heads, width);
}

int ts_attend_bf16(const void *q, const void *k, const void *v, void *out, const uint32_t *cu_seqlens, uint32_t seqs,
                   uint32_t queries, uint32_t keys, uint32_t heads, uint32_t kv_heads, uint32_t width, uint32_t back,
                   uint32_t ahead, float scale, void *workspace, size_t workspace_bytes, void *stream) {
    TS_REQUIRE(q && k && v && out, "attend: a buffer is NULL");
    TS_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), "attend: buffers must be 16-byte aligned");
    TS_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attend: %u heads do not split over %u kv heads", heads, kv_heads);
    TS_REQUIRE(scale > 0.0f, "attend: the score scale must be positive");
    if (seqs == 0 || queries == 0) return TS_OK;
    const bool causal = ahead == 0;
    TS_REQUIRE(!(causal && keys < queries && !cu_seqlens), "attend: %u queries, %u keys under a causal mask", queries,
               keys);  // engine/ir/interp/src/cpu.rs:62-68
    cudaStream_t s = (cudaStream_t)stream;
    if (flash_supports(width)) {
        // With cu_seqlens the rows are packed and `queries` bounds the longest sequence.
        const uint32_t total_q = cu_seqlens ? 0xFFFFFFFFu : seqs * queries;
        (void)total_q;
        return attend_flash(q, k, v, out, cu_seqlens, seqs, queries, keys, cu_seqlens ? keys : seqs * queries,
                            cu_seqlens ? keys : seqs * keys, heads, kv_heads, width, back, ahead, scale, s);
    }
    TS_REQUIRE(!cu_seqlens, "attend: packed sequences need width 128 or 256 (got %u)", width);
    TS_REQUIRE(width == 16 || width == 32 || width == 64, "attend: width %u is not 16, 32, 64, 128 or 256", width);
    const size_t rows = (size_t)seqs * queries;
    const size_t need = ts_attend_workspace_bytes(seqs, queries, keys, heads, kv_heads, width);
    TS_REQUIRE(workspace && workspace_bytes >= need, "attend: workspace of %zu bytes is smaller than the %zu needed",
               workspace_bytes, need);
    uint32_t *slots = (uint32_t *)workspace, *positions = slots + rows;
    const uint32_t past = keys > queries ? keys - queries : 0;
    int rc = iota_rows(slots, positions, seqs, queries, past, s);
    if (rc != TS_OK) return rc;
    KeptDev dense = {TS_KEPT_DENSE, 0, keys, nullptr};
    const size_t head = align_up(rows * 8, 256);
    return attend_rows(q, k, v, out, slots, positions, dense, true, (uint32_t)rows, keys, heads, kv_heads, width, back,
                       scale, (char *)workspace + head, workspace_bytes - head, s, ahead, nullptr);
}

int ts_scatter_bf16(const void *x, const uint32_t *slots, const uint32_t *positions, void *out, const ts_kept *kept,
                    uint32_t rows, uint32_t width, void *stream) {
    TS_REQUIRE(x && slots && positions && out, "scatter: a buffer is NULL");
    TS_REQUIRE(width % 8 == 0 && aligned16(x) && aligned16(out), "scatter: rows must be 16-byte multiples and aligned");
    KeptDev dev;
    bool contiguous;
    int rc = check_kept(kept, &dev, &contiguous);
    if (rc != TS_OK) return rc;
    return scatter_rows(x, slots, positions, out, dev, rows, width, (cudaStream_t)stream);
}

void ts_rope_inv_freq(float theta, uint32_t width, float *out) {
    // engine/ir/interp/src/cpu.rs:31-34: theta^(-2j / width), in f32
    for (uint32_t j = 0; j < width / 2; j++) out[j] = powf(theta, -((float)(2 * j)) / (float)width);
}

int ts_rope_angles(const uint32_t *positions, float *out, uint32_t count, uint32_t width, float theta, uint32_t turned,
                   void *stream) {
    TS_REQUIRE(positions && out, "rope angles: a buffer is NULL");
    TS_REQUIRE(((uintptr_t)out & 7) == 0, "rope angles: out must be 8-byte aligned");
    return rope_angles(positions, out, count, width, theta, turned, (cudaStream_t)stream);
}

int ts_rope(void *x, ts_dtype dtype, const float *freqs, uint32_t positions, uint32_t heads, uint32_t width, int adjacent,
            void *stream) {
    TS_REQUIRE(x && freqs, "rope: a buffer is NULL");
    TS_REQUIRE(dtype == TS_BF16 || dtype == TS_F32, "rope: dtype %d is neither bf16 nor f32", (int)dtype);
    TS_REQUIRE(((uintptr_t)freqs & 7) == 0, "rope: freqs must be 8-byte aligned");
    return rope(x, dtype, freqs, positions, heads, width, adjacent, (cudaStream_t)stream);
}

int ts_qk_norm_rope_append_bf16(const void *qkv, const float *q_norm, const float *k_norm, const float *inv_freq,
                                const uint32_t *slots, const uint32_t *positions, void *q_out, void *k_rows,
                                void *v_rows, const ts_kept *kept, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                                uint32_t width, float eps, void *stream) {
    TS_REQUIRE(qkv && inv_freq && slots && positions && q_out && k_rows && v_rows, "qk_norm_rope_append: a buffer is NULL");
    TS_REQUIRE(aligned16(qkv) && aligned16(q_out) && aligned16(k_rows) && aligned16(v_rows),
               "qk_norm_rope_append: buffers must be 16-byte aligned");
    KeptDev dev;
    bool contiguous;
    int rc = check_kept(kept, &dev, &contiguous);
    if (rc != TS_OK) return rc;
    return qk_norm_rope_append(qkv, q_norm, k_norm, inv_freq, slots, positions, q_out, k_rows, v_rows, dev, rows, heads,
                               kv_heads, width, eps, (cudaStream_t)stream);
}

int ts_rms_norm(const void *x, int x_dtype, const float *w, void *out, int out_dtype, uint32_t rows, uint32_t width,
                float eps, void *stream) {
    TS_REQUIRE(x && out, "rms_norm: a buffer is NULL");
    TS_REQUIRE((x_dtype == TS_BF16 || x_dtype == TS_F32) && (out_dtype == TS_BF16 || out_dtype == TS_F32),
               "rms_norm: unknown dtype");
    TS_REQUIRE(width > 0, "rms_norm: width is zero");
    return rms_norm(x, x_dtype, w, out, out_dtype, rows, width, eps, nullptr, (cudaStream_t)stream);
}

int ts_gather_bf16(const void *table, const uint32_t *ids, void *out, int out_dtype, uint32_t rows,
                   uint32_t table_rows, uint32_t width, uint32_t first, void *stream) {
    TS_REQUIRE(table && ids && out, "gather: a buffer is NULL");
    TS_REQUIRE(out_dtype == TS_BF16 || out_dtype == TS_F32, "gather: unknown dtype");
    return gather_rows(table, ids, out, out_dtype, rows, table_rows, width, first, (cudaStream_t)stream);
}

int ts_gather_scaled_bf16(const void *table, const uint32_t *ids, float *out, void *xs, const float *gain, float *ss,
                          uint32_t parts, uint32_t rows, uint32_t table_rows, uint32_t width, void *stream) {
    TS_REQUIRE(table && ids && out && xs && gain && ss, "gather (scaled): a buffer is NULL");
    return gather_scaled(table, ids, out, xs, gain, ss, parts, rows, table_rows, width, (cudaStream_t)stream);
}

size_t ts_top_k_workspace_bytes(uint32_t rows, uint32_t width, uint32_t k) {
    return top_k_workspace_bytes(rows, width, k);
}

int ts_top_k(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, uint32_t k, void *workspace,
             size_t workspace_bytes, void *stream) {
    TS_REQUIRE(x && ids, "top_k: a buffer is NULL");
    TS_REQUIRE(x_dtype == TS_BF16 || x_dtype == TS_F32, "top_k: unknown dtype");
    TS_REQUIRE(width > 0, "top_k: width is zero");
    return top_k(x, x_dtype, ids, rows, width, k, workspace, workspace_bytes, (cudaStream_t)stream);
}

int ts_top_1_static(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, void *stream) {
    TS_REQUIRE(x && ids, "top_1_static: a buffer is NULL");
    TS_REQUIRE(x_dtype == TS_BF16 || x_dtype == TS_F32, "top_1_static: unknown dtype");
    TS_REQUIRE(width > 0, "top_1_static: width is zero");
    return top_1_static(x, x_dtype, ids, rows, width, (cudaStream_t)stream);
}

int ts_mean_pool(const float *x, const uint32_t *cu_seqlens, float *out, uint32_t seqs, uint32_t width, int normalize,
                 void *stream) {
    TS_REQUIRE(x && cu_seqlens && out, "mean_pool: a buffer is NULL");
    TS_REQUIRE(width > 0, "mean_pool: width is zero");
    return mean_pool(x, cu_seqlens, out, seqs, width, normalize, (cudaStream_t)stream);
}

int ts_take_softmax(const float *x, const uint32_t *ids, float *gates, uint32_t rows, uint32_t width, uint32_t k,
                    void *stream) {
    TS_REQUIRE(x && ids && gates, "take_softmax: a buffer is NULL");
    TS_REQUIRE(k >= 1 && k <= 32, "take_softmax: k = %u is outside 1..32", k);
    return take_softmax(x, ids, gates, rows, width, k, (cudaStream_t)stream);
}

size_t ts_moe_workspace_bytes(uint32_t picks, uint32_t experts, uint32_t hidden, uint32_t ffn) {
    return moe_workspace_bytes(picks, experts, hidden, ffn);
}

static int check_moe(const void *x, const uint32_t *ids, const void *w_in, const void *w_out, const void *out,
                     uint32_t experts, uint32_t hidden, uint32_t ffn) {
    TS_REQUIRE(x && ids && w_in && w_out && out, "moe: a buffer is NULL");
    TS_REQUIRE(aligned16(x) && aligned16(w_in) && aligned16(w_out) && aligned16(out), "moe: buffers must be 16-byte aligned");
    TS_REQUIRE(experts >= 1 && experts <= 4096, "moe: %u experts is outside 1..4096", experts);
    TS_REQUIRE(hidden % 128 == 0 && ffn % 64 == 0, "moe: hidden must be a multiple of 128 and ffn of 64 (got %u, %u)",
               hidden, ffn);
    return TS_OK;
}

int ts_moe_experts_bf16(const void *x, const uint32_t *ids, const void *w_in, const void *w_out, float *out,
                        uint32_t picks, uint32_t repeat, uint32_t experts, uint32_t first, uint32_t hidden,
                        uint32_t ffn, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = check_moe(x, ids, w_in, w_out, out, experts, hidden, ffn);
    if (rc != TS_OK) return rc;
    TS_REQUIRE(repeat >= 1, "moe: repeat must be at least 1");
    if (picks == 0) return TS_OK;
    return moe_experts(x, ids, nullptr, nullptr, w_in, w_out, out, picks, repeat, 1, 0, experts, first, hidden, ffn,
                       workspace, workspace_bytes, (cudaStream_t)stream);
}

int ts_moe_bf16(const void *h, const uint32_t *ids, const float *gates, const float *add, const void *w_in,
                const void *w_out, float *y, uint32_t rows, uint32_t top, uint32_t experts, uint32_t first,
                uint32_t hidden, uint32_t ffn, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = check_moe(h, ids, w_in, w_out, y, experts, hidden, ffn);
    if (rc != TS_OK) return rc;
    TS_REQUIRE(gates != nullptr, "moe: gates is NULL");
    TS_REQUIRE(top >= 1 && top <= 32, "moe: top = %u is outside 1..32", top);
    if (rows == 0) return TS_OK;
    return moe_experts(h, ids, gates, add, w_in, w_out, y, rows * top, top, top, 1, experts, first, hidden, ffn, workspace,
                       workspace_bytes, (cudaStream_t)stream);
}

size_t ts_picked_workspace_bytes(uint32_t rows, uint32_t n, uint32_t k, uint32_t count) {
    return picked_workspace_bytes(rows, n, k, count);
}

int ts_picked_bf16(const void *x, const void *w, const uint32_t *ids, float *out, uint32_t rows, uint32_t n, uint32_t k,
                   uint32_t count, uint32_t stride, uint32_t offset, uint32_t repeat, uint32_t first, void *workspace,
                   size_t workspace_bytes, void *stream) {
    TS_REQUIRE(x && w && ids && out, "picked: a buffer is NULL");
    TS_REQUIRE(aligned16(x) && aligned16(w) && aligned16(out), "picked: buffers must be 16-byte aligned");
    TS_REQUIRE(count >= 1 && count <= 4096, "picked: %u matrices is outside 1..4096", count);
    return picked(x, w, ids, out, rows, n, k, count, stride, offset, repeat, first, workspace, workspace_bytes,
                  (cudaStream_t)stream);
}

int ts_moe_mix(const float *y_picks, const float *gates, const float *add, float *out, uint32_t rows, uint32_t top,
               uint32_t hidden, void *stream) {
    TS_REQUIRE(y_picks && gates && out, "moe mix: a buffer is NULL");
    TS_REQUIRE(top >= 1, "moe mix: top must be at least 1");
    return moe_mix(y_picks, gates, add, out, rows, top, hidden, (cudaStream_t)stream);
}

int ts_moe_permutation(const uint32_t *ids, uint32_t *order, uint32_t *place, uint32_t *offsets, uint32_t *batch_tiles,
                       uint32_t picks, uint32_t experts, uint32_t first, void *stream) {
    TS_REQUIRE(ids && order && place && offsets && batch_tiles, "moe permutation: a buffer is NULL");
    TS_REQUIRE(experts >= 1 && experts <= 4096, "moe: %u experts is outside 1..4096", experts);
    if (picks == 0) return TS_OK;
    return moe_permutation(ids, order, place, offsets, batch_tiles, picks, experts, first, (cudaStream_t)stream);
}

}  // extern "C"
#pragma GCC visibility pop
