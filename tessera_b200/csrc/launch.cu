// Launch by the reference's kernel names, with arguments in the reference's order.
//
// tessera's runner turns every planned `Launch { args, shape }` into device pointers and scalar words in the
// kernel's parameter order: read buffers, the output buffer, the page table if the kept layout has one, then
// u32 / f32 scalars, with the layout's own scalars last (engine/plan/lower/src/abi.rs:11-18, 148-153;
// engine/plan/lower/src/rule.rs:62-109; engine/plan/run/src/device.rs:91-104).  ts_launch takes exactly that
// list under the kernel's name, checks it against the kernel's signature before anything runs, and calls the
// typed entry point.  What the reference keeps outside the argument list stays outside here too: the kept
// layout is part of the kernel's name (`attend_rows_paged16`, as in `plan_attend_rows_{layout}`,
// engine/rules/attention/src/attend.rs:182-186), the head width of a whole-sequence kernel likewise
// (`flash_128`, engine/rules/attention/src/flash.rs:648-651), and queries arrive already scaled (the reference
// scales them in a `map` launch of its own, engine/rules/attention/src/lib.rs:22-31).  Activations are bf16
// where the typed entry points say so.
#include <cstring>

#include "ts_common.cuh"
#include "ts_kernels.cuh"

namespace ts {
namespace {

struct Args {
    const ts_arg *a;
    const void *ptr(int i) const { return a[i].v.ptr; }
    uint32_t u(int i) const { return a[i].v.u32; }
    float f(int i) const { return a[i].v.f32; }
};

typedef int (*RunFn)(const Args &, int nargs, const ts_shape *, int variant, void *ws, size_t ws_bytes, void *stream);
typedef size_t (*WsFn)(const Args &, int nargs, const ts_shape *, int variant);

// m of a linear is not an argument in the reference (it is a build parameter and shows in the launch shape):
// five arguments take it from shape->down, six carry it before n.
int run_linear(const Args &a, int nargs, const ts_shape *shape, int, void *ws, size_t ws_bytes, void *stream) {
    const bool with_m = nargs == 6;
    TS_REQUIRE(with_m || (shape && shape->down > 0), "ts_launch: a linear with five arguments needs its rows in shape->down");
    const uint32_t m = with_m ? a.u(3) : shape->down, n = a.u(with_m ? 4 : 3), k = a.u(with_m ? 5 : 4);
    return ts_linear_bf16(a.ptr(0), a.ptr(1), nullptr, const_cast<void *>(a.ptr(2)), m, n, k, TS_EPI_NONE, 1.0f, TS_BF16,
                          TS_LINEAR_AUTO, ws, ws_bytes, stream);
}
size_t ws_linear(const Args &a, int nargs, const ts_shape *shape, int) {
    const bool with_m = nargs == 6;
    const uint32_t m = with_m ? a.u(3) : (shape ? shape->down : 0);
    return ts_linear_workspace_bytes(m, a.u(with_m ? 4 : 3), a.u(with_m ? 5 : 4), TS_EPI_NONE, TS_LINEAR_AUTO);
}

// variant: 0 dense, 1 interleaved, 2 paged (64), 3 paged16
ts_kept kept_of(int variant, const void *table, uint32_t scalar, uint32_t table_len) {
    ts_kept k = {};
    k.kind = variant == 0 ? TS_KEPT_DENSE : variant == 1 ? TS_KEPT_INTERLEAVED : TS_KEPT_PAGED;
    k.page = variant == 3 ? 16 : 64;
    k.kept_scalar = scalar;
    k.table = (const uint32_t *)table;
    k.table_len = table_len;
    return k;
}

// q, k, v, out, slots, positions, [table], queries, keys, heads, kv_heads, width, back, <layout scalar>
int run_attend_rows(const Args &a, int, const ts_shape *, int variant, void *ws, size_t ws_bytes, void *stream) {
    const int t = variant >= 2 ? 1 : 0;  // a page table sits after the last buffer
    const ts_kept kept = kept_of(variant, t ? a.ptr(6) : nullptr, a.u(12 + t), 0);
    return ts_attend_rows_bf16(a.ptr(0), a.ptr(1), a.ptr(2), const_cast<void *>(a.ptr(3)), (const uint32_t *)a.ptr(4),
                               (const uint32_t *)a.ptr(5), &kept, a.u(6 + t), a.u(7 + t), a.u(8 + t), a.u(9 + t), a.u(10 + t),
                               a.u(11 + t), 1.0f, ws, ws_bytes, stream);
}
size_t ws_attend_rows(const Args &a, int, const ts_shape *, int variant) {
    const int t = variant >= 2 ? 1 : 0;
    return ts_attend_rows_workspace_bytes(a.u(6 + t), a.u(7 + t), a.u(8 + t), a.u(9 + t), a.u(10 + t));
}

// x, slots, positions, out, [table], rows, width, <layout scalar>
int run_scatter(const Args &a, int, const ts_shape *, int variant, void *, size_t, void *stream) {
    const int t = variant >= 2 ? 1 : 0;
    const ts_kept kept = kept_of(variant, t ? a.ptr(4) : nullptr, a.u(6 + t), 0);
    return ts_scatter_bf16(a.ptr(0), (const uint32_t *)a.ptr(1), (const uint32_t *)a.ptr(2), const_cast<void *>(a.ptr(3)), &kept,
                           a.u(4 + t), a.u(5 + t), stream);
}

// x (f32), out (u32 ids), rows, width, k
int run_top_k(const Args &a, int, const ts_shape *, int, void *ws, size_t ws_bytes, void *stream) {
    return ts_top_k(a.ptr(0), TS_F32, (uint32_t *)const_cast<void *>(a.ptr(1)), a.u(2), a.u(3), a.u(4), ws, ws_bytes, stream);
}
size_t ws_top_k(const Args &a, int, const ts_shape *, int) { return ts_top_k_workspace_bytes(a.u(2), a.u(3), a.u(4)); }

// x (f32), w (f32), out, rows, width, eps; variant 0: f32 out (as the reference), 1: bf16 out
int run_lane_norm(const Args &a, int, const ts_shape *, int variant, void *, size_t, void *stream) {
    return ts_rms_norm(a.ptr(0), TS_F32, (const float *)a.ptr(1), const_cast<void *>(a.ptr(2)), variant ? TS_BF16 : TS_F32, a.u(3),
                       a.u(4), a.f(5), stream);
}

// One sequence: q, k, v, out, queries, keys, past, heads, kv_heads, back, ahead; variant = head width
int run_flash(const Args &a, int, const ts_shape *, int variant, void *ws, size_t ws_bytes, void *stream) {
    const uint32_t queries = a.u(4), keys = a.u(5), past = a.u(6);
    TS_REQUIRE(past == (keys > queries ? keys - queries : 0), "ts_launch: flash: past = %u does not equal keys - queries", past);
    return ts_attend_bf16(a.ptr(0), a.ptr(1), a.ptr(2), const_cast<void *>(a.ptr(3)), nullptr, 1, queries, keys, a.u(7), a.u(8),
                          (uint32_t)variant, a.u(9), a.u(10), 1.0f, ws, ws_bytes, stream);
}

// x, w, ids, out, rows, n, k, count, stride, offset, repeat, first (engine/rules/linear/src/picked.rs:28-41); x and w bf16
int run_picked(const Args &a, int, const ts_shape *, int, void *ws, size_t ws_bytes, void *stream) {
    return ts_picked_bf16(a.ptr(0), a.ptr(1), (const uint32_t *)a.ptr(2), (float *)const_cast<void *>(a.ptr(3)), a.u(4), a.u(5),
                          a.u(6), a.u(7), a.u(8), a.u(9), a.u(10), a.u(11), ws, ws_bytes, stream);
}
size_t ws_picked(const Args &a, int, const ts_shape *, int) { return ts_picked_workspace_bytes(a.u(4), a.u(5), a.u(6), a.u(7)); }

// positions, out, count, width, theta, turned (engine/rules/kernels/src/rope.rs:36-44)
int run_angles(const Args &a, int, const ts_shape *, int, void *, size_t, void *stream) {
    return ts_rope_angles((const uint32_t *)a.ptr(0), (float *)const_cast<void *>(a.ptr(1)), a.u(2), a.u(3), a.f(4), a.u(5), stream);
}

// x (in place), freqs, positions, heads, width (rope.rs:10-16); variant bit 0: adjacent pairs, bit 1: bf16 rows
int run_rope(const Args &a, int, const ts_shape *, int variant, void *, size_t, void *stream) {
    return ts_rope(const_cast<void *>(a.ptr(0)), (variant & 2) ? TS_BF16 : TS_F32, (const float *)a.ptr(1), a.u(2), a.u(3), a.u(4),
                   variant & 1, stream);
}

struct Entry {
    const char *name;
    const char *signature;  // p = device pointer, u = u32, f = f32, in the reference's order
    const char *alt;        // a second accepted signature, or NULL
    int order;              // 0 = Order::Fixed (same bits in any batch), 1 = Order::PerConfig
    int variant;
    RunFn run;
    WsFn ws;
};

const Entry kTable[] = {
    {"lanes_bf16", "pppuu", "pppuuu", 1, 0, run_linear, ws_linear},
    {"thin_bf16", "pppuu", "pppuuu", 1, 0, run_linear, ws_linear},
    {"tiled_bf16", "pppuu", "pppuuu", 1, 0, run_linear, ws_linear},
    {"parts_bf16", "pppuu", "pppuuu", 1, 0, run_linear, ws_linear},
    {"attend_rows_dense", "ppppppuuuuuuu", nullptr, 1, 0, run_attend_rows, ws_attend_rows},
    {"attend_rows_interleaved", "ppppppuuuuuuu", nullptr, 1, 1, run_attend_rows, ws_attend_rows},
    {"attend_rows_paged", "pppppppuuuuuuu", nullptr, 1, 2, run_attend_rows, ws_attend_rows},
    {"attend_rows_paged16", "pppppppuuuuuuu", nullptr, 1, 3, run_attend_rows, ws_attend_rows},
    {"flash_rows_dense", "ppppppuuuuuuu", nullptr, 1, 0, run_attend_rows, ws_attend_rows},
    {"flash_rows_paged", "pppppppuuuuuuu", nullptr, 1, 2, run_attend_rows, ws_attend_rows},
    {"flash_rows_paged16", "pppppppuuuuuuu", nullptr, 1, 3, run_attend_rows, ws_attend_rows},
    {"scatter_dense", "ppppuuu", nullptr, 0, 0, run_scatter, nullptr},
    {"scatter_interleaved", "ppppuuu", nullptr, 0, 1, run_scatter, nullptr},
    {"scatter_paged", "pppppuuu", nullptr, 0, 2, run_scatter, nullptr},
    {"scatter_paged16", "pppppuuu", nullptr, 0, 3, run_scatter, nullptr},
    {"top_k", "ppuuu", nullptr, 0, 0, run_top_k, ws_top_k},
    {"lane_norm", "pppuuf", nullptr, 1, 0, run_lane_norm, nullptr},
    {"lane_norm_bf16", "pppuuf", nullptr, 1, 1, run_lane_norm, nullptr},
    {"picked_bf16", "ppppuuuuuuuu", nullptr, 1, 0, run_picked, ws_picked},
    {"angles", "ppuufu", nullptr, 1, 0, run_angles, nullptr},
    {"rope", "ppuuu", nullptr, 0, 0, run_rope, nullptr},
    {"rope_adjacent", "ppuuu", nullptr, 0, 1, run_rope, nullptr},
    {"rope_bf16", "ppuuu", nullptr, 0, 2, run_rope, nullptr},
    {"rope_adjacent_bf16", "ppuuu", nullptr, 0, 3, run_rope, nullptr},
    {"flash_128", "ppppuuuuuuu", nullptr, 1, 128, run_flash, nullptr},
    {"flash_256", "ppppuuuuuuu", nullptr, 1, 256, run_flash, nullptr},
};
constexpr int kEntries = (int)(sizeof(kTable) / sizeof(kTable[0]));

bool matches(const char *signature, const ts_arg *args, int nargs) {
    if (!signature || (int)strlen(signature) != nargs) return false;
    for (int i = 0; i < nargs; i++) {
        const int want = signature[i] == 'p' ? TS_ARG_PTR : signature[i] == 'u' ? TS_ARG_U32 : TS_ARG_F32;
        if (args[i].kind != want) return false;
        if (want == TS_ARG_PTR && args[i].v.ptr == nullptr) return false;
    }
    return true;
}

const Entry *find(const char *kernel) {
    for (int i = 0; i < kEntries; i++)
        if (strcmp(kTable[i].name, kernel) == 0) return &kTable[i];
    return nullptr;
}

int resolve(const char *kernel, const ts_arg *args, int nargs, const Entry **out) {
    TS_REQUIRE(kernel != nullptr, "ts_launch: the kernel name is NULL");
    const Entry *e = find(kernel);
    TS_REQUIRE(e != nullptr, "ts_launch: no kernel is called `%s`", kernel);
    TS_REQUIRE(nargs >= 0 && (nargs == 0 || args != nullptr), "ts_launch: %s: NULL argument list", kernel);
    TS_REQUIRE(matches(e->signature, args, nargs) || matches(e->alt, args, nargs),
               "ts_launch: %s takes `%s`%s%s (p = device pointer, u = u32, f = f32), got %d arguments of other kinds or a NULL "
               "pointer",
               kernel, e->signature, e->alt ? " or `" : "", e->alt ? e->alt : "", nargs);
    *out = e;
    return TS_OK;
}

}  // namespace
}  // namespace ts

using namespace ts;

#pragma GCC visibility push(default)
extern "C" {

int ts_kernel_count(void) { return kEntries; }

int ts_kernel_info_at(int index, ts_kernel_info *out) {
    TS_REQUIRE(out != nullptr && index >= 0 && index < kEntries, "ts_kernel_info_at: index %d is outside 0..%d", index, kEntries - 1);
    out->name = kTable[index].name;
    out->signature = kTable[index].signature;
    out->order = kTable[index].order;
    return TS_OK;
}

size_t ts_launch_workspace_bytes(const char *kernel, const ts_arg *args, int nargs, const ts_shape *shape) {
    const Entry *e = nullptr;
    if (resolve(kernel, args, nargs, &e) != TS_OK || !e->ws) return 0;
    return e->ws(Args{args}, nargs, shape, e->variant);
}

int ts_launch(const char *kernel, const ts_arg *args, int nargs, const ts_shape *shape, void *workspace, size_t workspace_bytes,
              void *stream) {
    const Entry *e = nullptr;
    int rc = resolve(kernel, args, nargs, &e);
    if (rc != TS_OK) return rc;
    return e->run(Args{args}, nargs, shape, e->variant, workspace, workspace_bytes, stream);
}

}  // extern "C"
#pragma GCC visibility pop
