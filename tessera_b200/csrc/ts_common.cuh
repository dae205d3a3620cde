// Shared host/device helpers for the tessera_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "tessera_b200.h"

namespace ts {

// Records the failure text for ts_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);

#define TS_REQUIRE(cond, ...)                                         \
    do {                                                              \
        if (!(cond)) return ts::fail(TS_ERR_BAD_INPUT, __VA_ARGS__);  \
    } while (0)

#define TS_CUDA(expr)                                                                          \
    do {                                                                                       \
        cudaError_t err__ = (expr);                                                            \
        if (err__ != cudaSuccess)                                                              \
            return ts::fail(TS_ERR_CUDA, "%s failed: %s (%d) %s", #expr, cudaGetErrorName(err__), \
                            (int)err__, cudaGetErrorString(err__));                            \
    } while (0)

// A failed launch reads like the reference's Error::Launch(step, kernel, cause).
#define TS_LAUNCHED(name)                                                                       \
    do {                                                                                        \
        cudaError_t err__ = cudaGetLastError();                                                 \
        if (err__ != cudaSuccess)                                                               \
            return ts::fail(TS_ERR_CUDA, "launch of %s failed: %s (%d) %s", name,               \
                            cudaGetErrorName(err__), (int)err__, cudaGetErrorString(err__));    \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

// SM count of the current device, cached per device ordinal.
int sm_count();

// Ordinal of the current device (0 when there is none).
int current_device();

// "Set up once" record for state CUDA keeps per device (a kernel's dynamic shared-memory limit, a symbol's
// address): one bit per device ordinal, safe to use from several host threads.  needs() is true until done()
// ran with that device current; two threads racing through the set-up both do it, which is harmless.
class OncePerDevice {
public:
    bool needs() const {
        const int d = current_device();
        return ((mask_[(d >> 6) & 3].load(std::memory_order_acquire) >> (d & 63)) & 1u) == 0;
    }
    void done() {
        const int d = current_device();
        mask_[(d >> 6) & 3].fetch_or(1ull << (d & 63), std::memory_order_release);
    }

private:
    std::atomic<uint64_t> mask_[4] = {};
};

// ---- device helpers -------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ uint16_t bf16_bits(float x) {
    __nv_bfloat16 v = __float2bfloat16_rn(x);
    return *reinterpret_cast<uint16_t *>(&v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// x / (1 + e^-x) and the tanh GELU, as engine/ir/interp/src/cpu.rs:9-23 writes them.
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
    const float coef = 0.7978846f;
    return 0.5f * x * (1.0f + tanhf(coef * (x + 0.044715f * x * x * x)));
}

// Programmatic dependent launch: wait for the upstream grid's memory, and let the
// downstream grid start its prologue (engine/plan/codegen/src/dialect.rs:77-84 does the same).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Kept-row address: engine/plan/codegen/src/kept.rs:135-194.
struct KeptDev {
    int kind;
    uint32_t shift;   // log2 page
    uint32_t scalar;  // kept_stride | kept_slots | kept_pages
    const uint32_t *table;
};

__device__ __forceinline__ uint32_t kept_row(const KeptDev &k, uint32_t slot, uint32_t position) {
    if (k.kind == TS_KEPT_DENSE) return slot * k.scalar + position;
    if (k.kind == TS_KEPT_INTERLEAVED) return position * k.scalar + slot;
    uint32_t page = k.table[(uint64_t)slot * k.scalar + (position >> k.shift)];
    return (page << k.shift) | (position & ((1u << k.shift) - 1u));
}

// Host-side check + conversion of a ts_kept.  Returns TS_OK or records the failure.
int kept_to_dev(const ts_kept *kept, KeptDev *out);

// Launch with the programmatic-stream-serialization attribute when `pdl` is set.
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                   bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Whether launches carry the PDL attribute (process-wide switch; off by default).
bool pdl_enabled();

}  // namespace ts

// Debug builds only (-DTS_DEBUG_STAMPS): per-block %globaltimer stamps, the reference's TS_MARK idea
// (engine/plan/run/src/marks.cuh).  Compiled out of the shipped library.
#ifdef TS_DEBUG_STAMPS
static __device__ unsigned long long g_stamps[16 * 32];  // one copy per translation unit
#ifndef TS_STAMP_X
#define TS_STAMP_X blockIdx.x   /* -DTS_STAMP_X='(gridDim.x - 1 - blockIdx.x)' stamps the last blocks instead of the first */
#endif
#define STAMP(slot)                                                         \
    do {                                                                    \
        const unsigned bx__ = TS_STAMP_X;                                   \
        if (bx__ < 4 && blockIdx.y < 4) {                                   \
            unsigned long long t__;                                         \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));         \
            g_stamps[(bx__ * 4 + blockIdx.y) * 32 + (slot)] = t__;          \
        }                                                                   \
    } while (0)
#else
#define STAMP(slot) do { } while (0)
#endif
