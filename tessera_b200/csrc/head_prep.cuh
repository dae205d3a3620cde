// Per-head preparation between the q,k,v projection and attention, shared by the stand-alone append
// kernel and the fused decode attention so that both produce the same bits.
// Norm: engine/ir/interp/src/cpu.rs:371-377; rotation with half pairs (j, j + width/2), angle =
// position * inv_freq[j]: cpu.rs:31-47.
#pragma once

#include "ts_common.cuh"

namespace ts {

// One warp per head.  Lane l owns the pairs j = l * PER + e (e < PER = WIDTH / 64): elements j and
// j + WIDTH / 2 of the head.  `gain` NULL: no norm.  Leaves the rotated values as bf16 bits in lo[e]
// (element j) and hi[e] (element j + WIDTH / 2).
template <int WIDTH>
__device__ __forceinline__ void norm_rope_head(const uint16_t *src, const float *gain, const float *inv_freq, uint32_t pos,
                                               float eps, uint32_t lane, uint16_t (&lo)[WIDTH / 64],
                                               uint16_t (&hi)[WIDTH / 64]) {
    constexpr int PER = WIDTH / 64;
    float a[PER], b[PER];
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < PER; e++) {
        const uint32_t j = lane * PER + e;
        a[e] = __uint_as_float((uint32_t)src[j] << 16);
        b[e] = __uint_as_float((uint32_t)src[j + WIDTH / 2] << 16);
        ss = fmaf(a[e], a[e], ss);
        ss = fmaf(b[e], b[e], ss);
    }
    if (gain) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)WIDTH + eps);
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const uint32_t j = lane * PER + e;
            a[e] = a[e] * (inv * gain[j]);
            b[e] = b[e] * (inv * gain[j + WIDTH / 2]);
        }
    }
#pragma unroll
    for (int e = 0; e < PER; e++) {
        const uint32_t j = lane * PER + e;
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        lo[e] = bf16_bits(a[e] * cs - b[e] * sn);
        hi[e] = bf16_bits(a[e] * sn + b[e] * cs);
    }
}

}  // namespace ts
