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
    // the lane's PER consecutive elements of each half in one load
    uint16_t ra[PER], rb[PER];
    if constexpr (PER == 4) {
        const uint2 va = *reinterpret_cast<const uint2 *>(src + lane * 4);
        const uint2 vb = *reinterpret_cast<const uint2 *>(src + WIDTH / 2 + lane * 4);
        ra[0] = va.x & 0xFFFF; ra[1] = va.x >> 16; ra[2] = va.y & 0xFFFF; ra[3] = va.y >> 16;
        rb[0] = vb.x & 0xFFFF; rb[1] = vb.x >> 16; rb[2] = vb.y & 0xFFFF; rb[3] = vb.y >> 16;
    } else if constexpr (PER == 2) {
        const uint32_t va = *reinterpret_cast<const uint32_t *>(src + lane * 2);
        const uint32_t vb = *reinterpret_cast<const uint32_t *>(src + WIDTH / 2 + lane * 2);
        ra[0] = va & 0xFFFF; ra[1] = va >> 16;
        rb[0] = vb & 0xFFFF; rb[1] = vb >> 16;
    } else {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            ra[e] = src[lane * PER + e];
            rb[e] = src[lane * PER + e + WIDTH / 2];
        }
    }
#pragma unroll
    for (int e = 0; e < PER; e++) {
        a[e] = __uint_as_float((uint32_t)ra[e] << 16);
        b[e] = __uint_as_float((uint32_t)rb[e] << 16);
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
