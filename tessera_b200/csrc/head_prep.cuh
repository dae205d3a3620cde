// Per-head preparation between the q,k,v projection and attention, shared by the stand-alone append
// kernel and the fused decode attention so that both produce the same bits.
// Norm: engine/ir/interp/src/cpu.rs:371-377; rotation with half pairs (j, j + width/2), angle =
// position * inv_freq[j]: cpu.rs:31-47.
#pragma once

#include "ts_common.cuh"

namespace ts {

// What a head's preparation needs besides the head itself, for a lane: the cosines and sines of its PER pairs'
// angles (position * inv_freq[j], j = lane * PER + e) and, with a norm, the gains of its 2 PER elements
// (g[e]: element j, g[PER + e]: element j + WIDTH / 2).  None of it depends on the projection, so a kernel may
// fetch and compute it while it still waits for the projection's launch to finish.
template <int WIDTH>
struct HeadTurn {
    float cs[WIDTH / 64], sn[WIDTH / 64];
};

template <int WIDTH>
__device__ __forceinline__ HeadTurn<WIDTH> head_turn(const float *inv_freq, uint32_t pos, uint32_t lane) {
    HeadTurn<WIDTH> t;
#pragma unroll
    for (int e = 0; e < WIDTH / 64; e++) sincosf((float)pos * inv_freq[lane * (WIDTH / 64) + e], &t.sn[e], &t.cs[e]);
    return t;
}

template <int WIDTH>
__device__ __forceinline__ void head_gains(const float *gain, uint32_t lane, float (&g)[WIDTH / 32]) {
    constexpr int PER = WIDTH / 64;
#pragma unroll
    for (int e = 0; e < PER; e++) {
        g[e] = gain ? gain[lane * PER + e] : 1.0f;
        g[PER + e] = gain ? gain[lane * PER + e + WIDTH / 2] : 1.0f;
    }
}

// One warp per head.  Lane l owns the pairs j = l * PER + e (e < PER = WIDTH / 64): elements j and
// j + WIDTH / 2 of the head.  `normed` false: no norm (g is not read).  Leaves the rotated values as bf16 bits in
// lo[e] (element j) and hi[e] (element j + WIDTH / 2).
template <int WIDTH>
__device__ __forceinline__ void norm_rope_head_with(const uint16_t *src, bool normed, const float (&g)[WIDTH / 32],
                                                    const HeadTurn<WIDTH> &turn, float eps, uint32_t lane,
                                                    uint16_t (&lo)[WIDTH / 64], uint16_t (&hi)[WIDTH / 64]) {
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
    if (normed) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)WIDTH + eps);
#pragma unroll
        for (int e = 0; e < PER; e++) {
            a[e] = a[e] * (inv * g[e]);
            b[e] = b[e] * (inv * g[PER + e]);
        }
    }
#pragma unroll
    for (int e = 0; e < PER; e++) {
        lo[e] = bf16_bits(a[e] * turn.cs[e] - b[e] * turn.sn[e]);
        hi[e] = bf16_bits(a[e] * turn.sn[e] + b[e] * turn.cs[e]);
    }
}

// The same with the gains and the angles fetched here.  `gain` NULL: no norm.
template <int WIDTH>
__device__ __forceinline__ void norm_rope_head(const uint16_t *src, const float *gain, const float *inv_freq, uint32_t pos,
                                               float eps, uint32_t lane, uint16_t (&lo)[WIDTH / 64],
                                               uint16_t (&hi)[WIDTH / 64]) {
    float g[WIDTH / 32];
    head_gains<WIDTH>(gain, lane, g);
    const HeadTurn<WIDTH> turn = head_turn<WIDTH>(inv_freq, pos, lane);
    norm_rope_head_with<WIDTH>(src, gain != nullptr, g, turn, eps, lane, lo, hi);
}

}  // namespace ts
