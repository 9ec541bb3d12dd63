// Per-head RMSNorm + RoPE on a head held in registers, with the reference's exact
// instruction order (batched_attn.rs:13-118, 128-219).  Shared by the append kernel and by
// the decode kernel's fused item prologue, so both produce identical bytes.
#pragma once
#include "common.cuh"

namespace oxi {

// One warp normalises (and optionally rotates) one head held in registers.
// x[i] is dim lane + 32*i; wv / cv / sv are the norm weight, cos and sin of the same dims
// (already converted to f32 by the caller, which can fetch them early).  Returns the f16 bit
// patterns in out[i].
// Core on values already in registers: x[i] is dim lane + 32*i as f32, x16[i] its f16 bit pattern.
template <bool kNorm, bool kRope>
__device__ __forceinline__ void head_norm_rope_vals(const float (&x)[4], const uint16_t (&x16)[4], const float (&wv)[4],
                                                    float eps, const float (&cv)[4], const float (&sv)[4],
                                                    uint16_t (&out)[4]) {
    uint16_t y16[4];
    if (kNorm) {
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) sum = __fmaf_rn(x[i], x[i], sum);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
            sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, off));
        float mean = div_approx_ftz(sum, 128.0f);
        mean = __fadd_rn(mean, eps);
        float r = rsqrt_approx_ftz(mean);
        r = __shfl_sync(0xffffffffu, r, 0);
#pragma unroll
        for (int i = 0; i < 4; i++) y16[i] = f2h(__fmul_rn(__fmul_rn(x[i], r), wv[i]));
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) y16[i] = x16[i];
    }
    if (kRope) {
        float y[4];
#pragma unroll
        for (int i = 0; i < 4; i++) y[i] = h2f(y16[i]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // dim d = lane + 32 i pairs with d + 64 (i < 2) or d - 64 (i >= 2)
            const float other = (i < 2) ? -y[i + 2] : y[i - 2];
            float res = __fmul_rn(y[i], cv[i]);
            res = __fmaf_rn(other, sv[i], res);
            out[i] = f2h(res);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = y16[i];
    }
}

template <bool kNorm, bool kRope>
__device__ __forceinline__ void head_norm_rope(const uint16_t* __restrict__ x_head, const float (&wv)[4],
                                               float eps, const float (&cv)[4], const float (&sv)[4],
                                               int lane, uint16_t (&out)[4]) {
    float x[4];
    uint16_t x16[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        x16[i] = x_head[lane + 32 * i];
        x[i] = h2f(x16[i]);
    }
    head_norm_rope_vals<kNorm, kRope>(x, x16, wv, eps, cv, sv, out);
}

__device__ __forceinline__ void load4(const uint16_t* __restrict__ p, int lane, float (&v)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = h2f(p[lane + 32 * i]);
}

}  // namespace oxi
