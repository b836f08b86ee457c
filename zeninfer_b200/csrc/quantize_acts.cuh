// Activation quantiser: fp32 -> int8 codes + one fp32 scale per 32 elements.
//
// Replaces the reference's quantise_acts_q8_0 (kernels/avx2.cpp:502-524, inlined
// again at src/quant.cpp:1094-1113; the D3D12 twin is shaders/quantize_acts.hlsl).
// Codes and scales are bit-identical to it:
//     d   = amax / 127          (IEEE division, fp32)
//     inv = 1 / d               (IEEE division; 0 when d == 0)
//     q   = lround(clamp(x * inv, -127, 127))     round half AWAY from zero
// so every operation below is an explicitly rounded intrinsic: no fast-math
// reciprocal, no fused multiply-add, no round-half-even conversion.
//
// A second, finer digit is available for the formats the reference evaluates
// with fp32 activations (Q4_0, Q6_K, and Q8_0 in its default mode): the residual
// x - d*q is quantised again with scale d/256, so x ~= (d/256) * (256*q + q2)
// with an error below d/512.  That keeps integer dot products within ~1e-5 of
// the fp32-activation result.
#pragma once
#include "zk_ptx.cuh"

namespace zk {

// lround() for |v| < 2^22: add half a unit with the sign of v, rounding toward zero, then
// truncate.  Rounding the sum toward zero can never carry it across an integer (integers in
// this range are representable), so floor(|v| + 0.5) is exact: 0.49999997 -> 0, 2.5 -> 3, -2.5 -> -3.
__device__ __forceinline__ int round_half_away(float v) {
    return __float2int_rz(__fadd_rz(v, copysignf(0.5f, v)));
}

__device__ __forceinline__ float clamp127(float v) { return v > 127.0f ? 127.0f : (v < -127.0f ? -127.0f : v); }

// One warp quantises one 32-element block, one element per lane.  All 32 lanes
// must call.  Returns the block scale d; q1 is the Q8 code, q2 the fine digit.
__device__ __forceinline__ float quantise_block_lane(float x, int& q1, int& q2) {
    float amax = fabsf(x);
    amax = amax > 0.0f ? amax : 0.0f;  // a NaN element never raises amax (same as the reference's compare)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, amax, o);
        amax = other > amax ? other : amax;
    }
    const float d = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    const float inv = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    q1 = round_half_away(clamp127(__fmul_rn(x, inv)));
    const float r = __fmaf_rn(-static_cast<float>(q1), d, x);  // residual, one rounding
    q2 = round_half_away(clamp127(__fmul_rn(r, __fmul_rn(inv, 256.0f))));
    return d;
}

// Four lanes quantise one 32-element block, eight consecutive elements per lane (lanes 4k..4k+3
// of a warp form one group; all 32 lanes must call).  Same arithmetic, bit for bit, as
// quantise_block_lane; only the reduction tree of the (order-independent) maximum differs.
// c1/c2 receive the eight codes packed little-endian, element 0 in the low byte.
__device__ __forceinline__ float quantise_block_quad(const float (&v)[8], uint2& c1, uint2& c2) {
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float a = fabsf(v[k]);
        amax = a > amax ? a : amax;
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, amax, o);
        amax = other > amax ? other : amax;
    }
    const float d = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    const float inv = d > 0.0f ? __frcp_rn(d) : 0.0f;   // the correctly rounded reciprocal is the IEEE quotient 1 / d
    const float inv256 = __fmul_rn(inv, 256.0f);
    uint32_t w1[2] = {0, 0}, w2[2] = {0, 0};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int q1 = round_half_away(clamp127(__fmul_rn(v[k], inv)));
        const float r = __fmaf_rn(-static_cast<float>(q1), d, v[k]);
        const int q2 = round_half_away(clamp127(__fmul_rn(r, inv256)));
        w1[k >> 2] |= (static_cast<uint32_t>(q1) & 0xffu) << (8 * (k & 3));
        w2[k >> 2] |= (static_cast<uint32_t>(q2) & 0xffu) << (8 * (k & 3));
    }
    c1 = make_uint2(w1[0], w1[1]);
    c2 = make_uint2(w2[0], w2[1]);
    return d;
}

// Standalone kernel: x [tokens][K] fp32 -> q [tokens][K] int8, sc [tokens][K/32] fp32,
// optionally q2 [tokens][K] int8 (the fine digit).  One warp per block.
__global__ void __launch_bounds__(256) quantize_acts_kernel(const float* __restrict__ x, int8_t* __restrict__ q,
                                                            float* __restrict__ sc, int8_t* __restrict__ q2,
                                                            size_t total_blocks) {
    const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= total_blocks) return;
    int c1, c2;
    const float d = quantise_block_lane(x[warp * 32 + lane], c1, c2);
    q[warp * 32 + lane] = static_cast<int8_t>(c1);
    if (q2) q2[warp * 32 + lane] = static_cast<int8_t>(c2);
    if (lane == 0) sc[warp] = d;
}

}  // namespace zk
