// Q4_K / Q5_K decode products straight from the raw GGUF super-blocks (no repack on upload).
//
// The reference computes these with fp32 activations only (gemv_q4k_q5k_avx2, kernels/avx2.cpp:329-378; its GPU entry
// is zen::d3d12::gemm_kquant, include/zen/d3d12_backend.h:75): per sub-block of 32, ds = d * sc and ms = dmin * m, a
// weight is (ds * q) - ms with both roundings, and the products are accumulated with fused multiply-adds.  This kernel
// does the same arithmetic per weight; only the order in which a row's products are summed differs (a lane owns one
// eight-element chunk of every super-block, then the warp adds its lanes).
//
// A warp takes a row.  Lane l of a super-block: sub-block l / 4, chunk l % 4 -- eight consecutive elements, i.e. one
// aligned 8-byte word of the nibble plane (and of the fifth-bit plane for Q5_K) and two float4 words of every
// activation row.  Super-blocks are 144 / 176 bytes, multiples of 16, so every word is naturally aligned.
// First version: correct and coalesced, not tuned (no shared-memory staging, activations through L1/L2).
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

#include "zk_ptx.cuh"

namespace zk {

constexpr int kK45Warps = 8, kK45MaxTokens = 8;

template <bool kQ5>
__global__ void __launch_bounds__(kK45Warps * 32) gemv_k45_kernel(const uint8_t* __restrict__ weights, const float* __restrict__ x, float* __restrict__ y,
                                                                    uint32_t rows, uint32_t nb, uint32_t tokens) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr uint32_t kBytes = kQ5 ? 176u : 144u, kNibbles = kQ5 ? 48u : 16u;
    const uint32_t row = blockIdx.x * kK45Warps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint32_t group = lane >> 2, chunk = lane & 3, shift = (group & 1u) * 4u;
    const uint8_t* prow = weights + static_cast<size_t>(row) * nb * kBytes;
    const size_t K = static_cast<size_t>(nb) * 256;
    float acc[kK45MaxTokens];
#pragma unroll
    for (int t = 0; t < kK45MaxTokens; ++t) acc[t] = 0.0f;
    for (uint32_t b = 0; b < nb; ++b) {
        const uint8_t* p = prow + static_cast<size_t>(b) * kBytes;
        const uint32_t hdr = __ldg(reinterpret_cast<const uint32_t*>(p));
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr & 0xffffu)));
        const float dm = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr >> 16)));
        // the 6-bit scale and minimum of sub-block `group` from the 12 packed bytes (src/quant.cpp:133-141)
        const uint8_t* s8 = p + 4;
        uint32_t sc, mn;
        if (group < 4) {
            sc = __ldg(s8 + group) & 63u;
            mn = __ldg(s8 + group + 4) & 63u;
        } else {
            const uint32_t hi = __ldg(s8 + group + 4);
            sc = (hi & 15u) | ((static_cast<uint32_t>(__ldg(s8 + group - 4)) >> 6) << 4);
            mn = (hi >> 4) | ((static_cast<uint32_t>(__ldg(s8 + group)) >> 6) << 4);
        }
        const float ds = __fmul_rn(d, static_cast<float>(sc)), ms = __fmul_rn(dm, static_cast<float>(mn));
        const uint2 qw = __ldg(reinterpret_cast<const uint2*>(p + kNibbles + (group >> 1) * 32u + chunk * 8u));
        uint2 hw = make_uint2(0u, 0u);
        if (kQ5) hw = __ldg(reinterpret_cast<const uint2*>(p + 16u + chunk * 8u));
        float w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t byte = ((j < 4 ? qw.x : qw.y) >> (8 * (j & 3))) & 0xffu;
            uint32_t q = (byte >> shift) & 15u;
            if (kQ5) q |= ((((j < 4 ? hw.x : hw.y) >> (8 * (j & 3))) >> group) & 1u) << 4;
            w[j] = __fsub_rn(__fmul_rn(ds, static_cast<float>(q)), ms);   // both roundings, as the reference's mul then sub
        }
        const size_t col = static_cast<size_t>(b) * 256 + group * 32u + chunk * 8u;
#pragma unroll
        for (int t = 0; t < kK45MaxTokens; ++t) {
            if (t < static_cast<int>(tokens)) {
                const float4* xp = reinterpret_cast<const float4*>(x + static_cast<size_t>(t) * K + col);
                const float4 a = __ldg(xp), c = __ldg(xp + 1);
                float s = acc[t];
                s = fmaf(w[0], a.x, s); s = fmaf(w[1], a.y, s); s = fmaf(w[2], a.z, s); s = fmaf(w[3], a.w, s);
                s = fmaf(w[4], c.x, s); s = fmaf(w[5], c.y, s); s = fmaf(w[6], c.z, s); s = fmaf(w[7], c.w, s);
                acc[t] = s;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kK45MaxTokens; ++t) {
        if (t < static_cast<int>(tokens)) {
            float s = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) y[static_cast<size_t>(t) * rows + row] = s;
        }
    }
}

}  // namespace zk
