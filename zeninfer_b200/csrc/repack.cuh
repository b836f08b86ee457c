// Upload-time re-layout of raw GGUF blocks into aligned planes.
//
// A GGUF tensor arrives as rows of interleaved blocks (Q8_0: 34 B, Q4_0: 18 B,
// Q6_K: 210 B).  None of those sizes is a multiple of 16, so neither 128-bit
// loads nor TMA copies can address the codes directly.  Like the reference's
// GPU backends (src/backends/hip/hip_backend.hip:321-333 splits Q8_0 into
// "quants | scales"), the device copy is split into planes, each row of each
// plane starting on a 16-byte boundary.  Byte counts are unchanged (padding
// aside), and the split is a pure byte move: no value is re-quantised.
//
//   Q8_0: codes  [rows][K]      int8      scales [rows][nbp] f16   (nbp = blocks rounded up to 8)
//   Q4_0: nibs   [rows][K/2]    uint8     scales [rows][nbp] f16
//   Q6_K: ql     [rows][K/2]    uint8     qh [rows][K/4] uint8
//         sc     [rows][K/16]   int8      d  [rows][sbp] f16       (sbp = super-blocks rounded up to 8)
//   Q4_K: qs     [rows][K/2]    uint8     scm [rows][K/16] uint8   dd [rows][sbp] (f16 d, f16 dmin)
//   Q5_K: qs     [rows][K/2]    uint8     qh  [rows][K/8]  uint8   scm, dd as Q4_K
//         scm holds, per super-block, the eight 6-bit sub-block scales and the eight 6-bit minimums unpacked to one
//         byte each (16 bytes instead of the 12 packed ones, src/quant.cpp:133-141): the only plane that is not a pure
//         byte move, and the values are unchanged.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace zk {

__device__ __forceinline__ uint16_t ld_u16_unaligned(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }

// One thread per 32-element block.  raw: [rows][nb*34].
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ codes, uint16_t* __restrict__ scales,
                                   size_t rows, uint32_t nb, uint32_t nbp) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * nb) return;
    const size_t r = i / nb;
    const uint32_t b = static_cast<uint32_t>(i % nb);
    const uint8_t* p = raw + i * 34;  // 2-byte aligned
    scales[r * nbp + b] = *reinterpret_cast<const uint16_t*>(p);
    const uint16_t* src = reinterpret_cast<const uint16_t*>(p + 2);
    uint16_t* dst = reinterpret_cast<uint16_t*>(codes + (r * nb + b) * 32);
#pragma unroll
    for (int k = 0; k < 16; ++k) dst[k] = src[k];
}

// One thread per 32-element block.  raw: [rows][nb*18].
__global__ void repack_q4_0_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ nibs, uint16_t* __restrict__ scales,
                                   size_t rows, uint32_t nb, uint32_t nbp) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * nb) return;
    const size_t r = i / nb;
    const uint32_t b = static_cast<uint32_t>(i % nb);
    const uint8_t* p = raw + i * 18;
    scales[r * nbp + b] = *reinterpret_cast<const uint16_t*>(p);
    const uint16_t* src = reinterpret_cast<const uint16_t*>(p + 2);
    uint16_t* dst = reinterpret_cast<uint16_t*>(nibs + (r * nb + b) * 16);
#pragma unroll
    for (int k = 0; k < 8; ++k) dst[k] = src[k];
}

// One thread per 256-element super-block.  raw: [rows][nsb*210].
__global__ void repack_q6_k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ ql, uint8_t* __restrict__ qh,
                                   int8_t* __restrict__ sc, uint16_t* __restrict__ d, size_t rows, uint32_t nsb, uint32_t sbp) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * nsb) return;
    const size_t r = i / nsb;
    const uint32_t b = static_cast<uint32_t>(i % nsb);
    const uint16_t* p = reinterpret_cast<const uint16_t*>(raw + i * 210);  // 210 is even
    uint16_t* o_ql = reinterpret_cast<uint16_t*>(ql + (r * nsb + b) * 128);
    uint16_t* o_qh = reinterpret_cast<uint16_t*>(qh + (r * nsb + b) * 64);
    uint16_t* o_sc = reinterpret_cast<uint16_t*>(sc + (r * nsb + b) * 16);
    for (int k = 0; k < 64; ++k) o_ql[k] = p[k];
    for (int k = 0; k < 32; ++k) o_qh[k] = p[64 + k];
    for (int k = 0; k < 8; ++k) o_sc[k] = p[96 + k];
    d[r * sbp + b] = p[104];
}

// One thread per 256-element super-block.  raw: [rows][nsb*144] (Q4_K: d, dmin, scales[12], qs[128]) or
// [rows][nsb*176] (Q5_K: d, dmin, scales[12], qh[32], qs[128]).  Both sizes are multiples of 16.
template <bool kQ5>
__global__ void repack_k45_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ qs, uint8_t* __restrict__ qh, uint8_t* __restrict__ scm,
                                  uint32_t* __restrict__ dd, size_t rows, uint32_t nsb, uint32_t sbp) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * nsb) return;
    const size_t r = i / nsb;
    const uint32_t b = static_cast<uint32_t>(i % nsb);
    const uint8_t* p = raw + i * (kQ5 ? 176 : 144);
    dd[r * sbp + b] = *reinterpret_cast<const uint32_t*>(p);
    const uint8_t* s8 = p + 4;
    uint8_t out[16];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        if (g < 4) {
            out[g] = s8[g] & 63u;
            out[8 + g] = s8[g + 4] & 63u;
        } else {
            out[g] = static_cast<uint8_t>((s8[g + 4] & 15u) | ((s8[g - 4] >> 6) << 4));
            out[8 + g] = static_cast<uint8_t>((s8[g + 4] >> 4) | ((s8[g] >> 6) << 4));
        }
    }
    uint4 packed;
    packed.x = out[0] | (out[1] << 8) | (out[2] << 16) | (static_cast<uint32_t>(out[3]) << 24);
    packed.y = out[4] | (out[5] << 8) | (out[6] << 16) | (static_cast<uint32_t>(out[7]) << 24);
    packed.z = out[8] | (out[9] << 8) | (out[10] << 16) | (static_cast<uint32_t>(out[11]) << 24);
    packed.w = out[12] | (out[13] << 8) | (out[14] << 16) | (static_cast<uint32_t>(out[15]) << 24);
    *reinterpret_cast<uint4*>(scm + (r * nsb + b) * 16) = packed;
    const uint4* src = reinterpret_cast<const uint4*>(p + 16);
    if (kQ5) {
        uint4* o = reinterpret_cast<uint4*>(qh + (r * nsb + b) * 32);
        o[0] = src[0]; o[1] = src[1];
        src += 2;
    }
    uint4* o = reinterpret_cast<uint4*>(qs + (r * nsb + b) * 128);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = src[k];
}

// Q6_K with the codes unpacked: one thread per 16-weight group.  codes [rows][K] int8 = q - 32 in element order (element
// half*128 + g*32 + l of a super-block is ql byte half*64 + (g%2)*32 + l, low nibble for g < 2, plus bits 2g.. of qh byte
// half*32 + l, src/quant.cpp:500-517); sc and d as repack_q6_k_kernel leaves them.
__global__ void unpack_q6_k_codes_kernel(const uint8_t* __restrict__ raw, int8_t* __restrict__ codes, int8_t* __restrict__ sc, uint16_t* __restrict__ d,
                                         size_t rows, uint32_t nsb, uint32_t sbp) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // group index over the tensor
    if (i >= rows * nsb * 16) return;
    const size_t sb = i / 16;
    const uint32_t g16 = static_cast<uint32_t>(i % 16);      // 16-weight group within the super-block: elements g16*16 ..
    const size_t r = sb / nsb;
    const uint32_t b = static_cast<uint32_t>(sb % nsb);
    const uint8_t* p = raw + sb * 210;
    const uint32_t e0 = g16 * 16, half = e0 >> 7, g = (e0 >> 5) & 3, l0 = e0 & 31;
    int8_t out[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const uint32_t l = l0 + k;
        const uint32_t lo = (p[half * 64 + (g & 1) * 32 + l] >> (g >= 2 ? 4 : 0)) & 15u;
        const uint32_t hi = (p[128 + half * 32 + l] >> (2 * g)) & 3u;
        out[k] = static_cast<int8_t>(static_cast<int>(lo | (hi << 4)) - 32);
    }
    int8_t* dst = codes + (r * nsb + b) * 256 + e0;
#pragma unroll
    for (int k = 0; k < 16; ++k) dst[k] = out[k];
    sc[(r * nsb + b) * 16 + g16] = static_cast<int8_t>(p[192 + g16]);
    if (g16 == 0) d[r * sbp + b] = static_cast<uint16_t>(p[208] | (p[209] << 8));
}

// Q4_0 nibble plane -> int8 codes n - 8 in element order, [rows][K]: with the tensor's own f16 block scales this is a
// Q8_0 tensor, which is how the tensor-core GEMM multiplies Q4_0 (a pass per call into scratch memory; the resident copy
// stays 4-bit).  One thread per 32-weight block; low nibbles are elements 0..15, high nibbles 16..31 (src/quant.cpp:391-397).
__global__ void unpack_q4_0_codes_kernel(const uint8_t* __restrict__ nibs, int8_t* __restrict__ codes, size_t blocks) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= blocks) return;
    const uint4 w = reinterpret_cast<const uint4*>(nibs)[i];
    // n - 8 per byte without borrows between bytes: set the top bit, subtract, flip it back
    auto sub8 = [](uint32_t n) { return ((n | 0x80808080u) - 0x08080808u) ^ 0x80808080u; };
    const uint32_t m = 0x0F0F0F0Fu;
    uint4* out = reinterpret_cast<uint4*>(codes + i * 32);
    out[0] = make_uint4(sub8(w.x & m), sub8(w.y & m), sub8(w.z & m), sub8(w.w & m));
    out[1] = make_uint4(sub8((w.x >> 4) & m), sub8((w.y >> 4) & m), sub8((w.z >> 4) & m), sub8((w.w >> 4) & m));
}

// Q4_K / Q5_K planes -> int8 codes (0..15, 0..31) in element order [rows][K] plus, per 32-weight sub-block, the fp32
// factors the reference forms (kernels/avx2.cpp:329-378): scale = d * sc and offset = dmin * m, [rows][K / 32] each, so
// that w = scale * q - offset.  One thread per 32 nibble bytes = sub-blocks 2 j (low nibbles) and 2 j + 1 (high nibbles)
// of a super-block; the fifth bits of both are bits 2 j and 2 j + 1 of the same 32 qh bytes (src/quant.cpp:133-141).
template <bool kQ5>
__global__ void unpack_k45_codes_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ qh, const uint8_t* __restrict__ scm,
                                        const uint32_t* __restrict__ dd, int8_t* __restrict__ codes, float* __restrict__ scales,
                                        float* __restrict__ offsets, size_t rows, uint32_t nsb, uint32_t sbp) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * nsb * 4) return;
    const size_t sbi = i / 4;                       // r * nsb + b
    const uint32_t j = static_cast<uint32_t>(i % 4);
    const size_t r = sbi / nsb;
    const uint32_t b = static_cast<uint32_t>(sbi % nsb);
    const uint4* src = reinterpret_cast<const uint4*>(qs + sbi * 128 + j * 32);
    const uint4 w[2] = {src[0], src[1]};
    uint4 h[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (kQ5) {
        const uint4* q5 = reinterpret_cast<const uint4*>(qh + sbi * 32);
        h[0] = q5[0]; h[1] = q5[1];
    }
    const uint32_t m = 0x0F0F0F0Fu, one = 0x01010101u, s_lo = 2 * j, s_hi = 2 * j + 1;
    auto lo = [&](uint32_t v, uint32_t f) { return (v & m) | (((f >> s_lo) & one) << 4); };
    auto hi = [&](uint32_t v, uint32_t f) { return ((v >> 4) & m) | (((f >> s_hi) & one) << 4); };
    uint4* out = reinterpret_cast<uint4*>(codes + sbi * 256 + j * 64);
    out[0] = make_uint4(lo(w[0].x, h[0].x), lo(w[0].y, h[0].y), lo(w[0].z, h[0].z), lo(w[0].w, h[0].w));
    out[1] = make_uint4(lo(w[1].x, h[1].x), lo(w[1].y, h[1].y), lo(w[1].z, h[1].z), lo(w[1].w, h[1].w));
    out[2] = make_uint4(hi(w[0].x, h[0].x), hi(w[0].y, h[0].y), hi(w[0].z, h[0].z), hi(w[0].w, h[0].w));
    out[3] = make_uint4(hi(w[1].x, h[1].x), hi(w[1].y, h[1].y), hi(w[1].z, h[1].z), hi(w[1].w, h[1].w));
    const uint8_t* sm = scm + sbi * 16;
    const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(dd + r * sbp + b));
    const size_t o = (r * nsb + b) * 8 + 2 * j;     // block index of sub-block 2 j within the row-major [rows][K / 32] planes
    scales[o] = dm.x * static_cast<float>(sm[2 * j]);
    scales[o + 1] = dm.x * static_cast<float>(sm[2 * j + 1]);
    offsets[o] = dm.y * static_cast<float>(sm[8 + 2 * j]);
    offsets[o + 1] = dm.y * static_cast<float>(sm[8 + 2 * j + 1]);
}

}  // namespace zk
