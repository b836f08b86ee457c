// Prefill Q8_0 GEMM on the 5th-generation tensor cores: out[t][r] = sum_b d_x[t,b] d_w[r,b] sum_k q_x[t,b,k] q_w[r,b,k].
//
// Replaces zen::quant::gemm / gemm_batch for Q8_0 at prefill sizes (src/quant.cpp:1613-1680, :1521-1565);
// the arithmetic is the reference's int8-activation arithmetic (kernels/avx2.cpp:562-585 per token, restated
// per (row, token, block) by shaders/q8_0_gemm_i8.hlsl:249-257): exact int32 block dot products, then one
// fp32 multiply-add per block with the product of the two block scales.
//
// Shape of the kernel (one persistent CTA per SM, 10 warps):
//   warp 0      TMA producer: per 128-wide K tile, one tile of weight codes (128 rows x 128 B), one of
//               activation codes (N tokens x 128 B), both K-major with the 128-byte swizzle, and the four
//               rows of block-major activation scales the tile's blocks need, into a 4-stage ring;
//   warp 1      MMA issuer: tcgen05.mma kind::i8, M = 128 weight rows, N = tokens, K = 32 = ONE Q8_0 block per
//               instruction, because every block has its own pair of scales the int32 sums of two blocks can
//               not share an accumulator.  Accumulators alternate between two TMEM buffers of N columns;
//   warps 2..9  epilogue: tcgen05.ld the block's int32 sums (thread = weight row = TMEM lane, registers =
//               tokens), release the TMEM buffer, convert, and fused-multiply-add with d_w[r,b] (a per-thread
//               constant for the block) times d_x[t,b] (broadcast reads from the stage) into fp32 registers.
//               Warps of the same lane quadrant split the token columns.
// Weights are the M operand so that, for a fixed token, the 32 lanes of a warp hold 32 consecutive weight rows:
// the token-major output [T][rows] is written with full 128-byte lines.
//
// Roofline: the tensor work is 2*T*rows*K int8 operations.  The epilogue costs one conversion and two fp32
// operations per (row, token, block) on CUDA cores, about six times the tensor time of the block's MMA, so
// this kernel is bound by the fp32/int32 pipes, not by the tensor pipe.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "quantize_acts.cuh"
#include "zk_ptx.cuh"

namespace zk {

constexpr int kGemmM = 128;            // weight rows per tile (TMEM lanes)
constexpr int kGemmKTile = 128;        // K bytes per stage = 4 Q8_0 blocks
constexpr int kGemmBlocksPerTile = kGemmKTile / 32;
constexpr int kGemmStages = 4;
constexpr int kGemmEpiWarps = 16;       // four per TMEM lane quadrant
constexpr int kGemmSplit = kGemmEpiWarps / 4;  // the warps of a quadrant split the token columns
constexpr int kGemmThreads = (2 + kGemmEpiWarps) * 32;
constexpr int kGemmMaxN = 256;         // tokens per tile, a multiple of 32

struct GemmParams {
    CUtensorMap map_w;                 // weight codes  [rows][K] int8, box 128 B x 128 rows, SWIZZLE_128B
    CUtensorMap map_x;                 // act codes     [tokens_padded][K] int8, box 128 B x n_tile rows, SWIZZLE_128B
    CUtensorMap map_xs;                // act scales    [nb][t_ld] fp32 (block-major), box n_tile x 4
    const __half* w_scales;            // [rows][nbp]
    float* out;                        // [tokens][rows]
    uint32_t rows, tokens, nb, nbp;
    uint32_t n_tile;                   // tokens per tile: 32, 64, 128 or 256
    uint32_t m_tiles, n_tiles;
    int* error_word;
};

__host__ __device__ inline uint32_t gemm_stage_bytes(uint32_t n_tile) {
    return kGemmM * kGemmKTile + n_tile * kGemmKTile + kGemmBlocksPerTile * n_tile * 4;
}
__host__ __device__ inline size_t gemm_smem_bytes(uint32_t n_tile) {
    return 1024 /* alignment slack */ + static_cast<size_t>(kGemmStages) * gemm_stage_bytes(n_tile) + 256 /* barriers */;
}

// Packed fp32 pairs (sm_100 f32x2 arithmetic): one instruction scales or accumulates two token columns.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// Two int32 block sums -> two exact floats without the (quarter-rate) conversion unit: |v| < 2^22, so
// adding v to the bit pattern of 1.5 * 2^23 yields the float 1.5 * 2^23 + v exactly, and subtracting
// 1.5 * 2^23 is exact as well.  One integer add per value plus one packed fp32 add per pair.
__device__ __forceinline__ uint64_t ints_to_float2(uint32_t v0, uint32_t v1) {
    const uint64_t biased = pack2(__uint_as_float(v0 + 0x4B400000u), __uint_as_float(v1 + 0x4B400000u));
    return add2(biased, pack2(-12582912.0f, -12582912.0f));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// acc[c/2] += float(v[c], v[c+1]) * (sw * sx[c], sw * sx[c+1]) for 32 token columns.
// ZK_GEMM_VARIANT selects how: 0 = convert unit + packed fp32, 1 = magic-number convert + packed fp32,
// 2 = convert unit + scalar fp32, 3 = magic-number convert + scalar fp32.
#ifndef ZK_GEMM_VARIANT
#define ZK_GEMM_VARIANT 0
#endif
__device__ __forceinline__ float int_to_float(uint32_t v) {
#if ZK_GEMM_VARIANT == 1 || ZK_GEMM_VARIANT == 3
    return __uint_as_float(v + 0x4B400000u) - 12582912.0f;
#else
    return static_cast<float>(static_cast<int>(v));
#endif
}
__device__ __forceinline__ void gemm_fma32(const uint32_t (&v)[32], uint64_t sw2, const float* __restrict__ sx, uint64_t* __restrict__ acc) {
#if ZK_GEMM_VARIANT >= 2
    float sw, sw_hi;
    unpack2(sw2, sw, sw_hi);
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
        const float4 s4 = *reinterpret_cast<const float4*>(sx + c);
        float a0, a1, a2, a3;
        unpack2(acc[c / 2], a0, a1);
        unpack2(acc[c / 2 + 1], a2, a3);
        a0 = fmaf(int_to_float(v[c + 0]), sw * s4.x, a0);
        a1 = fmaf(int_to_float(v[c + 1]), sw * s4.y, a1);
        a2 = fmaf(int_to_float(v[c + 2]), sw * s4.z, a2);
        a3 = fmaf(int_to_float(v[c + 3]), sw * s4.w, a3);
        acc[c / 2] = pack2(a0, a1);
        acc[c / 2 + 1] = pack2(a2, a3);
    }
#else
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
        const ulonglong2 s4 = *reinterpret_cast<const ulonglong2*>(sx + c);  // same address in every lane: a broadcast
#if ZK_GEMM_VARIANT == 1
        const uint64_t f01 = ints_to_float2(v[c + 0], v[c + 1]);
        const uint64_t f23 = ints_to_float2(v[c + 2], v[c + 3]);
#else
        const uint64_t f01 = pack2(int_to_float(v[c + 0]), int_to_float(v[c + 1]));
        const uint64_t f23 = pack2(int_to_float(v[c + 2]), int_to_float(v[c + 3]));
#endif
        acc[c / 2] = fma2(f01, mul2(s4.x, sw2), acc[c / 2]);
        acc[c / 2 + 1] = fma2(f23, mul2(s4.y, sw2), acc[c / 2 + 1]);
    }
#endif
}

// One block's int32 sums for this warp's kNHalf token columns: TMEM -> registers 32 columns at a time (the next
// chunk is in flight while the current one is folded into the accumulators), then acc += float(sum) * (sw * sx).
// The TMEM buffer is handed back to the MMA warp as soon as the last chunk has been read.
template <int kNHalf>  // token columns per epilogue warp
__device__ __forceinline__ void gemm_epilogue_block(uint32_t taddr, float sw_scalar, const float* __restrict__ sx, uint64_t (&acc)[kNHalf / 2],
                                                    uint64_t* tmem_empty_bar, int lane) {
    const uint64_t sw = pack2(sw_scalar, sw_scalar);
    if constexpr (kNHalf <= 64) {
        uint32_t va[32], vb[32];
        tmem_ld_32x32(taddr, va);
        if (kNHalf > 32) tmem_ld_32x32(taddr + 32, vb);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar);
        gemm_fma32(va, sw, sx, acc);
        if (kNHalf > 32) gemm_fma32(vb, sw, sx + 32, acc + 16);
    } else {
        // 128 accumulators leave room for one 32-column staging buffer only
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < kNHalf; c += 32) {
            tmem_ld_32x32(taddr + c, v);
            tmem_ld_wait();
            if (c + 32 >= kNHalf) { tc_fence_before_sync(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
            gemm_fma32(v, sw, sx + c, acc + c / 2);
        }
    }
}

template <int kNTile>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_q8_0_i8_kernel(const __grid_constant__ GemmParams p) {
    constexpr int kNHalf = kNTile / kGemmSplit;     // token columns per epilogue warp
    constexpr uint32_t kBufs = 512 / kNTile > 4 ? 4 : 512 / kNTile;  // TMEM accumulator buffers
    constexpr uint32_t kStageBytes = kGemmM * kGemmKTile + kNTile * kGemmKTile + kGemmBlocksPerTile * kNTile * 4;
    constexpr uint32_t kTmemCols = kBufs * kNTile;  // 512: a power of two
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGemmStages * kStageBytes);
    uint64_t* empty = full + kGemmStages;
    uint64_t* tmem_full = empty + kGemmStages;
    uint64_t* tmem_empty = tmem_full + 4;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 4);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ktiles = (p.nb + kGemmBlocksPerTile - 1) / kGemmBlocksPerTile;
    const uint32_t total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1 + kGemmEpiWarps);
        }
        for (int b = 0; b < static_cast<int>(kBufs); ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kGemmEpiWarps);
        }
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_descriptor(&p.map_w);
        tma_prefetch_descriptor(&p.map_x);
        tma_prefetch_descriptor(&p.map_xs);
    }
    if (warp == 1) tmem_alloc(tmem_base_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const uint32_t mt = tile % p.m_tiles, nt = tile / p.m_tiles;
                for (uint32_t kt = 0; kt < ktiles; ++kt, ++it) {
                    const uint32_t stage = it % kGemmStages;
                    if (it >= kGemmStages && !mbar_wait(&empty[stage], ((it / kGemmStages) - 1) & 1)) {
                        *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); ok = false;
                    }
                    if (*abort_word) ok = false;
                    if (!ok) break;
                    uint8_t* st = smem + stage * kStageBytes;
                    mbar_arrive_expect_tx(&full[stage], kStageBytes);
                    tma_load_2d(st, &p.map_w, static_cast<int>(kt * kGemmKTile), static_cast<int>(mt * kGemmM), &full[stage]);
                    tma_load_2d(st + kGemmM * kGemmKTile, &p.map_x, static_cast<int>(kt * kGemmKTile), static_cast<int>(nt * kNTile), &full[stage]);
                    tma_load_2d(st + kGemmM * kGemmKTile + kNTile * kGemmKTile, &p.map_xs, static_cast<int>(nt * kNTile),
                                static_cast<int>(kt * kGemmBlocksPerTile), &full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(kGemmM, kNTile);
            uint32_t it = 0, blk = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (uint32_t kt = 0; kt < ktiles && ok; ++kt, ++it) {
                    const uint32_t stage = it % kGemmStages;
                    if (*abort_word || !mbar_wait(&full[stage], (it / kGemmStages) & 1)) {
                        if (!*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
                    const uint64_t a_desc = umma_desc_k_sw128(a_addr), b_desc = umma_desc_k_sw128(a_addr + kGemmM * kGemmKTile);
                    const uint32_t nblk = min(static_cast<uint32_t>(kGemmBlocksPerTile), p.nb - kt * kGemmBlocksPerTile);
                    for (uint32_t j = 0; j < nblk; ++j, ++blk) {
                        const uint32_t buf = blk % kBufs;
                        if (blk >= kBufs) {
                            if (!mbar_wait(&tmem_empty[buf], ((blk / kBufs) - 1) & 1)) {
                                *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                        }
                        // one Q8_0 block: 32 bytes of K = two 16-byte units further into the swizzle atom
                        tc_mma_i8(tmem_base + buf * kNTile, a_desc + 2 * j, b_desc + 2 * j, idesc, 0u);
                        tc_commit(&tmem_full[buf]);
                    }
                    if (ok) tc_commit(&empty[stage]);  // the stage is free once its MMAs have read it
                }
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int e = warp - 2;
        const uint32_t quad = static_cast<uint32_t>(warp) & 3;   // the TMEM lanes a warp may touch: 32 * (warp id % 4)
        const uint32_t half = static_cast<uint32_t>(e) >> 2;      // which share of the token columns this warp takes
        const uint32_t lane_addr = (quad * 32) << 16;
        uint32_t it = 0, blk = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const uint32_t mt = tile % p.m_tiles, nt = tile / p.m_tiles;
            const uint32_t r = mt * kGemmM + quad * 32 + lane;
            const bool row_ok = r < p.rows;
            uint64_t acc[kNHalf / 2];  // packed pairs of fp32 accumulators, token columns (2i, 2i+1)
#pragma unroll
            for (int c = 0; c < kNHalf / 2; ++c) acc[c] = 0ull;
            for (uint32_t kt = 0; kt < ktiles && ok; ++kt, ++it) {
                const uint32_t stage = it % kGemmStages;
                // this tile's four weight scales of row r (8-byte aligned: nbp is a multiple of 8)
                uint2 sw4 = make_uint2(0, 0);
                if (row_ok) sw4 = __ldg(reinterpret_cast<const uint2*>(p.w_scales + static_cast<size_t>(r) * p.nbp + kt * kGemmBlocksPerTile));
                if (*abort_word || !mbar_wait(&full[stage], (it / kGemmStages) & 1)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                    ok = false;
                    break;
                }
                const float* sxs = reinterpret_cast<const float*>(smem + stage * kStageBytes + kGemmM * kGemmKTile + kNTile * kGemmKTile);
                const __half2 h01 = *reinterpret_cast<const __half2*>(&sw4.x), h23 = *reinterpret_cast<const __half2*>(&sw4.y);
                const float swf[4] = {__low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23)};
                const uint32_t nblk = min(static_cast<uint32_t>(kGemmBlocksPerTile), p.nb - kt * kGemmBlocksPerTile);
#pragma unroll
                for (uint32_t j = 0; j < kGemmBlocksPerTile; ++j) {
                    if (j < nblk && ok) {
                        const uint32_t buf = blk % kBufs;
                        if (!mbar_wait(&tmem_full[buf], (blk / kBufs) & 1)) {
                            if (lane == 0) { *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); }
                            ok = false;
                        } else {
                            tc_fence_after_sync();
                            gemm_epilogue_block<kNHalf>(tmem_base + lane_addr + buf * kNTile + half * kNHalf, swf[j],
                                                        sxs + j * kNTile + half * kNHalf, acc, &tmem_empty[buf], lane);
                            ++blk;
                        }
                    }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stage]);  // done with the stage's activation scales
            }
            if (!ok) break;
            if (row_ok) {
#pragma unroll
                for (int c = 0; c < kNHalf; c += 2) {
                    const uint32_t t = nt * kNTile + half * kNHalf + c;
                    float lo, hi;
                    unpack2(acc[c / 2], lo, hi);
                    if (t < p.tokens) p.out[static_cast<size_t>(t) * p.rows + r] = lo;
                    if (t + 1 < p.tokens) p.out[static_cast<size_t>(t + 1) * p.rows + r] = hi;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Activation quantiser for the GEMM: codes [t_pad][K] int8 (rows >= tokens are zero-filled by the caller's memset)
// and scales in block-major order [nb][t_ld] fp32, so the scales of one block for a tile of tokens are contiguous.
__global__ void __launch_bounds__(256) quantize_acts_gemm_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ sc_t,
                                                                 uint32_t tokens, uint32_t nb, uint32_t t_ld) {
    const size_t wid = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<size_t>(tokens) * nb) return;
    const uint32_t t = static_cast<uint32_t>(wid / nb), b = static_cast<uint32_t>(wid % nb);
    int c1, c2;
    const float d = quantise_block_lane(x[wid * 32 + lane], c1, c2);
    q[wid * 32 + lane] = static_cast<int8_t>(c1);
    if (lane == 0) sc_t[static_cast<size_t>(b) * t_ld + t] = d;
}

}  // namespace zk
