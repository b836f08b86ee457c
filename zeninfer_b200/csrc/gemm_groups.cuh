// Many-row products that keep the tensor cores busy: weights and activations as two int8 digits under ONE scale per
// 256-weight group, so that a whole group accumulates in TMEM and the CUDA cores touch a sum once per 256 weights.
//
// The per-block kernel (gemm_q8_0_i8.cuh) follows the reference's blocks literally: every 32-weight block has its own
// pair of scales, so every block's int32 sums have to be read back, converted and scaled -- one conversion and two fp32
// operations per (row, token, block), about six times the tensor time of the block's MMA.  That kernel is bound by its
// epilogue at a tenth of the tensor rate.  Here the scales are made common first:
//
//   weights      w[r, k] = d_w[r, b] * q[r, k]  (the dequantised value, exact in fp32; any format)
//                        ~= u_w[r, g] * (256 * wh + wl),   u_w = max|w| of the group / 32639,  wh in -127..127, wl in -128..127
//   activations  x[t, k] (fp32, or d_x[t, b] * q_x[t, k] after the reference's int8 quantisation, kernels/avx2.cpp:502-524)
//                        ~= u_x[t, g] * (256 * xh + xl)
//
// Both are 16-bit fixed point relative to the group's largest magnitude: an error of at most 1/65278 of that magnitude per
// value, the same resolution the two-digit activations of the per-block kernel have.  Then
//
//   sum_k w x ~= u_w u_x * (65536 * sum wh xh + 256 * (sum wh xl + sum wl xh) + sum wl xl)
//
// and the last term (at most 2^-16 of the first per product) is dropped: three MMAs per 32 columns of K, two TMEM
// accumulators A = sum wh xh and B = sum wh xl + sum wl xh over the group's eight K steps, and the epilogue forms
// (256 * u_w * u_x) * (256 * A + B) once per group.  Results agree with the reference's sums to ~5e-5 of the largest result
// (bar 1e-3).
//
// Replaces zen::quant::gemm / gemm_batch at prefill sizes (src/quant.cpp:1613-1680, :1521-1565) for both activation
// modes, and the batched products of the other formats (gemm_q6k_kblk_avx2, gemm_q4k_kblk_avx2, gemm_q5k_kblk_avx2,
// kernels/avx2.cpp:1605-1620, :1762-1770; Q4_0's generic route).  The two-digit weight planes are built once per resident
// tensor (group_digits_q8_0_kernel, group_digits_kq_kernel) and kept beside the decode planes: 2 bytes per weight of extra
// device memory.
//
// Shape: one persistent CTA per SM, 18 warps.  Warp 0: TMA producer, per 128-wide K tile four tiles (wh, wl, xh, xl; 128
// rows x 128 B, K-major, 128-byte swizzle) into a 3-stage ring.  Warp 1: MMA issuer, tcgen05.mma kind::i8, M = 128 weight
// rows, N = 128 tokens, K = 32; accumulator sets alternate between the two halves of TMEM.  Warps 2..17: epilogue, thread =
// weight row = TMEM lane, 32 token columns per warp.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "gemm_q8_0_i8.cuh"

namespace zk {

constexpr int kGgGroup = 256;                       // weights per common scale
constexpr int kGgKTilesPerGroup = kGgGroup / kGemmKTile;
constexpr int kGgStages = 3;
constexpr int kGgNTile = 128;
constexpr uint32_t kGgTileBytes = kGemmM * kGemmKTile;          // 16 KB: 128 rows x 128 B
constexpr uint32_t kGgStageBytes = 4 * kGgTileBytes;            // wh | wl | xh | xl
constexpr int kGgEpiWarps = 16;
constexpr int kGgThreads = (2 + kGgEpiWarps) * 32;
constexpr float kGgFullScale = 32639.0f;                        // 256 * 127 + 127

struct GroupGemmParams {
    CUtensorMap map_wh[kGemmMaxTensors], map_wl[kGemmMaxTensors];   // [rows][K] int8, box 128 B x 128 rows, SWIZZLE_128B
    CUtensorMap map_xh, map_xl;                                     // [tokens][K] int8, same box
    const float* w_unit[kGemmMaxTensors];   // [rows][groups]
    const float* x_unit;                    // [groups][t_ld]
    float* out[kGemmMaxTensors];            // [tokens][rows]
    uint32_t rows[kGemmMaxTensors];
    uint32_t m_start[kGemmMaxTensors];      // first row tile of each tensor in the launch's numbering (0xffffffff: unused)
    uint32_t tensors, tokens, groups, t_ld;
    uint32_t m_tiles, n_tiles;
    uint32_t stream_k;                      // 1: CTAs share the (tile, group) units evenly; a tile is split between at most two CTAs
    int* error_word;
};

__host__ __device__ inline size_t gemm_groups_smem_bytes() { return 1024 + static_cast<size_t>(kGgStages) * kGgStageBytes + 256; }

__device__ __forceinline__ void gg_locate(const GroupGemmParams& p, uint32_t mt_all, uint32_t& ti, uint32_t& mt) {
    ti = (mt_all >= p.m_start[1] ? 1u : 0u) + (mt_all >= p.m_start[2] ? 1u : 0u);
    mt = mt_all - p.m_start[ti];
}

// The work of one CTA: (tile, group) units, tile-major, in gridDim.x equal contiguous ranges (see GemmWork).
struct GroupWork {
    uint32_t u, u_end, groups, stride;
    __device__ explicit GroupWork(const GroupGemmParams& p) : groups(p.groups) {
        const uint32_t tiles = p.m_tiles * p.n_tiles;
        if (p.stream_k) {
            const uint64_t total = static_cast<uint64_t>(tiles) * groups;
            u = static_cast<uint32_t>(total * blockIdx.x / gridDim.x);
            u_end = static_cast<uint32_t>(total * (blockIdx.x + 1) / gridDim.x);
            stride = 0;
        } else {
            u = blockIdx.x; u_end = tiles; stride = gridDim.x;
        }
    }
    __device__ bool next(uint32_t& tile, uint32_t& g0, uint32_t& g1) {
        if (u >= u_end) return false;
        if (stride) { tile = u; g0 = 0; g1 = groups; u += stride; return true; }
        tile = u / groups; g0 = u % groups;
        g1 = min(groups, g0 + (u_end - u));
        u += g1 - g0;
        return true;
    }
};

// Clears the output tiles two CTAs of a stream-K launch share (launched right before it, same grid).
__global__ void gg_zero_split_tiles_kernel(const __grid_constant__ GroupGemmParams p) {
    if (blockIdx.x == 0) return;
    const uint64_t total = static_cast<uint64_t>(p.m_tiles) * p.n_tiles * p.groups;
    const uint32_t cut = static_cast<uint32_t>(total * blockIdx.x / gridDim.x);
    if (cut % p.groups == 0) return;
    const uint32_t tile = cut / p.groups, nt = tile / p.m_tiles;
    uint32_t ti, mt;
    gg_locate(p, tile % p.m_tiles, ti, mt);
    float* out = p.out[ti];
    const uint32_t rows = p.rows[ti];
    for (uint32_t i = threadIdx.x; i < kGgNTile * kGemmM; i += blockDim.x) {
        const uint32_t t = nt * kGgNTile + i / kGemmM, r = mt * kGemmM + i % kGemmM;
        if (t < p.tokens && r < rows) out[static_cast<size_t>(t) * rows + r] = 0.0f;
    }
}

// acc[c / 2] += (uw256 * ux[c]) * float(256 * a[c] + b[c]) for sixteen token columns; ux: their activation units.  The
// two sums are combined as integers (|256 A + B| <= 256 * 256 * 127^2 + 512 * 127 * 128 < 2^31), so a column costs one
// conversion, the scarce instruction here, instead of two.
__device__ __forceinline__ void gg_fold16(const uint32_t (&a)[16], const uint32_t (&b)[16], float uw256, const float* __restrict__ ux, uint64_t* __restrict__ acc) {
    const uint64_t uw2 = pack2(uw256, uw256);
    auto both = [&](int c) { return static_cast<float>(static_cast<int>(a[c]) * 256 + static_cast<int>(b[c])); };
#pragma unroll
    for (int c = 0; c < 16; c += 4) {
        const float4 u4 = __ldg(reinterpret_cast<const float4*>(ux + c));
        acc[c / 2] = fma2(pack2(both(c), both(c + 1)), mul2(pack2(u4.x, u4.y), uw2), acc[c / 2]);
        acc[c / 2 + 1] = fma2(pack2(both(c + 2), both(c + 3)), mul2(pack2(u4.z, u4.w), uw2), acc[c / 2 + 1]);
    }
}

__global__ void __launch_bounds__(kGgThreads, 1) gemm_groups_kernel(const __grid_constant__ GroupGemmParams p) {
    constexpr uint32_t kTmemCols = 512;             // two accumulator sets of (A, B) x 128 columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGgStages * kGgStageBytes);
    uint64_t* empty = full + kGgStages;
    uint64_t* tmem_full = empty + kGgStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kGgStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);      // the MMA issuer's commit: nobody else reads a stage
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kGgEpiWarps);
        }
        *abort_word = 0;
        mbar_fence_init();
        for (uint32_t i = 0; i < p.tensors; ++i) { tma_prefetch_descriptor(&p.map_wh[i]); tma_prefetch_descriptor(&p.map_wl[i]); }
        tma_prefetch_descriptor(&p.map_xh);
        tma_prefetch_descriptor(&p.map_xl);
    }
    if (warp == 1) tmem_alloc(tmem_base_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0, tile, g0, g1;
            bool ok = true;
            GroupWork work(p);
            while (ok && work.next(tile, g0, g1)) {
                const uint32_t nt = tile / p.m_tiles;
                uint32_t ti, mt;
                gg_locate(p, tile % p.m_tiles, ti, mt);
                for (uint32_t kt = g0 * kGgKTilesPerGroup; kt < g1 * kGgKTilesPerGroup; ++kt, ++it) {
                    const uint32_t stage = it % kGgStages;
                    if (it >= kGgStages && !mbar_wait(&empty[stage], ((it / kGgStages) - 1) & 1)) {
                        *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); ok = false;
                    }
                    if (*abort_word) ok = false;
                    if (!ok) break;
                    uint8_t* st = smem + stage * kGgStageBytes;
                    const int kx = static_cast<int>(kt * kGemmKTile);
                    mbar_arrive_expect_tx(&full[stage], kGgStageBytes);
                    tma_load_2d(st, &p.map_wh[ti], kx, static_cast<int>(mt * kGemmM), &full[stage]);
                    tma_load_2d(st + kGgTileBytes, &p.map_wl[ti], kx, static_cast<int>(mt * kGemmM), &full[stage]);
                    tma_load_2d(st + 2 * kGgTileBytes, &p.map_xh, kx, static_cast<int>(nt * kGgNTile), &full[stage]);
                    tma_load_2d(st + 3 * kGgTileBytes, &p.map_xl, kx, static_cast<int>(nt * kGgNTile), &full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(kGemmM, kGgNTile);
            uint32_t it = 0, gcount = 0, tile, g0, g1;
            bool ok = true;
            GroupWork work(p);
            while (ok && work.next(tile, g0, g1)) {
                for (uint32_t g = g0; g < g1 && ok; ++g, ++gcount) {
                    const uint32_t set = gcount & 1;
                    if (gcount >= 2) {
                        if (!mbar_wait(&tmem_empty[set], ((gcount >> 1) - 1) & 1)) {
                            *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                    }
                    const uint32_t acc_a = tmem_base + set * 256, acc_b = acc_a + 128;
                    for (uint32_t h = 0; h < static_cast<uint32_t>(kGgKTilesPerGroup) && ok; ++h, ++it) {
                        const uint32_t stage = it % kGgStages;
                        if (*abort_word || !mbar_wait(&full[stage], (it / kGgStages) & 1)) {
                            if (!*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t base = smem_u32(smem + stage * kGgStageBytes);
                        const uint64_t wh = umma_desc_k_sw128(base), wl = umma_desc_k_sw128(base + kGgTileBytes);
                        const uint64_t xh = umma_desc_k_sw128(base + 2 * kGgTileBytes), xl = umma_desc_k_sw128(base + 3 * kGgTileBytes);
#pragma unroll
                        for (uint32_t j = 0; j < static_cast<uint32_t>(kGemmBlocksPerTile); ++j) {
                            // 32 bytes of K = two 16-byte units further into the swizzle atom
                            const uint32_t first = (h == 0 && j == 0) ? 0u : 1u;
                            tc_mma_i8(acc_a, wh + 2 * j, xh + 2 * j, idesc, first);
                            tc_mma_i8(acc_b, wh + 2 * j, xl + 2 * j, idesc, first);
                            tc_mma_i8(acc_b, wl + 2 * j, xh + 2 * j, idesc, 1u);
                        }
                        tc_commit(&empty[stage]);   // the stage is free once its MMAs have read it
                    }
                    if (ok) tc_commit(&tmem_full[set]);
                }
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int e = warp - 2;
        const uint32_t quad = static_cast<uint32_t>(warp) & 3;   // the TMEM lanes a warp may touch: 32 * (warp id % 4)
        const uint32_t part = static_cast<uint32_t>(e) >> 2;      // which 32 token columns
        const uint32_t lane_addr = tmem_base + ((quad * 32) << 16) + part * 32;
        uint32_t gcount = 0, tile, g0, g1;
        bool ok = true;
        GroupWork work(p);
        while (ok && work.next(tile, g0, g1)) {
            const uint32_t nt = tile / p.m_tiles;
            uint32_t ti, mt;
            gg_locate(p, tile % p.m_tiles, ti, mt);
            const uint32_t r = mt * kGemmM + quad * 32 + lane, rows = p.rows[ti];
            const bool row_ok = r < rows;
            uint64_t acc[16];   // packed pairs of fp32 accumulators, token columns (2 i, 2 i + 1)
#pragma unroll
            for (int c = 0; c < 16; ++c) acc[c] = 0ull;
            const float* uw_row = p.w_unit[ti] + static_cast<size_t>(row_ok ? r : 0) * p.groups;
            const uint32_t col0 = nt * kGgNTile + part * 32;    // below t_ld: the unit plane is padded to whole tiles
            float uw_next = __ldg(uw_row + g0);
            for (uint32_t g = g0; g < g1 && ok; ++g, ++gcount) {
                const uint32_t set = gcount & 1;
                const float uw256 = uw_next * 256.0f;
                if (g + 1 < g1) uw_next = __ldg(uw_row + g + 1);
                if (*abort_word || !mbar_wait(&tmem_full[set], (gcount >> 1) & 1)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const float* ux = p.x_unit + static_cast<size_t>(g) * p.t_ld + col0;
                uint32_t va[16], vb[16];
                tmem_ld_32x16(lane_addr + set * 256, va);
                tmem_ld_32x16(lane_addr + set * 256 + 128, vb);
                tmem_ld_wait();
                gg_fold16(va, vb, uw256, ux, acc);
                tmem_ld_32x16(lane_addr + set * 256 + 16, va);
                tmem_ld_32x16(lane_addr + set * 256 + 128 + 16, vb);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[set]);   // both halves are in registers
                gg_fold16(va, vb, uw256, ux + 16, acc + 8);
            }
            if (!ok) break;
            if (row_ok) {
                const bool whole = g0 == 0 && g1 == p.groups;   // otherwise another CTA holds the rest of this tile's K range
                float* out_t = p.out[ti];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const uint32_t t = col0 + c;
                    float lo, hi;
                    unpack2(acc[c / 2], lo, hi);
                    float* o = out_t + static_cast<size_t>(t) * rows + r;
                    if (whole) {
                        if (t < p.tokens) o[0] = lo;
                        if (t + 1 < p.tokens) o[rows] = hi;
                    } else {
                        if (t < p.tokens) atomicAdd(o, lo);
                        if (t + 1 < p.tokens) atomicAdd(o + rows, hi);
                    }
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

// ---- two-digit planes --------------------------------------------------------------------------------------------------

// Eight values of a lane -> their group's unit (max |v| of the 256 values of the warp / 32639) and two digits each.
__device__ __forceinline__ float group_digits8(const float (&v)[8], uint2& hi, uint2& lo) {
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float u = amax > 0.0f ? amax / kGgFullScale : 0.0f;
    const float inv = u > 0.0f ? 1.0f / u : 0.0f;
    uint32_t h[2] = {0, 0}, l[2] = {0, 0};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        int V = __float2int_rn(v[k] * inv);
        V = max(-32639, min(32639, V));
        const int H = (V + 128) >> 8;             // floor((V + 128) / 256): the low digit lands in -128..127
        const int L = V - 256 * H;
        h[k >> 2] |= (static_cast<uint32_t>(H) & 0xffu) << (8 * (k & 3));
        l[k >> 2] |= (static_cast<uint32_t>(L) & 0xffu) << (8 * (k & 3));
    }
    hi = make_uint2(h[0], h[1]);
    lo = make_uint2(l[0], l[1]);
    return u;
}

// Q8_0 planes (codes [rows][K] int8, f16 block scales [rows][nbp]) -> wh, wl [rows][K] int8 and units [rows][K / 256].
// One warp per (row, group); a lane owns a quarter of a 32-weight block.
__global__ void __launch_bounds__(256) group_digits_q8_0_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, uint32_t nbp,
                                                                int8_t* __restrict__ wh, int8_t* __restrict__ wl, float* __restrict__ unit,
                                                                size_t rows, uint32_t K) {
    const size_t wid = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t groups = K / kGgGroup;
    if (wid >= rows * groups) return;
    const size_t r = wid / groups;
    const uint32_t g = static_cast<uint32_t>(wid % groups);
    const size_t e0 = r * K + static_cast<size_t>(g) * kGgGroup + lane * 8;
    const uint2 q = *reinterpret_cast<const uint2*>(codes + e0);
    const float d = __half2float(scales[r * nbp + g * 8 + (lane >> 2)]);
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = d * static_cast<float>(static_cast<int8_t>((k < 4 ? q.x : q.y) >> (8 * (k & 3))));
    uint2 hi, lo;
    const float u = group_digits8(v, hi, lo);
    *reinterpret_cast<uint2*>(wh + e0) = hi;
    *reinterpret_cast<uint2*>(wl + e0) = lo;
    if (lane == 0) unit[r * groups + g] = u;
}

// The same from the device planes of the other formats (repack.cuh): the dequantised value of every weight, formed as the
// reference forms it, then the group's two digits.  A lane owns eight consecutive weights of the group.
//   Q4_0        w = d * (n - 8)                          nibble plane [rows][K / 2], f16 scales [rows][nbp]
//   Q6_K codes  w = (d * sc) * q                         codes q - 32 [rows][K] int8, sc [rows][K / 16], d [rows][sbp]
//   Q4_K, Q5_K  w = (d * sc) * q - (dmin * m)            nibbles [rows][K / 2], (fifth bits [rows][K / 8],) scales|mins [rows][K / 16], (d, dmin) [rows][sbp]
template <int kFormat>
__global__ void __launch_bounds__(256) group_digits_kq_kernel(const uint8_t* __restrict__ p0, const uint8_t* __restrict__ p1, const uint8_t* __restrict__ p2,
                                                              const uint8_t* __restrict__ p3, uint32_t nbp, int8_t* __restrict__ wh, int8_t* __restrict__ wl,
                                                              float* __restrict__ unit, size_t rows, uint32_t K) {
    const size_t wid = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t groups = K / kGgGroup;
    if (wid >= rows * groups) return;
    const size_t r = wid / groups;
    const uint32_t g = static_cast<uint32_t>(wid % groups);
    float v[8];
    if constexpr (kFormat == 2) {          // Q4_0: block g * 8 + lane / 4, elements (lane % 4) * 8 .. + 7 of it
        const uint32_t b = g * 8 + (lane >> 2), o = (lane & 3) * 8;
        const uint2 n = *reinterpret_cast<const uint2*>(p0 + r * (K / 2) + static_cast<size_t>(b) * 16 + (o & 15));
        const uint32_t sh = o >= 16 ? 4u : 0u;      // low nibbles are elements 0..15, high nibbles 16..31 (src/quant.cpp:391-397)
        const float d = __half2float(reinterpret_cast<const __half*>(p1)[r * nbp + b]);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = d * static_cast<float>(static_cast<int>(((k < 4 ? n.x : n.y) >> (8 * (k & 3) + sh)) & 15u) - 8);
    } else if constexpr (kFormat == 114) { // Q6_K, codes unpacked: super-block g, group lane / 2
        const uint2 q = *reinterpret_cast<const uint2*>(p0 + r * K + static_cast<size_t>(g) * 256 + lane * 8);
        const float sc = static_cast<float>(reinterpret_cast<const int8_t*>(p1)[r * (K / 16) + g * 16 + (lane >> 1)]);
        const float ds = __half2float(reinterpret_cast<const __half*>(p2)[r * nbp + g]) * sc;     // (d * scale): the reference's order (kernels/avx2.cpp:380-422)
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = ds * static_cast<float>(static_cast<int8_t>((k < 4 ? q.x : q.y) >> (8 * (k & 3))));
    } else {                               // Q4_K (12) / Q5_K (13): sub-block j = lane / 4, elements l = (lane % 4) * 8 .. + 7 of it
        constexpr bool kQ5 = kFormat == 13;
        const uint8_t* scm = kQ5 ? p2 : p1;
        const uint8_t* dd = kQ5 ? p3 : p2;
        const uint32_t j = lane >> 2, l = (lane & 3) * 8;
        const uint2 n = *reinterpret_cast<const uint2*>(p0 + r * (K / 2) + static_cast<size_t>(g) * 128 + (j >> 1) * 32 + l);
        uint2 h = make_uint2(0u, 0u);
        if (kQ5) h = *reinterpret_cast<const uint2*>(p1 + r * (K / 8) + static_cast<size_t>(g) * 32 + l);
        const uint32_t sh = (j & 1) * 4;
        const uint8_t* sm = scm + r * (K / 16) + static_cast<size_t>(g) * 16;
        const float2 dm = __half22float2(reinterpret_cast<const __half2*>(dd)[r * nbp + g]);
        const float ds = dm.x * static_cast<float>(sm[j]), ms = dm.y * static_cast<float>(sm[8 + j]);   // the reference's factors (kernels/avx2.cpp:329-378)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t nw = k < 4 ? n.x : n.y, hw = k < 4 ? h.x : h.y;
            const uint32_t q = ((nw >> (8 * (k & 3) + sh)) & 15u) | (((hw >> (8 * (k & 3) + j)) & 1u) << 4);
            v[k] = ds * static_cast<float>(q) - ms;
        }
    }
    uint2 hi, lo;
    const float u = group_digits8(v, hi, lo);
    const size_t e0 = r * K + static_cast<size_t>(g) * kGgGroup + lane * 8;
    *reinterpret_cast<uint2*>(wh + e0) = hi;
    *reinterpret_cast<uint2*>(wl + e0) = lo;
    if (lane == 0) unit[r * groups + g] = u;
}

// Activations x [tokens][K] fp32 -> xh, xl [tokens][K] int8 and units [K / 256][t_ld] (group-major).  int8_mode: the values
// are first quantised per 32-block exactly as the reference's int8 route does (round(x * 127 / amax), fp32 scale), and it is
// d_x * q_x that gets the two digits; otherwise x itself (the reference's fp32-activation prefill).
__global__ void __launch_bounds__(256) group_digits_acts_kernel(const float* __restrict__ x, int8_t* __restrict__ xh, int8_t* __restrict__ xl,
                                                                float* __restrict__ unit_t, uint32_t tokens, uint32_t K, uint32_t t_ld, int int8_mode) {
    const size_t wid = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t groups = K / kGgGroup;
    if (wid >= static_cast<size_t>(tokens) * groups) return;
    const uint32_t t = static_cast<uint32_t>(wid / groups), g = static_cast<uint32_t>(wid % groups);
    const size_t e0 = static_cast<size_t>(t) * K + static_cast<size_t>(g) * kGgGroup + lane * 8;
    const float4 a = *reinterpret_cast<const float4*>(x + e0), b = *reinterpret_cast<const float4*>(x + e0 + 4);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (int8_mode) {
        uint2 c1, c2;
        const float d = quantise_block_quad(v, c1, c2);   // the four lanes of a block agree on d; c1 are the Q8 codes
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = d * static_cast<float>(static_cast<int8_t>((k < 4 ? c1.x : c1.y) >> (8 * (k & 3))));
    }
    uint2 hi, lo;
    const float u = group_digits8(v, hi, lo);
    *reinterpret_cast<uint2*>(xh + e0) = hi;
    *reinterpret_cast<uint2*>(xl + e0) = lo;
    if (lane == 0) unit_t[static_cast<size_t>(g) * t_ld + t] = u;
}

}  // namespace zk
