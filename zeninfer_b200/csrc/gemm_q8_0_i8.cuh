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
// Two activation digits (kDigits == 2): the reference's default prefill kernel takes fp32 activations
// (src/quant.cpp:1667-1680 -> gemm_q8_0_kblk_avx2, kernels/avx2.cpp:878-1248).  Here an activation enters as
// (d/256) * (256 * q1 + q2), q1 the Q8 code and q2 the code of the residual (quantize_acts.cuh; error below d/512), so
// a block costs two MMAs (weights x q1, weights x q2) into the two buffers of a TMEM pair, and the epilogue forms
// 256 * S1 + S2 with one integer multiply-add before the single conversion.  |256 * S1 + S2| < 2^27, so that
// conversion rounds at 2^-24 relative: the result stays within ~1e-5 of the fp32-activation product.
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
// Narrow tiles (32 columns: a handful of activation rows) are bound by the latency of the hand-offs, not by bytes or
// arithmetic: they get a deeper ring and, below, all of TMEM as accumulator buffers.
__host__ __device__ constexpr int gemm_stages(uint32_t n_tile) { return n_tile <= 32 ? 8 : kGemmStages; }
#ifndef ZK_GEMM_EPI_WARPS
#define ZK_GEMM_EPI_WARPS 16
#endif
constexpr int kGemmEpiWarps = ZK_GEMM_EPI_WARPS;   // four (or two) per TMEM lane quadrant
constexpr int kGemmSplit = kGemmEpiWarps / 4;  // the warps of a quadrant split the token columns
constexpr int kGemmThreads = (2 + kGemmEpiWarps) * 32;
constexpr int kGemmMaxN = 256;         // tokens per tile, a multiple of 32

constexpr int kGemmMaxTensors = 3;     // weight tensors of one launch (they share the activation block): q|k|v, gate|up

struct GemmParams {
    CUtensorMap map_w[kGemmMaxTensors];  // weight codes  [rows][K] int8, box 128 B x 128 rows, SWIZZLE_128B
    CUtensorMap map_x;                 // act codes     [tokens_padded][K] int8, box 128 B x n_tile rows, SWIZZLE_128B
    CUtensorMap map_x2;                // fine digits   same shape (two-digit kernels only)
    CUtensorMap map_xs;                // act scales    [nb][t_ld] fp32 (block-major), box n_tile x 4
    const __half* w_scales[kGemmMaxTensors];   // [rows][nbp]: Q8_0 block scales; Q6_K: super-block scales
    const int8_t* w_group_scales[kGemmMaxTensors];   // Q6_K only: [rows][group_pitch] int8, one per 16 weights
    uint32_t group_pitch;
    CUtensorMap map_zs;                // kOffsets only: [nb][t_ld] fp32, (d_x / 256) * (sum of the block's two-digit activation codes)
    const float* w_scales32[kGemmMaxTensors];   // kOffsets only: [rows][nb] fp32 block scales (d * sc) ...
    const float* w_offsets[kGemmMaxTensors];    // ... and block offsets (dmin * m), subtracted per unit of activation sum
    float* out[kGemmMaxTensors];               // [tokens][rows]
    uint32_t rows[kGemmMaxTensors];
    uint32_t m_start[kGemmMaxTensors];         // first row tile of each tensor in the launch's row-tile numbering (0xffffffff: unused)
    uint32_t tensors, tokens, nb, nbp;
    uint32_t n_tile;                   // tokens per tile: 32, 64, 128 or 256
    uint32_t m_tiles, n_tiles;         // m_tiles: row tiles of all the tensors together
    uint32_t stream_k;                 // 1: CTAs share the (tile, K tile) units evenly (see GemmWork); 0: whole tiles in turn
    int* error_word;
};

// A stage: weight tile | activation codes | (fine digits) | activation scales, the last rounded up so that the next
// stage's swizzled tiles start on a 1024-byte boundary again.
__host__ __device__ constexpr uint32_t gemm_stage_bytes(uint32_t n_tile, uint32_t digits = 1, bool offsets = false) {
    return kGemmM * kGemmKTile + digits * n_tile * kGemmKTile + (offsets ? 2u : 1u) * ((kGemmBlocksPerTile * n_tile * 4 + 1023u) & ~1023u);
}
__host__ __device__ inline size_t gemm_smem_bytes(uint32_t n_tile, uint32_t digits = 1, bool offsets = false) {
    return 1024 /* alignment slack */ + static_cast<size_t>(gemm_stages(n_tile)) * gemm_stage_bytes(n_tile, digits, offsets) + 512 /* barriers */;
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
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// acc[c/2] += float(v[c], v[c+1]) * (sw * sx[c], sw * sx[c+1]) for 32 token columns: one conversion per sum (exact:
// |sum| < 2^24), one packed multiply and one packed multiply-add per pair of token columns.
__device__ __forceinline__ float int_to_float(uint32_t v) { return static_cast<float>(static_cast<int>(v)); }
// Four consecutive activation scales from the stage, by shared-memory address: the same address in every lane (a
// broadcast), and a 32-bit shared-space address with an immediate offset costs no address arithmetic, where a generic
// pointer costs a 64-bit add per load and a slower load.
#define ZK_LDS128(v, addr, byte_off) \
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4+" #byte_off "];" : "=r"((v).x), "=r"((v).y), "=r"((v).z), "=r"((v).w) : "r"(addr))

__device__ __forceinline__ void gemm_fma4(const uint32_t* v, uint64_t sw2, const uint4& s4, uint64_t* acc) {
    uint64_t s01, s23;
    asm("mov.b64 %0, {%1, %2};" : "=l"(s01) : "r"(s4.x), "r"(s4.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(s23) : "r"(s4.z), "r"(s4.w));
    const uint64_t f01 = pack2(int_to_float(v[0]), int_to_float(v[1]));
    const uint64_t f23 = pack2(int_to_float(v[2]), int_to_float(v[3]));
    acc[0] = fma2(f01, mul2(s01, sw2), acc[0]);
    acc[1] = fma2(f23, mul2(s23, sw2), acc[1]);
}
__device__ __forceinline__ void gemm_fma32(const uint32_t (&v)[32], uint64_t sw2, uint32_t sx_addr, uint64_t* __restrict__ acc) {
    uint4 s;
    ZK_LDS128(s, sx_addr, 0);   gemm_fma4(v + 0, sw2, s, acc + 0);
    ZK_LDS128(s, sx_addr, 16);  gemm_fma4(v + 4, sw2, s, acc + 2);
    ZK_LDS128(s, sx_addr, 32);  gemm_fma4(v + 8, sw2, s, acc + 4);
    ZK_LDS128(s, sx_addr, 48);  gemm_fma4(v + 12, sw2, s, acc + 6);
    ZK_LDS128(s, sx_addr, 64);  gemm_fma4(v + 16, sw2, s, acc + 8);
    ZK_LDS128(s, sx_addr, 80);  gemm_fma4(v + 20, sw2, s, acc + 10);
    ZK_LDS128(s, sx_addr, 96);  gemm_fma4(v + 24, sw2, s, acc + 12);
    ZK_LDS128(s, sx_addr, 112); gemm_fma4(v + 28, sw2, s, acc + 14);
}

// Sixteen token columns of a two-digit block: v1 holds the sums over the Q8 codes, v2 those over the fine digits.
__device__ __forceinline__ void gemm_fma16_two(uint32_t (&v1)[16], const uint32_t (&v2)[16], uint64_t sw2, uint32_t sx_addr, uint64_t* __restrict__ acc) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v1[i] = static_cast<uint32_t>(static_cast<int>(v1[i]) * 256 + static_cast<int>(v2[i]));
    uint4 s;
    ZK_LDS128(s, sx_addr, 0);   gemm_fma4(v1 + 0, sw2, s, acc + 0);
    ZK_LDS128(s, sx_addr, 16);  gemm_fma4(v1 + 4, sw2, s, acc + 2);
    ZK_LDS128(s, sx_addr, 32);  gemm_fma4(v1 + 8, sw2, s, acc + 4);
    ZK_LDS128(s, sx_addr, 48);  gemm_fma4(v1 + 12, sw2, s, acc + 6);
}

// Sixteen token columns of the offset term of a block: acc -= offset * zs[c], zs = (d_x / 256) * (sum of the block's codes).
__device__ __forceinline__ void gemm_off16(uint64_t neg_off2, uint32_t zs_addr, uint64_t* __restrict__ acc) {
    uint4 z;
    uint64_t z01, z23;
#define ZK_OFF4(byte_off, a)                                                     \
    ZK_LDS128(z, zs_addr, byte_off);                                             \
    asm("mov.b64 %0, {%1, %2};" : "=l"(z01) : "r"(z.x), "r"(z.y));                \
    asm("mov.b64 %0, {%1, %2};" : "=l"(z23) : "r"(z.z), "r"(z.w));                \
    acc[a] = fma2(z01, neg_off2, acc[a]);                                        \
    acc[a + 1] = fma2(z23, neg_off2, acc[a + 1]);
    ZK_OFF4(0, 0) ZK_OFF4(16, 2) ZK_OFF4(32, 4) ZK_OFF4(48, 6)
#undef ZK_OFF4
}

// Which tensor a row tile of the launch belongs to, and its index there.
__device__ __forceinline__ void gemm_locate(const GemmParams& p, uint32_t mt_all, uint32_t& ti, uint32_t& mt) {
    ti = (mt_all >= p.m_start[1] ? 1u : 0u) + (mt_all >= p.m_start[2] ? 1u : 0u);
    mt = mt_all - p.m_start[ti];
}

// The work of one CTA.  With `stream_k` the (tile, K tile) units of the whole product, tile-major, are cut into
// gridDim.x equal contiguous ranges, so every SM gets the same number of K tiles even when the tile count is not a
// multiple of the SM count (448 tiles on 148 SMs would otherwise take four rounds for 3.03 rounds of work).  A
// range is at least one tile long, so a tile is shared by at most two CTAs; both add their partial sums to an
// output that gemm_zero_split_tiles_kernel cleared, and the sum of two floats does not depend on their order.
// Without it, CTAs take whole tiles in turn.
struct GemmWork {
    uint32_t u, u_end, ktiles, stride;   // stride != 0: whole tiles, `u` counts tiles
    __device__ GemmWork(const GemmParams& p, uint32_t ktiles_) : ktiles(ktiles_) {
        const uint32_t tiles = p.m_tiles * p.n_tiles;
        if (p.stream_k) {
            const uint64_t total = static_cast<uint64_t>(tiles) * ktiles;
            u = static_cast<uint32_t>(total * blockIdx.x / gridDim.x);
            u_end = static_cast<uint32_t>(total * (blockIdx.x + 1) / gridDim.x);
            stride = 0;
        } else {
            u = blockIdx.x; u_end = tiles; stride = gridDim.x;
        }
    }
    __device__ bool next(uint32_t& tile, uint32_t& kt0, uint32_t& kt1) {
        if (u >= u_end) return false;
        if (stride) { tile = u; kt0 = 0; kt1 = ktiles; u += stride; return true; }
        tile = u / ktiles; kt0 = u % ktiles;
        kt1 = min(ktiles, kt0 + (u_end - u));
        u += kt1 - kt0;
        return true;
    }
};

// Clears the output tiles that two CTAs of a stream-K launch share (launched right before it, same grid).
__global__ void gemm_zero_split_tiles_kernel(const __grid_constant__ GemmParams p, uint32_t ktiles) {
    if (blockIdx.x == 0) return;
    const uint64_t total = static_cast<uint64_t>(p.m_tiles) * p.n_tiles * ktiles;
    const uint32_t cut = static_cast<uint32_t>(total * blockIdx.x / gridDim.x);
    if (cut % ktiles == 0) return;   // the boundary falls between two tiles
    const uint32_t tile = cut / ktiles, nt = tile / p.m_tiles;
    uint32_t ti, mt;
    gemm_locate(p, tile % p.m_tiles, ti, mt);
    float* out = p.out[ti];
    const uint32_t rows = p.rows[ti];
    for (uint32_t i = threadIdx.x; i < p.n_tile * kGemmM; i += blockDim.x) {
        const uint32_t t = nt * p.n_tile + i / kGemmM, r = mt * kGemmM + i % kGemmM;
        if (t < p.tokens && r < rows) out[static_cast<size_t>(t) * rows + r] = 0.0f;
    }
}

// Eighteen warps put five on one of the SM's four register files (16384 registers each), so 96 registers per thread is
// the ceiling: 5 x 32 x 96 = 15360.
//
// kQ6K: the weights are Q6_K with the codes unpacked (q - 32 as int8 [rows][K], gemv_kq.cuh), two activation digits.  A
// 16-weight group has its own int8 scale (src/quant.cpp:500-517), but one instruction sums K = 32 = two groups.  The
// groups are kept apart on the activation side: token t enters as TWO columns, 2 t with the codes of the odd groups
// zeroed and 2 t + 1 with those of the even groups zeroed (quantize_acts_q6k_gemm_kernel).  Column 2 t of a block's sums
// is then the even group's integer dot product and column 2 t + 1 the odd group's, and the packed pair of accumulators
// (2 t, 2 t + 1) takes the pair of group scales (d * sc_even, d * sc_odd); a token's output is the sum of its pair.  A tile
// of kNTile columns holds kNTile / 2 tokens; with kNTile = 32 this is the product for the two to sixteen activation rows of
// batched decoding (the lm_head for eight sequences) as well as the reference's gemm_q6k_kblk_avx2 (kernels/avx2.cpp:1762-1770).
//
// kOffsets: blocks of the form w = scale * q - offset with fp32 scale and offset per (row, 32-block): Q4_K and Q5_K with
// their codes widened to int8 per call (scale = d * sc, offset = dmin * m; repack.cuh, unpack_k45_codes_kernel).  The
// epilogue takes the scales from a fp32 plane and subtracts offset * zs[t, b], zs = (d_x / 256) * (sum of the block's
// two-digit activation codes), which travels through the ring like the activation scales.
template <int kNTile, int kDigits = 1, bool kQ6K = false, bool kOffsets = false>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_q8_0_i8_kernel(const __grid_constant__ GemmParams p) {
    static_assert(kDigits == 1 || kDigits == 2, "one or two activation digits");
    static_assert(!kQ6K || kDigits == 2, "Q6_K takes fp32-equivalent activations");
    static_assert(!kOffsets || (kDigits == 2 && !kQ6K), "offset blocks take fp32-equivalent activations");
    constexpr int kSplit = kNTile >= 128 ? kGemmSplit : kNTile / 16;   // warps of a lane quadrant that share a tile's columns
    constexpr int kEpiActive = 4 * kSplit;                              // narrow tiles leave the other epilogue warps idle
    static_assert(kSplit >= 1 && kSplit <= kGemmSplit, "tile width");
    constexpr int kNHalf = kNTile / kSplit;         // token columns per epilogue warp
    static_assert(kNHalf % (kDigits == 2 ? 16 : 32) == 0, "an epilogue warp takes whole 32-column (two digits: 16-column) chunks");
    constexpr int kStages = gemm_stages(kNTile);
    constexpr uint32_t kPairs = 512 / (2 * kNTile) < 8 ? 512 / (2 * kNTile) : 8;   // TMEM accumulator buffers come in pairs (one hand-off per pair): 2 pairs of 128 columns, 8 of 32
    constexpr uint32_t kStageBytes = gemm_stage_bytes(kNTile, kDigits, kOffsets);
    constexpr uint32_t kScaleOff = kGemmM * kGemmKTile + kDigits * kNTile * kGemmKTile;   // the stage: weights | codes | (fine digits) | scales | (code sums)
    constexpr uint32_t kZsOff = kScaleOff + ((kGemmBlocksPerTile * kNTile * 4 + 1023u) & ~1023u);
    constexpr uint32_t kLoadBytes = kScaleOff + (kOffsets ? 2 : 1) * kGemmBlocksPerTile * kNTile * 4;   // what the copies of a stage deliver
    static_assert(kStageBytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
    constexpr uint32_t kTmemCols = 2 * kPairs * kNTile;  // four accumulator buffers of kNTile columns: a power of two
    static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM allocations are powers of two from 32 to 512 columns");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* tmem_full = empty + kStages;
    uint64_t* tmem_empty = tmem_full + kPairs;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + kPairs);
    static_assert((2 * kStages + 2 * kPairs) * 8 + 8 <= 512, "barrier area");
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ktiles = (p.nb + kGemmBlocksPerTile - 1) / kGemmBlocksPerTile;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1 + kEpiActive);
        }
        for (int b = 0; b < static_cast<int>(kPairs); ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpiActive);
        }
        *abort_word = 0;
        mbar_fence_init();
        for (uint32_t i = 0; i < p.tensors; ++i) tma_prefetch_descriptor(&p.map_w[i]);
        tma_prefetch_descriptor(&p.map_x);
        if (kDigits == 2) tma_prefetch_descriptor(&p.map_x2);
        tma_prefetch_descriptor(&p.map_xs);
        if (kOffsets) tma_prefetch_descriptor(&p.map_zs);
    }
    if (warp == 1) tmem_alloc(tmem_base_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0, tile, kt0, kt1;
            bool ok = true;
            GemmWork work(p, ktiles);
            while (ok && work.next(tile, kt0, kt1)) {
                const uint32_t nt = tile / p.m_tiles;
                uint32_t ti, mt;
                gemm_locate(p, tile % p.m_tiles, ti, mt);
                const CUtensorMap* map_w = &p.map_w[ti];
                for (uint32_t kt = kt0; kt < kt1; ++kt, ++it) {
                    const uint32_t stage = it % kStages;
                    if (it >= kStages && !mbar_wait(&empty[stage], ((it / kStages) - 1) & 1)) {
                        *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); ok = false;
                    }
                    if (*abort_word) ok = false;
                    if (!ok) break;
                    uint8_t* st = smem + stage * kStageBytes;
                    mbar_arrive_expect_tx(&full[stage], kLoadBytes);
                    tma_load_2d(st, map_w, static_cast<int>(kt * kGemmKTile), static_cast<int>(mt * kGemmM), &full[stage]);
                    tma_load_2d(st + kGemmM * kGemmKTile, &p.map_x, static_cast<int>(kt * kGemmKTile), static_cast<int>(nt * kNTile), &full[stage]);
                    if (kDigits == 2)
                        tma_load_2d(st + kGemmM * kGemmKTile + kNTile * kGemmKTile, &p.map_x2, static_cast<int>(kt * kGemmKTile), static_cast<int>(nt * kNTile), &full[stage]);
                    tma_load_2d(st + kScaleOff, &p.map_xs, static_cast<int>(nt * kNTile), static_cast<int>(kt * kGemmBlocksPerTile), &full[stage]);
                    if (kOffsets) tma_load_2d(st + kZsOff, &p.map_zs, static_cast<int>(nt * kNTile), static_cast<int>(kt * kGemmBlocksPerTile), &full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(kGemmM, kNTile);
            uint32_t it = 0, pair = 0, tile, kt0, kt1;
            bool ok = true;
            GemmWork work(p, ktiles);
            while (ok && work.next(tile, kt0, kt1)) {
                for (uint32_t kt = kt0; kt < kt1 && ok; ++kt, ++it) {
                    const uint32_t stage = it % kStages;
                    if (*abort_word || !mbar_wait(&full[stage], (it / kStages) & 1)) {
                        if (!*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
                    const uint64_t a_desc = umma_desc_k_sw128(a_addr), b_desc = umma_desc_k_sw128(a_addr + kGemmM * kGemmKTile);
                    const uint32_t nblk = min(static_cast<uint32_t>(kGemmBlocksPerTile), p.nb - kt * kGemmBlocksPerTile);
                    for (uint32_t j0 = 0; j0 < nblk; j0 += (kDigits == 2 ? 1 : 2), ++pair) {
                        const uint32_t pr = pair % kPairs;
                        if (pair >= kPairs) {
                            if (!mbar_wait(&tmem_empty[pr], ((pair / kPairs) - 1) & 1)) {
                                *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                        }
                        // one Q8_0 block per instruction: 32 bytes of K = two 16-byte units further into the swizzle atom
                        if (kDigits == 2) {   // the block's two digits fill the pair
                            const uint64_t b2_desc = umma_desc_k_sw128(a_addr + kGemmM * kGemmKTile + kNTile * kGemmKTile);
                            tc_mma_i8(tmem_base + (2 * pr) * kNTile, a_desc + 2 * j0, b_desc + 2 * j0, idesc, 0u);
                            tc_mma_i8(tmem_base + (2 * pr + 1) * kNTile, a_desc + 2 * j0, b2_desc + 2 * j0, idesc, 0u);
                        } else {
                            tc_mma_i8(tmem_base + (2 * pr) * kNTile, a_desc + 2 * j0, b_desc + 2 * j0, idesc, 0u);
                            if (j0 + 1 < nblk) tc_mma_i8(tmem_base + (2 * pr + 1) * kNTile, a_desc + 2 * (j0 + 1), b_desc + 2 * (j0 + 1), idesc, 0u);
                        }
                        tc_commit(&tmem_full[pr]);
                    }
                    if (ok) tc_commit(&empty[stage]);  // the stage is free once its MMAs have read it
                }
            }
        }
    } else if (warp - 2 < kEpiActive) {
        // ---------------- epilogue warps ----------------
        const int e = warp - 2;
        const uint32_t quad = static_cast<uint32_t>(warp) & 3;   // the TMEM lanes a warp may touch: 32 * (warp id % 4)
        const uint32_t half = static_cast<uint32_t>(e) >> 2;      // which share of the token columns this warp takes
        const uint32_t taddr0 = tmem_base + ((quad * 32) << 16) + half * kNHalf;
        uint32_t it = 0, pair = 0, tile, kt0, kt1;
        bool ok = true;
        GemmWork work(p, ktiles);
        while (ok && work.next(tile, kt0, kt1)) {
            const uint32_t nt = tile / p.m_tiles;
            uint32_t ti, mt;
            gemm_locate(p, tile % p.m_tiles, ti, mt);
            const uint32_t r = mt * kGemmM + quad * 32 + lane, rows = p.rows[ti];
            const bool row_ok = r < rows;
            // Q6_K: a warp whose columns all lie past the last token (eight rows fill half a tile) only keeps the hand-offs going
            const bool live_cols = !kQ6K || nt * kNTile + half * kNHalf < 2 * p.tokens;
            uint64_t acc[kNHalf / 2];  // packed pairs of fp32 accumulators, token columns (2i, 2i+1)
#pragma unroll
            for (int c = 0; c < kNHalf / 2; ++c) acc[c] = 0ull;
            // the four weight scales of row r per K tile (8-byte aligned: nbp is a multiple of 8), fetched one K tile ahead
            // Q6_K: a K tile is eight groups, i.e. eight int8 group scales (8-byte aligned) and half a super-block
            // offset blocks: four fp32 scales and four fp32 offsets per K tile (16-byte aligned: nb is a multiple of 8)
            const uint2* sw_row = kOffsets ? nullptr
                                  : kQ6K   ? reinterpret_cast<const uint2*>(p.w_group_scales[ti] + static_cast<size_t>(row_ok ? r : 0) * p.group_pitch)
                                           : reinterpret_cast<const uint2*>(p.w_scales[ti] + static_cast<size_t>(row_ok ? r : 0) * p.nbp);
            const __half* d_row = kOffsets ? nullptr : p.w_scales[ti] + static_cast<size_t>(row_ok ? r : 0) * p.nbp;   // Q6_K: super-block scales
            const float4* s32_row = kOffsets ? reinterpret_cast<const float4*>(p.w_scales32[ti] + static_cast<size_t>(row_ok ? r : 0) * p.nb) : nullptr;
            const float4* o32_row = kOffsets ? reinterpret_cast<const float4*>(p.w_offsets[ti] + static_cast<size_t>(row_ok ? r : 0) * p.nb) : nullptr;
            uint2 sw_next = make_uint2(0u, 0u);
            float4 s32_next = make_float4(0.f, 0.f, 0.f, 0.f), o32_next = s32_next;
            if constexpr (kOffsets) { s32_next = __ldg(s32_row + kt0); o32_next = __ldg(o32_row + kt0); }
            else sw_next = __ldg(sw_row + kt0);
            for (uint32_t kt = kt0; kt < kt1 && ok; ++kt, ++it) {
                const uint32_t stage = it % kStages;
                const uint2 sw4 = sw_next;
                const float4 s32 = s32_next, o32 = o32_next;
                if (kt + 1 < kt1) {
                    if constexpr (kOffsets) { s32_next = __ldg(s32_row + kt + 1); o32_next = __ldg(o32_row + kt + 1); }
                    else sw_next = __ldg(sw_row + kt + 1);
                }
                float dq = 0.0f;
                if constexpr (kQ6K) dq = __half2float(__ldg(d_row + (kt >> 1))) * 0.00390625f;   // the digits' common unit is d_x / 256
                if (*abort_word || !mbar_wait(&full[stage], (it / kStages) & 1)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                    ok = false;
                    break;
                }
                const uint32_t sxs = smem_u32(smem + stage * kStageBytes + kScaleOff) + half * kNHalf * 4;
                const __half2 h01 = *reinterpret_cast<const __half2*>(&sw4.x), h23 = *reinterpret_cast<const __half2*>(&sw4.y);
                const float swf[4] = {kOffsets ? s32.x : __low2float(h01), kOffsets ? s32.y : __high2float(h01), kOffsets ? s32.z : __low2float(h23),
                                      kOffsets ? s32.w : __high2float(h23)};
                const float off[4] = {o32.x, o32.y, o32.z, o32.w};
                const uint32_t zss = smem_u32(smem + stage * kStageBytes + kZsOff) + half * kNHalf * 4;
                const uint32_t nblk = min(static_cast<uint32_t>(kGemmBlocksPerTile), p.nb - kt * kGemmBlocksPerTile);
                if constexpr (kDigits == 2) {
#pragma unroll
                    for (uint32_t j = 0; j < kGemmBlocksPerTile; ++j) {
                        if (j < nblk && ok) {
                            const uint32_t pr = pair % kPairs;
                            if (!mbar_wait(&tmem_full[pr], (pair / kPairs) & 1)) {
                                if (lane == 0) { *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); }
                                ok = false;
                            } else {
                                tc_fence_after_sync();
                                if (!live_cols) {
                                    tc_fence_before_sync(); __syncwarp();
                                    if (lane == 0) mbar_arrive(&tmem_empty[pr]);
                                    ++pair;
                                    continue;
                                }
                                uint64_t sw2;
                                if constexpr (kQ6K) {   // the block's even and odd group: (d * scale), the reference's factor (kernels/avx2.cpp:380-422)
                                    const uint32_t two = (j < 2 ? sw4.x : sw4.y) >> (16 * (j & 1));
                                    sw2 = pack2(dq * static_cast<float>(static_cast<int8_t>(two)), dq * static_cast<float>(static_cast<int8_t>(two >> 8)));
                                } else {
                                    sw2 = pack2(swf[j] * 0.00390625f, swf[j] * 0.00390625f);   // the digits' common unit is d / 256
                                }
                                uint32_t v1[16], v2[16];
#pragma unroll
                                for (int c = 0; c < kNHalf; c += 16) {
                                    tmem_ld_32x16(taddr0 + (2 * pr) * kNTile + c, v1);
                                    tmem_ld_32x16(taddr0 + (2 * pr + 1) * kNTile + c, v2);
                                    tmem_ld_wait();
                                    if (c + 16 == kNHalf) { tc_fence_before_sync(); __syncwarp(); if (lane == 0) mbar_arrive(&tmem_empty[pr]); }
                                    gemm_fma16_two(v1, v2, sw2, sxs + (j * kNTile + c) * 4, acc + c / 2);
                                    if constexpr (kOffsets) gemm_off16(pack2(-off[j], -off[j]), zss + (j * kNTile + c) * 4, acc + c / 2);
                                }
                                ++pair;
                            }
                        }
                    }
                } else {
#pragma unroll
                for (uint32_t j0 = 0; j0 < kGemmBlocksPerTile; j0 += 2) {
                    if (j0 < nblk && ok) {
                        const uint32_t pr = pair % kPairs;
                        if (!mbar_wait(&tmem_full[pr], (pair / kPairs) & 1)) {
                            if (lane == 0) { *abort_word = 1; atomicExch(p.error_word, kErrTmemWaitTimeout); }
                            ok = false;
                        } else {
                            tc_fence_after_sync();
                            const bool two = j0 + 1 < nblk;
                            uint32_t v[32];
#pragma unroll
                            for (int c = 0; c < kNHalf; c += 32) {
                                tmem_ld_32x32(taddr0 + (2 * pr) * kNTile + c, v);
                                tmem_ld_wait();
                                if (!two && c + 32 == kNHalf) { tc_fence_before_sync(); __syncwarp(); if (lane == 0) mbar_arrive(&tmem_empty[pr]); }
                                gemm_fma32(v, pack2(swf[j0], swf[j0]), sxs + (j0 * kNTile + c) * 4, acc + c / 2);
                            }
                            if (two) {
#pragma unroll
                                for (int c = 0; c < kNHalf; c += 32) {
                                    tmem_ld_32x32(taddr0 + (2 * pr + 1) * kNTile + c, v);
                                    tmem_ld_wait();
                                    if (c + 32 == kNHalf) {   // both buffers of the pair have been read
                                        tc_fence_before_sync();
                                        __syncwarp();
                                        if (lane == 0) mbar_arrive(&tmem_empty[pr]);
                                    }
                                    gemm_fma32(v, pack2(swf[j0 + 1], swf[j0 + 1]), sxs + ((j0 + 1) * kNTile + c) * 4, acc + c / 2);
                                }
                            }
                            ++pair;
                        }
                    }
                }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stage]);  // done with the stage's activation scales
            }
            if (!ok) break;
            if (row_ok) {
                const bool whole = kt0 == 0 && kt1 == ktiles;   // otherwise another CTA holds the rest of this tile's K range
                float* out_t = p.out[ti];
#pragma unroll
                for (int c = 0; c < kNHalf; c += 2) {
                    const uint32_t t = nt * kNTile + half * kNHalf + c;
                    float lo, hi;
                    unpack2(acc[c / 2], lo, hi);
                    if constexpr (kQ6K) {   // columns (2 t, 2 t + 1) are token t's even and odd groups
                        const uint32_t tok = t >> 1;
                        float* o = out_t + static_cast<size_t>(tok) * rows + r;
                        if (tok < p.tokens) { if (whole) o[0] = lo + hi; else atomicAdd(o, lo + hi); }
                        continue;
                    }
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

// Activation quantiser for the GEMM: codes [t_pad][K] int8 (rows >= tokens are zero-filled by the caller's memset)
// and scales in block-major order [nb][t_ld] fp32, so the scales of one block for a tile of tokens are contiguous.
// q2 != nullptr: also the fine digits of the two-digit kernels.
// zs_t != nullptr (offset blocks): also (d / 256) * sum over the block of (256 * q1 + q2), same layout as the scales.
__global__ void __launch_bounds__(256) quantize_acts_gemm_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ sc_t,
                                                                 uint32_t tokens, uint32_t nb, uint32_t t_ld, int8_t* __restrict__ q2,
                                                                 float* __restrict__ zs_t = nullptr) {
    const size_t wid = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<size_t>(tokens) * nb) return;
    const uint32_t t = static_cast<uint32_t>(wid / nb), b = static_cast<uint32_t>(wid % nb);
    int c1, c2;
    const float d = quantise_block_lane(x[wid * 32 + lane], c1, c2);
    q[wid * 32 + lane] = static_cast<int8_t>(c1);
    if (q2) q2[wid * 32 + lane] = static_cast<int8_t>(c2);   // the fine digit, same layout
    if (lane == 0) sc_t[static_cast<size_t>(b) * t_ld + t] = d;
    if (zs_t) {
        int sum = c1 * 256 + c2;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) zs_t[static_cast<size_t>(b) * t_ld + t] = (d * 0.00390625f) * static_cast<float>(sum);
    }
}

// The same for the Q6_K product: token t becomes rows 2 t (codes of the odd 16-weight groups zeroed) and 2 t + 1 (codes
// of the even groups zeroed) of q and q2, and both rows carry the block's scale.  One warp per (token, block).
__global__ void __launch_bounds__(256) quantize_acts_q6k_gemm_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ sc_t,
                                                                     uint32_t tokens, uint32_t nb, uint32_t t_ld, int8_t* __restrict__ q2) {
    const size_t wid = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<size_t>(tokens) * nb) return;
    const uint32_t t = static_cast<uint32_t>(wid / nb), b = static_cast<uint32_t>(wid % nb);
    int c1, c2;
    const float d = quantise_block_lane(x[wid * 32 + lane], c1, c2);
    const size_t K = static_cast<size_t>(nb) * 32;
    const size_t even = (2 * static_cast<size_t>(t)) * K + b * 32 + lane, odd = even + K;
    const bool in_even = lane < 16;   // elements 0..15 of a block are group 2 b, elements 16..31 group 2 b + 1
    q[even] = static_cast<int8_t>(in_even ? c1 : 0);
    q[odd] = static_cast<int8_t>(in_even ? 0 : c1);
    q2[even] = static_cast<int8_t>(in_even ? c2 : 0);
    q2[odd] = static_cast<int8_t>(in_even ? 0 : c2);
    if (lane < 2) sc_t[static_cast<size_t>(b) * t_ld + 2 * t + lane] = d;
}

}  // namespace zk
