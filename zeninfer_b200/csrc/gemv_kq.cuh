// Decode-time matrix-vector products for Q4_0, Q6_K, Q4_K and Q5_K (batch 1..8).
//
// The reference evaluates both formats with fp32 activations: Q4_0 through its generic
// dequantise-then-dot route (src/quant.cpp:1135-1162 over gemv_avx2, kernels/avx2.cpp:16-40) and
// Q6_K through gemv_q6k_avx2 / gemm_q6k_kblk_avx2 (kernels/avx2.cpp:380-422, :1762-1770).  Decoding
// every weight to fp32 costs several ALU operations per weight, more than an SM can issue at HBM
// speed, so the dot products here stay in integers: weights are used as the small integers they
// are, and each activation enters as two int8 digits, x ~= (d/256) * (256*q1 + q2) with an error
// below d/512 (quantize_acts.cuh).  Results agree with the fp32-activation reference to ~1e-5.
//
//   Q4_0 : y += d_w * (d_x/256) * ( sum n*(256*q1+q2)  -  8 * sum(256*q1+q2) )      n = nibble 0..15
//   Q6_K : y += d * sc_g * (d_x/256) * sum (q-32)*(256*q1+q2)                        per 16-weight group
//   Q4_K / Q5_K (the reference: gemv_q4k_q5k_avx2, kernels/avx2.cpp:329-378, fp32 activations; its GPU entry is
//          zen::d3d12::gemm_kquant, include/zen/d3d12_backend.h:75), per 32-weight sub-block g of a super-block:
//          y += d * sc_g * (d_x/256) * sum q*(256*q1+q2)  -  dmin * m_g * (d_x/256) * sum (256*q1+q2)
//          with q the 4-bit (Q4_K) or 5-bit (Q5_K: nibble + 16 * fifth bit) code
//
// Same streaming skeleton as the Q8_0 kernel (gemv_q8_0.cuh): a persistent CTA per SM owns a
// byte-balanced row slice, a producer warp feeds a ring of shared-memory stages with TMA bulk
// copies, sixteen consumer warps in two teams own one row each.  Algorithmic traffic is the raw
// GGUF size (18 B per Q4_0 block, 210 B per Q6_K super-block, 144 / 176 B per Q4_K / Q5_K super-block; the device
// planes of the last two are 4 bytes per super-block larger, because the 12 packed bytes of 6-bit scales and minimums
// are kept unpacked as 16, see repack.cuh).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "gemv_q8_0.cuh"

namespace zk {

constexpr int kKqSegElems = 4096;   // weights per row per stage segment (128 Q4_0 blocks, 16 Q6_K super-blocks)
constexpr int kKqMaxPlanes = 4;
constexpr int kKqPartialFloats = kTeams * 2 * kTeamWarps * kTeamWarps;   // [team][unit parity][K slice][row]

// Per-format geometry of the planes a row is split into (repack.cuh).
template <int kFormat> struct KqFormat;

template <> struct KqFormat<2> {   // Q4_0: nibbles [K/2], f16 scales [K/32]
    static constexpr int kPlanes = 2;
    static constexpr int kStages = 6;   // a multiple of the team count, see kGemvStages
    __host__ __device__ static constexpr uint32_t seg_bytes(int plane) { return plane == 0 ? kKqSegElems / 2 : kKqSegElems / 32 * 2; }
    __host__ __device__ static constexpr uint32_t bytes_per_256(int plane) { return plane == 0 ? 128 : 16; }
};
template <> struct KqFormat<14> {  // Q6_K: ql [K/2], qh [K/4], int8 sc [K/16], f16 d [K/256]
    static constexpr int kPlanes = 4;
    static constexpr int kStages = 4;
    __host__ __device__ static constexpr uint32_t seg_bytes(int plane) {
        return plane == 0 ? kKqSegElems / 2 : plane == 1 ? kKqSegElems / 4 : plane == 2 ? kKqSegElems / 16 : kKqSegElems / 256 * 2;
    }
    __host__ __device__ static constexpr uint32_t bytes_per_256(int plane) { return plane == 0 ? 128 : plane == 1 ? 64 : plane == 2 ? 16 : 2; }
};

template <> struct KqFormat<12> {  // Q4_K: nibbles [K/2], unpacked sub-block scales|minimums [K/16], (d, dmin) f16 pairs [K/256]
    static constexpr int kPlanes = 3;
    static constexpr int kStages = 6;
    __host__ __device__ static constexpr uint32_t seg_bytes(int plane) { return plane == 0 ? kKqSegElems / 2 : plane == 1 ? kKqSegElems / 16 : kKqSegElems / 256 * 4; }
    __host__ __device__ static constexpr uint32_t bytes_per_256(int plane) { return plane == 0 ? 128 : plane == 1 ? 16 : 4; }
};
template <> struct KqFormat<13> {  // Q5_K: nibbles [K/2], fifth bits [K/8], scales|minimums [K/16], (d, dmin) [K/256]
    static constexpr int kPlanes = 4;
    static constexpr int kStages = 4;
    __host__ __device__ static constexpr uint32_t seg_bytes(int plane) {
        return plane == 0 ? kKqSegElems / 2 : plane == 1 ? kKqSegElems / 8 : plane == 2 ? kKqSegElems / 16 : kKqSegElems / 256 * 4;
    }
    __host__ __device__ static constexpr uint32_t bytes_per_256(int plane) { return plane == 0 ? 128 : plane == 1 ? 32 : plane == 2 ? 16 : 4; }
};
// Q6_K with the codes unpacked on upload (kFormatQ6KCodes): q - 32 as one int8 per weight in element order, the group
// scales and super-block scales as in the packed layout.  The device copy is 1.07 bytes per weight instead of the file's
// 0.82, and the inner loop loses the 24 shift/mask operations per 16 weights that rebuild a code from ql and qh: the
// packed kernel is bound by instruction issue at 0.45 of the HBM rate, this one streams 1.3 x the bytes at 0.9 of it.
// The integer sums, and therefore the results, are the packed kernel's bit for bit.
constexpr int kFormatQ6KCodes = 114;
template <> struct KqFormat<kFormatQ6KCodes> {  // codes [K] int8, sc [K/16] int8, d [K/256] f16
    static constexpr int kPlanes = 3;
    static constexpr int kStages = 4;
    __host__ __device__ static constexpr uint32_t seg_bytes(int plane) { return plane == 0 ? kKqSegElems : plane == 1 ? kKqSegElems / 16 : kKqSegElems / 256 * 2; }
    __host__ __device__ static constexpr uint32_t bytes_per_256(int plane) { return plane == 0 ? 256 : plane == 1 ? 16 : 2; }
};
// Q4_K and Q5_K share everything but the fifth-bit plane.
template <int kFormat> constexpr bool kq_is_k45 = kFormat == 12 || kFormat == 13;

template <int kFormat> __host__ __device__ constexpr uint32_t kq_row_stage_bytes() {
    uint32_t b = 0;
    for (int i = 0; i < KqFormat<kFormat>::kPlanes; ++i) b += KqFormat<kFormat>::seg_bytes(i);
    return b;
}
template <int kFormat> __host__ __device__ constexpr uint32_t kq_plane_offset(int plane) {  // within a stage
    uint32_t b = 0;
    for (int i = 0; i < plane; ++i) b += KqFormat<kFormat>::seg_bytes(i) * kTeamWarps;
    return b;
}
template <int kFormat> __host__ __device__ constexpr uint32_t kq_stage_bytes() { return kq_row_stage_bytes<kFormat>() * kTeamWarps; }

// Tensor maps of one resident tensor whose rows span several K segments (built on upload, kept in device memory): per
// plane, boxes of 8, 4, 2 and 1 rows x one segment.  A plane whose segment is at most 256 bytes is a 2-D byte view
// [rows][pitch]; a wider one is the 3-D view [rows][pitch / 256][256], because a tile's innermost extent is limited to
// 256 elements.  One copy per plane then fetches a row group's segment where the per-row path issues 16 to 32 small ones.
struct alignas(64) KqTileMaps {
    CUtensorMap map[kKqMaxPlanes][4];
};

struct KqTask {
    const uint8_t* plane[kKqMaxPlanes];
    float* y;               // [batch][rows]
    uint32_t rows;
    uint32_t first_row;
};

struct KqParams {
    KqTask task[kMaxTasks];
    uint32_t ntasks, total_rows;
    const float* x;         // [batch][K] fp32; null with a gather: the vector gathered by the previous launch
    uint32_t K;             // columns, a multiple of the format's block size
    uint32_t nseg;          // ceil(K / kKqSegElems)
    uint32_t pitch[kKqMaxPlanes];  // global row pitch of each plane, bytes
    int* error_word;
    PeerGather gather;      // world == 0: outputs go to task[].y only
    const KqTileMaps* tile_maps[kMaxTasks];   // null: the tensor's rows go one copy per row and plane when K spans several segments
};

template <int kFormat>
__host__ __device__ inline size_t gemv_kq_smem_bytes(uint32_t nseg, int batch) {
    const size_t kpad = static_cast<size_t>(nseg) * kKqSegElems;
    return static_cast<size_t>(KqFormat<kFormat>::kStages) * kq_stage_bytes<kFormat>()
           + static_cast<size_t>(batch) * 2 * kpad                 // two digit planes, natural order
           + static_cast<size_t>(batch) * (kpad / 32) * 8          // per-block scale (d/256) and code sum
           + 2 * KqFormat<kFormat>::kStages * 8 + 16
           + kKqPartialFloats * sizeof(float);                      // batch 1: per-warp partial row sums
}

struct KqWalk {  // GroupWalk over KqParams
    uint32_t r, r_end, ti;
    __device__ KqWalk(uint32_t first, uint32_t last) : r(first), r_end(last), ti(0) {}
    __device__ bool done() const { return r >= r_end; }
    __device__ RowGroup next(const KqParams& p) {
        RowGroup g{0, 0, 0};
        if (done()) return g;
        while (r >= p.task[ti].first_row + p.task[ti].rows) ++ti;
        g.task = ti;
        g.row0 = r - p.task[ti].first_row;
        g.nrows = min(min(static_cast<uint32_t>(kTeamWarps), p.task[ti].rows - g.row0), r_end - r);
        r += g.nrows;
        return g;
    }
};

__device__ __forceinline__ int dot16(const uint4& w, const uint4& x) {
    int s = dp4a_ss(w.x, x.x, 0);
    s = dp4a_ss(w.y, x.y, s);
    s = dp4a_ss(w.z, x.z, s);
    return dp4a_ss(w.w, x.w, s);
}

// Bytes 0..63 minus 32, per byte, as signed bytes: setting the top bit first keeps the subtraction
// from borrowing across bytes, flipping it back afterwards leaves the two's-complement difference.
__device__ __forceinline__ uint32_t sub32_bytes(uint32_t q) { return ((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u; }

// Sum of `v` over the lanes of a warp for R rows at once.  Each exchange step halves the number of rows a lane still
// carries, so R rows cost R - 1 + (5 - log2 R) shuffles instead of 5 R.  On return every lane holds the complete sum
// of row `row` (lanes that share the low bits hold the same row); the order of additions is fixed.
template <int R>
__device__ __forceinline__ float kq_reduce_rows(const float (&acc)[R], int lane, uint32_t& row) {
    static_assert(R == 4 || R == 8, "four or eight rows per warp");
    float a4[4];
    if constexpr (R == 8) {
        const bool up = lane & 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float send = up ? acc[i] : acc[i + 4], keep = up ? acc[i + 4] : acc[i];
            a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) a4[i] = acc[i];
    }
    constexpr int o2 = R == 8 ? 8 : 16, o1 = R == 8 ? 4 : 8;
    float a2[2];
    {
        const bool up = lane & o2;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float send = up ? a4[i] : a4[i + 2], keep = up ? a4[i + 2] : a4[i];
            a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, o2);
        }
    }
    float a1;
    {
        const bool up = lane & o1;
        const float send = up ? a2[0] : a2[1], keep = up ? a2[1] : a2[0];
        a1 = keep + __shfl_xor_sync(0xffffffffu, send, o1);
    }
#pragma unroll
    for (int o = o1 >> 1; o > 0; o >>= 1) a1 += __shfl_xor_sync(0xffffffffu, a1, o);
    if constexpr (R == 8) row = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    else row = ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1);
    return a1;
}

// Team-wide barrier that also agrees on failure: true when any of the team's threads passed `failed`.
__device__ __forceinline__ bool team_barrier_any(int team, bool failed) {
    uint32_t any;
    asm volatile(
        "{ .reg .pred p, q; setp.ne.u32 q, %3, 0; barrier.red.or.pred p, %1, %2, q; selp.u32 %0, 1, 0, p; }"
        : "=r"(any) : "r"(2 + team), "r"(kTeamWarps * 32), "r"(static_cast<uint32_t>(failed)) : "memory");
    return any != 0;
}

template <int kFormat, int kBatch>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kq_kernel(const __grid_constant__ KqParams p) {
    using F = KqFormat<kFormat>;
    constexpr int kStages = F::kStages;
    static_assert(kStages % kTeams == 0, "ring depth must be a multiple of the number of consumer teams");
    constexpr uint32_t kStageBytes = kq_stage_bytes<kFormat>();
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t kpad = p.nseg * kKqSegElems;
    uint8_t* ring = smem;
    uint8_t* xd = ring + kStages * kStageBytes;                                  // [batch][2][kpad] int8, natural order
    float* xscale = reinterpret_cast<float*>(xd + static_cast<size_t>(kBatch) * 2 * kpad);   // [batch][kpad/32]  d/256
    int* xsum = reinterpret_cast<int*>(xscale + static_cast<size_t>(kBatch) * (kpad / 32));  // [batch][kpad/32]  sum(256*q1+q2)
    uint64_t* full = reinterpret_cast<uint64_t*>(xsum + static_cast<size_t>(kBatch) * (kpad / 32));
    uint64_t* empty = full + kStages;
    volatile int* abort_word = reinterpret_cast<volatile int*>(empty + kStages);
    float* partial = reinterpret_cast<float*>(empty + kStages + 2);   // batch 1: [team][unit parity][K slice][row]
    float* stash = partial + kKqPartialFloats;                        // gather only: [batch][rows of this CTA's slice]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t r_first, r_last;
    cta_row_slice(p.total_rows, blockIdx.x, gridDim.x, r_first, r_last);
    const uint32_t n_mine = r_last - r_first;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kTeamWarps);
        }
        *abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kGemvWarps) {
        // ---------------- producer warp ----------------
        uint32_t unit = 0;
        bool ok = true;
        bool announce = p.gather.world != 0 && blockIdx.x == 0;   // see gemv_q8_0_kernel
        KqWalk walk(r_first, r_last);
        const int my_row = lane / F::kPlanes, my_plane = lane % F::kPlanes;  // one copy per (row, plane) of a unit
        bool contiguous = p.nseg == 1 && p.K == static_cast<uint32_t>(kKqSegElems);
#pragma unroll
        for (int pl = 0; pl < F::kPlanes; ++pl) contiguous = contiguous && p.pitch[pl] == F::seg_bytes(pl);
        while (!walk.done() && ok) {
            RowGroup pair[kTeams];
#pragma unroll
            for (int m = 0; m < kTeams; ++m) pair[m] = walk.next(p);
            for (uint32_t s = 0; s < p.nseg && ok; ++s) {
#pragma unroll
                for (int m = 0; m < kTeams; ++m, ++unit) {
                    const uint32_t stage = unit % kStages;
                    if (unit >= static_cast<uint32_t>(kStages) && announce) {
                        announce = false;
                        if (lane == 0) { pdl_wait(); gather_publish_pending(p.gather); }
                        __syncwarp();
                    }
                    if (unit >= static_cast<uint32_t>(kStages)) {
                        if (!mbar_wait(&empty[stage], ((unit / kStages) - 1) & 1)) {
                            if (lane == 0) { *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); }
                            ok = false;
                        }
                    }
                    if (*abort_word) ok = false;
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const RowGroup g = pair[m];
                    if (g.nrows == 0) {
                        if (lane == 0) mbar_arrive(&full[stage]);
                        continue;
                    }
                    const KqTask& t = p.task[g.task];
                    const uint32_t elems = min(static_cast<uint32_t>(kKqSegElems), p.K - s * kKqSegElems);  // multiple of the block size
                    uint32_t row_bytes = 0;
#pragma unroll
                    for (int pl = 0; pl < F::kPlanes; ++pl) row_bytes += (elems / 256 * F::bytes_per_256(pl) + (elems % 256) * F::bytes_per_256(pl) / 256 + 15) & ~15u;
                    const bool tiled = !contiguous && p.tile_maps[g.task] != nullptr;
                    // A tiled copy always delivers whole segments (columns past the row arrive as zeros).  A tile must land on a
                    // 128-byte boundary, so planes whose segment is narrower than that always arrive as ONE box of eight rows
                    // (the rows past a partial group are a few bytes that nobody reads; past the tensor they are zeros).
                    uint32_t tiled_bytes = 0;
#pragma unroll
                    for (int pl = 0; pl < F::kPlanes; ++pl) tiled_bytes += (F::seg_bytes(pl) < 128 ? static_cast<uint32_t>(kTeamWarps) : g.nrows) * F::seg_bytes(pl);
                    if (lane == 0) mbar_arrive_expect_tx(&full[stage], tiled ? tiled_bytes : g.nrows * row_bytes);
                    __syncwarp();
                    if (contiguous) {
                        // rows of one full segment follow each other in every plane: one copy per plane for the whole group
                        if (lane < F::kPlanes) {
                            bulk_g2s(ring + stage * kStageBytes + kq_plane_offset<kFormat>(lane),
                                     t.plane[lane] + static_cast<size_t>(g.row0) * p.pitch[lane], g.nrows * F::seg_bytes(lane), &full[stage]);
                        }
                    } else if (tiled) {
                        // tiled copies: per plane one for a whole row group, or boxes of 4, 2 and 1 rows for a partial one
                        if (lane == 0) {
                            const KqTileMaps* maps = p.tile_maps[g.task];
#pragma unroll
                            for (int pl = 0; pl < F::kPlanes; ++pl) {
                                uint32_t done_rows = 0;
                                const uint32_t want = F::seg_bytes(pl) < 128 ? static_cast<uint32_t>(kTeamWarps) : g.nrows;
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    const uint32_t box = 8u >> k;
                                    if (want - done_rows >= box) {
                                        uint8_t* dst = ring + stage * kStageBytes + kq_plane_offset<kFormat>(pl) + done_rows * F::seg_bytes(pl);
                                        if (F::seg_bytes(pl) <= 256)
                                            tma_load_2d(dst, &maps->map[pl][k], static_cast<int>(s * F::seg_bytes(pl)), static_cast<int>(g.row0 + done_rows), &full[stage]);
                                        else
                                            tma_load_3d(dst, &maps->map[pl][k], 0, static_cast<int>(s * (F::seg_bytes(pl) / 256)), static_cast<int>(g.row0 + done_rows), &full[stage]);
                                        done_rows += box;
                                    }
                                }
                            }
                        }
                    } else if (my_row < static_cast<int>(g.nrows) && my_row < kTeamWarps) {
                        const uint32_t per256 = F::bytes_per_256(my_plane);
                        const uint32_t bytes = (elems / 256 * per256 + (elems % 256) * per256 / 256 + 15) & ~15u;
                        const uint32_t seg_off = static_cast<uint32_t>(static_cast<uint64_t>(s) * kKqSegElems / 256 * per256);
                        uint8_t* dst = ring + stage * kStageBytes + kq_plane_offset<kFormat>(my_plane) + my_row * F::seg_bytes(my_plane);
                        bulk_g2s(dst, t.plane[my_plane] + static_cast<size_t>(g.row0 + my_row) * p.pitch[my_plane] + seg_off, bytes, &full[stage]);
                    }
                }
            }
        }
        if (announce && lane == 0) { pdl_wait(); gather_publish_pending(p.gather); }
        if (lane == 0) {
            const uint32_t armed = unit < static_cast<uint32_t>(kStages) ? unit : kStages;
            for (uint32_t k = 0; k < armed; ++k) {
                const uint32_t u = unit - 1 - k;
                if (!mbar_wait(&full[u % kStages], (u / kStages) & 1)) atomicExch(p.error_word, kErrDrainTimeout);
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    pdl_wait();
    // Row-sharded launch (peer_gather.cuh): wait for every rank's previous launch; a null x means "what it gathered".
    unsigned long long epoch = 0;
    const float* x_src = p.x;
    if (p.gather.world) {
        epoch = gather_epoch(p.gather);
        if (!x_src) {   // chained: the other ranks' previous outputs are this launch's input, so they are needed now
            if (!gather_wait(p.gather, lane, epoch)) {
                if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrPeerWaitTimeout); }
            }
            x_src = gather_previous(p.gather, epoch);
        }
    }
    // Prologue: two-digit quantisation of the activations, natural element order.
    {
        const uint32_t quad = static_cast<uint32_t>(lane) >> 2, part = static_cast<uint32_t>(lane) & 3;
        const uint32_t nblk = p.K / 32;
        for (int t = 0; t < kBatch; ++t) {
            for (uint32_t b0 = warp * 8; b0 < nblk; b0 += kGemvWarps * 8) {
                const uint32_t b = b0 + quad;
                const bool live = b < nblk;
                const float4* src = reinterpret_cast<const float4*>(x_src + static_cast<size_t>(t) * p.K + b * 32 + part * 8);
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 lo = live ? __ldcg(src) : zero, hi = live ? __ldcg(src + 1) : zero;  // L2: coherent with peers' stores
                const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                uint2 c1, c2;
                const float d = quantise_block_quad(v, c1, c2);
                // sum of the eight two-digit codes of this lane, then of the block's four lanes
                int sum = dp4a_ss(c1.x, 0x01010101u, 0) + dp4a_ss(c1.y, 0x01010101u, 0);
                sum = sum * 256 + dp4a_ss(c2.x, 0x01010101u, 0) + dp4a_ss(c2.y, 0x01010101u, 0);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (!live) continue;
                uint8_t* base = xd + static_cast<size_t>(t) * 2 * kpad + b * 32 + part * 8;
                *reinterpret_cast<uint2*>(base) = c1;
                *reinterpret_cast<uint2*>(base + kpad) = c2;
                if (part == 0) {
                    xscale[static_cast<size_t>(t) * (kpad / 32) + b] = d * (1.0f / 256.0f);
                    xsum[static_cast<size_t>(t) * (kpad / 32) + b] = sum;
                }
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");

    const int team = warp / kTeamWarps, twarp = warp % kTeamWarps;
    bool ok = *abort_word == 0;
    if constexpr (kBatch == 1) {
        // ---- batch 1: a warp owns a slice of K and walks every row of the unit with its activations in registers ----
        // Shared memory is then read for weights only (reading two activation digits per weight from it costs several
        // times the weight bytes in wavefronts and capped the kernel at a third of the HBM rate).
        //   Q4_0: warp = (K slice of 32 blocks, half of the eight rows); a lane owns one 32-weight block
        //   Q6_K: warp = K slice of two super-blocks, all eight rows;     a lane owns one 16-weight scale group
        //   Q4_K / Q5_K: warp = (K slice of four super-blocks, half of the eight rows); a lane owns 16 nibble bytes, i.e. 16
        //         weights of sub-block 2j (low nibbles) and the 16 of sub-block 2j+1 at the same positions (high nibbles)
        constexpr bool kK45 = kq_is_k45<kFormat>;
        constexpr bool kCodes = kFormat == kFormatQ6KCodes;   // a lane owns the 16 weights of group (lane & 15) of its super-block, in element order
        constexpr int kR = (kFormat == 2 || kK45) ? 4 : 8;             // rows per warp
        constexpr int kSlices = (kFormat == 2 || kK45) ? 4 : 8;        // K slices per segment
        const uint32_t kslice = static_cast<uint32_t>(twarp) % kSlices;
        const uint32_t rowbase = kR == 4 ? (static_cast<uint32_t>(twarp) / kSlices) * kR : 0u;
        // Q4_K / Q5_K lane geometry (src/quant.cpp:133-141 and the kernels at kernels/avx2.cpp:329-378): element
        // g*32 + l of a super-block is the nibble (g & 1) of byte (g >> 1)*32 + l, its fifth bit is bit g of qh[l]
        const uint32_t k_sb = kslice * 4 + (static_cast<uint32_t>(lane) >> 3), k_j = (static_cast<uint32_t>(lane) >> 1) & 3, k_h = lane & 1;
        float k_xs_hi = 0.0f, k_f_lo = 0.0f, k_f_hi = 0.0f;   // the high sub-block's activation scale; scale x code sum of both
        // Q6_K lane geometry (src/quant.cpp:500-517): element e = half*128 + group*32 + l lives in ql byte
        // half*64 + (group%2)*32 + l (low nibble for group < 2), qh byte half*32 + l bits 2*group.., scale half*8 + group*2 + l/16
        const uint32_t sg = lane & 15, qhalf = sg >> 3, group = (sg >> 1) & 3, six = sg & 1;
        const uint32_t shift4 = group >= 2 ? 4u : 0u, shift2 = group * 2;
        const uint32_t sbl = kslice * 2 + (static_cast<uint32_t>(lane) >> 4);   // super-block within the segment

        uint4 xa = make_uint4(0, 0, 0, 0), xb = xa, xc = xa, xd4 = xa;   // Q4_0: digit 1 lo/hi halves, digit 2 lo/hi; Q6_K: digit 1, digit 2
        float xs = 0.0f;     // activation scale of the lane's block, with the digit weight folded in
        int bias = 0;        // minus (zero point x sum of the lane's activation codes), the dp4a chain's starting value
        // A lane whose block lies past the end of the row reads the segment's first block instead (valid bytes, so a
        // finite scale) with zero activations and a zero scale: its terms are exactly zero and need no select.
        uint32_t wofs = 0;   // byte offset of the lane's weights within a row of plane 0 (Q4_0) / super-block index (Q6_K)
        auto load_x = [&](uint32_t seg) {
            const uint4 zero = make_uint4(0, 0, 0, 0);
            if (kFormat == 2) {
                const uint32_t b = seg * (kKqSegElems / 32) + kslice * 32 + lane;
                const bool live = b * 32 < p.K;
                const uint4* x1 = reinterpret_cast<const uint4*>(xd + b * 32);
                const uint4* x2 = reinterpret_cast<const uint4*>(xd + kpad + b * 32);
                xa = live ? x1[0] : zero; xb = live ? x1[1] : zero; xc = live ? x2[0] : zero; xd4 = live ? x2[1] : zero;
                xs = live ? xscale[b] * (1.0f / 16.0f) : 0.0f;   // high nibbles enter sixteen-fold, so every sum is sixteen-fold
                bias = live ? -128 * xsum[b] : 0;                 // -8 * sum, sixteen-fold
                wofs = live ? kslice * 32 + lane : 0u;
            } else if (kK45) {
                const uint32_t e_lo = seg * kKqSegElems + k_sb * 256 + k_j * 64 + k_h * 16, e_hi = e_lo + 32;
                const bool live = e_lo < p.K;   // K is a multiple of 256: the lane's two sub-blocks are both inside or both outside
                xa = live ? *reinterpret_cast<const uint4*>(xd + e_lo) : zero;
                xb = live ? *reinterpret_cast<const uint4*>(xd + e_hi) : zero;
                xc = live ? *reinterpret_cast<const uint4*>(xd + kpad + e_lo) : zero;
                xd4 = live ? *reinterpret_cast<const uint4*>(xd + kpad + e_hi) : zero;
                xs = live ? xscale[e_lo / 32] : 0.0f;
                k_xs_hi = live ? xscale[e_hi / 32] : 0.0f;
                const uint4 ones = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
                k_f_lo = xs * static_cast<float>(dot16(ones, xa) * 256 + dot16(ones, xc));        // for the minimum term
                k_f_hi = k_xs_hi * static_cast<float>(dot16(ones, xb) * 256 + dot16(ones, xd4));
                wofs = live ? k_sb : 0u;
            } else if (kCodes) {
                const uint32_t e0 = seg * kKqSegElems + sbl * 256 + sg * 16;
                const bool live = e0 < p.K;
                xa = live ? *reinterpret_cast<const uint4*>(xd + e0) : zero;
                xc = live ? *reinterpret_cast<const uint4*>(xd + kpad + e0) : zero;
                xs = live ? xscale[e0 / 32] : 0.0f;
                wofs = live ? sbl : 0u;
            } else {
                const uint32_t e0 = seg * kKqSegElems + sbl * 256 + qhalf * 128 + group * 32 + six * 16;
                const bool live = e0 < p.K;
                xa = live ? *reinterpret_cast<const uint4*>(xd + e0) : zero;
                xc = live ? *reinterpret_cast<const uint4*>(xd + kpad + e0) : zero;
                xs = live ? xscale[e0 / 32] : 0.0f;
                const uint4 ones = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
                bias = -32 * (dot16(ones, xa) * 256 + dot16(ones, xc));
                wofs = live ? sbl : 0u;
            }
        };
        if (p.nseg == 1) load_x(0);

        uint32_t pair_index = 0;
        KqWalk walk(r_first, r_last);
        while (!walk.done()) {
            RowGroup pair[kTeams];
#pragma unroll
            for (int m = 0; m < kTeams; ++m) pair[m] = walk.next(p);
            RowGroup g = pair[0];
            if constexpr (kTeams > 1) { if (team == 1) g = pair[kTeams - 1]; }
            const KqTask& t = p.task[g.task];
            float acc[kR];
#pragma unroll
            for (int r = 0; r < kR; ++r) acc[r] = 0.0f;
            bool failed = false;
            for (uint32_t s = 0; s < p.nseg; ++s) {
                const uint32_t unit = (pair_index * p.nseg + s) * kTeams + team;
                const uint32_t stage = unit % kStages;
                if (*abort_word || !mbar_wait(&full[stage], (unit / kStages) & 1)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                    failed = true;
                    break;
                }
                if (p.nseg > 1) load_x(s);
                const uint8_t* st = ring + stage * kStageBytes;
                const uint8_t* w0;   // the lane's weights in row 0 of the stage
                const uint8_t* w1;
                const int8_t* sc = nullptr;
                const __half* dd = nullptr;
                if (kFormat == 2) {
                    w0 = st + kq_plane_offset<kFormat>(0) + rowbase * F::seg_bytes(0) + wofs * 16;   // nibbles
                    w1 = st + kq_plane_offset<kFormat>(1) + rowbase * F::seg_bytes(1) + wofs * 2;    // scale
                } else if (kK45) {
                    constexpr int kScm = F::kPlanes - 2, kDd = F::kPlanes - 1;
                    w0 = st + kq_plane_offset<kFormat>(0) + rowbase * F::seg_bytes(0) + wofs * 128 + k_j * 32 + k_h * 16;   // nibbles
                    w1 = st + kq_plane_offset<kFormat>(1) + rowbase * F::seg_bytes(1) + wofs * 32 + k_h * 16;             // Q5_K: fifth bits
                    sc = reinterpret_cast<const int8_t*>(st + kq_plane_offset<kFormat>(kScm) + rowbase * F::seg_bytes(kScm)) + wofs * 16 + k_j * 2;
                    dd = reinterpret_cast<const __half*>(st + kq_plane_offset<kFormat>(kDd) + rowbase * F::seg_bytes(kDd)) + wofs * 2;
                } else if (kCodes) {
                    w0 = st + kq_plane_offset<kFormat>(0) + wofs * 256 + sg * 16;   // codes
                    w1 = w0;
                    sc = reinterpret_cast<const int8_t*>(st + kq_plane_offset<kFormat>(1)) + wofs * 16 + sg;
                    dd = reinterpret_cast<const __half*>(st + kq_plane_offset<kFormat>(2)) + wofs;
                } else {
                    w0 = st + kq_plane_offset<kFormat>(0) + wofs * 128 + qhalf * 64 + (group & 1) * 32 + six * 16;   // ql
                    w1 = st + kq_plane_offset<kFormat>(1) + wofs * 64 + qhalf * 32 + six * 16;                       // qh
                    sc = reinterpret_cast<const int8_t*>(st + kq_plane_offset<kFormat>(2)) + wofs * 16 + sg;
                    dd = reinterpret_cast<const __half*>(st + kq_plane_offset<kFormat>(3)) + wofs;
                }
                auto row_body = [&](int r) {
                    if (kFormat == 2) {
                        const uint4 w = *reinterpret_cast<const uint4*>(w0 + r * F::seg_bytes(0));
                        const float dw = __half2float(*reinterpret_cast<const __half*>(w1 + r * F::seg_bytes(1)));
                        // low nibbles are elements 0..15, high nibbles elements 16..31 (src/quant.cpp:391-397); the high
                        // nibbles stay in place (value x 16, an unsigned byte), which saves the shifts
                        const uint32_t m = 0x0F0F0F0Fu;
                        int a = dp4a_us(w.x & m, xa.x, 0), b = dp4a_us(w.x & ~m, xb.x, 0), c = dp4a_us(w.x & m, xc.x, 0), d = dp4a_us(w.x & ~m, xd4.x, bias);
                        a = dp4a_us(w.y & m, xa.y, a); b = dp4a_us(w.y & ~m, xb.y, b); c = dp4a_us(w.y & m, xc.y, c); d = dp4a_us(w.y & ~m, xd4.y, d);
                        a = dp4a_us(w.z & m, xa.z, a); b = dp4a_us(w.z & ~m, xb.z, b); c = dp4a_us(w.z & m, xc.z, c); d = dp4a_us(w.z & ~m, xd4.z, d);
                        a = dp4a_us(w.w & m, xa.w, a); b = dp4a_us(w.w & ~m, xb.w, b); c = dp4a_us(w.w & m, xc.w, c); d = dp4a_us(w.w & ~m, xd4.w, d);
                        // 16 * (256 * (lo.q1 + hi.q1) + (lo.q2 + hi.q2) - 8 * sum) = 4096 a + 256 b + 16 c + d
                        const int isum = ((a * 16 + b) * 16 + c) * 16 + d;
                        acc[r] = fmaf(dw * xs, static_cast<float>(isum), acc[r]);
                    } else if (kK45) {
                        constexpr int kScm = F::kPlanes - 2, kDd = F::kPlanes - 1;
                        const uint4 w = *reinterpret_cast<const uint4*>(w0 + r * F::seg_bytes(0));
                        const uint32_t m = 0x0F0F0F0Fu;
                        uint4 lo = make_uint4(w.x & m, w.y & m, w.z & m, w.w & m);
                        uint4 hi = make_uint4((w.x >> 4) & m, (w.y >> 4) & m, (w.z >> 4) & m, (w.w >> 4) & m);
                        if (kFormat == 13) {
                            const uint4 q5 = *reinterpret_cast<const uint4*>(w1 + r * F::seg_bytes(1));
                            const uint32_t s_lo = 2 * k_j, s_hi = 2 * k_j + 1, one = 0x01010101u;
                            lo.x |= ((q5.x >> s_lo) & one) << 4; lo.y |= ((q5.y >> s_lo) & one) << 4; lo.z |= ((q5.z >> s_lo) & one) << 4; lo.w |= ((q5.w >> s_lo) & one) << 4;
                            hi.x |= ((q5.x >> s_hi) & one) << 4; hi.y |= ((q5.y >> s_hi) & one) << 4; hi.z |= ((q5.z >> s_hi) & one) << 4; hi.w |= ((q5.w >> s_hi) & one) << 4;
                        }
                        const int i_lo = dot16(lo, xa) * 256 + dot16(lo, xc);     // codes are 0..31: signed and unsigned dp4a agree
                        const int i_hi = dot16(hi, xb) * 256 + dot16(hi, xd4);
                        const uint32_t sc2 = *reinterpret_cast<const uint16_t*>(sc + r * F::seg_bytes(kScm));        // scales of sub-blocks 2j, 2j+1
                        const uint32_t mn2 = *reinterpret_cast<const uint16_t*>(sc + r * F::seg_bytes(kScm) + 8);    // their minimums
                        const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(dd + r * (F::seg_bytes(kDd) / 2)));
                        const float pos = static_cast<float>(sc2 & 0xffu) * (xs * static_cast<float>(i_lo)) + static_cast<float>(sc2 >> 8) * (k_xs_hi * static_cast<float>(i_hi));
                        const float neg = static_cast<float>(mn2 & 0xffu) * k_f_lo + static_cast<float>(mn2 >> 8) * k_f_hi;
                        acc[r] = fmaf(dm.x, pos, fmaf(-dm.y, neg, acc[r]));
                    } else if (kCodes) {
                        const uint4 q = *reinterpret_cast<const uint4*>(w0 + r * F::seg_bytes(0));
                        const int a = dot16(q, xa), c = dot16(q, xc);
                        const float dsc = __half2float(dd[r * (F::seg_bytes(2) / 2)]) * static_cast<float>(sc[r * F::seg_bytes(1)]);  // (d * scale), the reference's order
                        acc[r] = fmaf(dsc * xs, static_cast<float>(a * 256 + c), acc[r]);
                    } else {
                        const uint4 l4 = *reinterpret_cast<const uint4*>(w0 + r * F::seg_bytes(0));
                        const uint4 h4 = *reinterpret_cast<const uint4*>(w1 + r * F::seg_bytes(1));
                        // codes stay 0..63; the zero point 32 is in `bias`
                        const uint32_t q0 = ((l4.x >> shift4) & 0x0F0F0F0Fu) | (((h4.x >> shift2) & 0x03030303u) << 4);
                        const uint32_t q1 = ((l4.y >> shift4) & 0x0F0F0F0Fu) | (((h4.y >> shift2) & 0x03030303u) << 4);
                        const uint32_t q2 = ((l4.z >> shift4) & 0x0F0F0F0Fu) | (((h4.z >> shift2) & 0x03030303u) << 4);
                        const uint32_t q3 = ((l4.w >> shift4) & 0x0F0F0F0Fu) | (((h4.w >> shift2) & 0x03030303u) << 4);
                        int a = dp4a_us(q0, xa.x, 0), c = dp4a_us(q0, xc.x, bias);
                        a = dp4a_us(q1, xa.y, a); c = dp4a_us(q1, xc.y, c);
                        a = dp4a_us(q2, xa.z, a); c = dp4a_us(q2, xc.z, c);
                        a = dp4a_us(q3, xa.w, a); c = dp4a_us(q3, xc.w, c);
                        const float dsc = __half2float(dd[r * (F::seg_bytes(3) / 2)]) * static_cast<float>(sc[r * F::seg_bytes(2)]);  // (d * scale), the reference's order
                        acc[r] = fmaf(dsc * xs, static_cast<float>(a * 256 + c), acc[r]);
                    }
                };
                if (g.nrows == static_cast<uint32_t>(kTeamWarps)) {   // the common case: no per-row test
#pragma unroll
                    for (int r = 0; r < kR; ++r) row_body(r);
                } else {
#pragma unroll
                    for (int r = 0; r < kR; ++r)
                        if (rowbase + r < g.nrows) row_body(r);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stage]);
            }
            // rows of the unit: sum over the warp's lanes, then over the K slices through shared memory
            uint32_t prow;
            const float psum = kq_reduce_rows<kR>(acc, lane, prow);
            float* part = partial + (team * 2 + (pair_index & 1)) * (kTeamWarps * kTeamWarps);
            if ((lane & (kR == 8 ? 3 : 7)) == 0) part[kslice * kTeamWarps + rowbase + prow] = psum;
            if (team_barrier_any(team, failed)) { ok = false; break; }
            if (twarp == 0 && static_cast<uint32_t>(lane) < g.nrows) {
                float v = part[lane];
#pragma unroll
                for (int k = 1; k < kSlices; ++k) v += part[k * kTeamWarps + lane];
                const uint32_t row = g.row0 + lane;
                if (t.y) t.y[row] = v;
                if (p.gather.world) stash[t.first_row + row - r_first] = v;
            }
            ++pair_index;
        }
    } else {
        uint32_t pair_base = 0;
        KqWalk walk(r_first, r_last);
        while (!walk.done() && ok) {
            RowGroup pair[kTeams];
    #pragma unroll
            for (int m = 0; m < kTeams; ++m) pair[m] = walk.next(p);
            RowGroup g = pair[0];
            if constexpr (kTeams > 1) { if (team == 1) g = pair[kTeams - 1]; }
            const KqTask& t = p.task[g.task];
            const uint32_t row = g.row0 + twarp;
            const bool valid = static_cast<uint32_t>(twarp) < g.nrows;
            float acc[kBatch];
    #pragma unroll
            for (int b = 0; b < kBatch; ++b) acc[b] = 0.0f;

            for (uint32_t s = 0; s < p.nseg; ++s) {
                const uint32_t unit = pair_base + s * kTeams + team;
                const uint32_t stage = unit % kStages;
                if (*abort_word || !mbar_wait(&full[stage], (unit / kStages) & 1)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                    ok = false;
                    break;
                }
                if (valid) {
                    const uint8_t* st = ring + stage * kStageBytes;
                    const uint32_t e_base = s * kKqSegElems;
                    const uint32_t elems = min(static_cast<uint32_t>(kKqSegElems), p.K - e_base);
                    if (kFormat == 2) {
                        // ---- Q4_0: a lane owns a 32-weight block: 16 nibble bytes + one scale ----
                        const uint4* nib = reinterpret_cast<const uint4*>(st + kq_plane_offset<kFormat>(0) + twarp * F::seg_bytes(0));
                        const __half* ws = reinterpret_cast<const __half*>(st + kq_plane_offset<kFormat>(1) + twarp * F::seg_bytes(1));
    #pragma unroll
                        for (int i = 0; i < kKqSegElems / 32 / 32; ++i) {
                            const uint32_t bl = i * 32 + lane;
                            if (bl * 32 < elems) {
                                const uint4 w = nib[bl];
                                const float dw = __half2float(ws[bl]);
                                // low nibbles are elements 0..15, high nibbles elements 16..31 (src/quant.cpp:391-397)
                                const uint4 lo = make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu);
                                const uint4 hi = make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
                                const uint32_t b = e_base / 32 + bl;
    #pragma unroll
                                for (int tk = 0; tk < kBatch; ++tk) {
                                    const uint4* x1 = reinterpret_cast<const uint4*>(xd + static_cast<size_t>(tk) * 2 * kpad + b * 32);
                                    const uint4* x2 = reinterpret_cast<const uint4*>(xd + static_cast<size_t>(tk) * 2 * kpad + kpad + b * 32);
                                    const int i1 = dot16(lo, x1[0]) + dot16(hi, x1[1]);
                                    const int i2 = dot16(lo, x2[0]) + dot16(hi, x2[1]);
                                    const int isum = i1 * 256 + i2 - 8 * xsum[static_cast<size_t>(tk) * (kpad / 32) + b];
                                    acc[tk] = fmaf(dw * xscale[static_cast<size_t>(tk) * (kpad / 32) + b], static_cast<float>(isum), acc[tk]);
                                }
                            }
                        }
                    } else if (kq_is_k45<kFormat>) {
                        // ---- Q4_K / Q5_K: a lane owns 16 nibble bytes (16 weights of sub-block 2j and 16 of 2j+1); a warp covers four super-blocks a pass ----
                        constexpr int kScm = F::kPlanes - 2, kDd = F::kPlanes - 1;
                        const uint8_t* qs = st + kq_plane_offset<kFormat>(0) + twarp * F::seg_bytes(0);
                        const uint8_t* q5p = st + kq_plane_offset<kFormat>(1) + twarp * F::seg_bytes(1);
                        const uint8_t* scm = st + kq_plane_offset<kFormat>(kScm) + twarp * F::seg_bytes(kScm);
                        const __half2* dd = reinterpret_cast<const __half2*>(st + kq_plane_offset<kFormat>(kDd) + twarp * F::seg_bytes(kDd));
                        const uint32_t j = (static_cast<uint32_t>(lane) >> 1) & 3, h = lane & 1;
    #pragma unroll
                        for (int i = 0; i < kKqSegElems / 256 / 4; ++i) {
                            const uint32_t sbl = i * 4 + (lane >> 3);
                            if (sbl * 256 < elems) {
                                const uint4 w = *reinterpret_cast<const uint4*>(qs + sbl * 128 + j * 32 + h * 16);
                                const uint32_t m = 0x0F0F0F0Fu;
                                uint4 lo = make_uint4(w.x & m, w.y & m, w.z & m, w.w & m);
                                uint4 hi = make_uint4((w.x >> 4) & m, (w.y >> 4) & m, (w.z >> 4) & m, (w.w >> 4) & m);
                                if (kFormat == 13) {
                                    const uint4 q5 = *reinterpret_cast<const uint4*>(q5p + sbl * 32 + h * 16);
                                    const uint32_t s_lo = 2 * j, s_hi = 2 * j + 1, one = 0x01010101u;
                                    lo.x |= ((q5.x >> s_lo) & one) << 4; lo.y |= ((q5.y >> s_lo) & one) << 4; lo.z |= ((q5.z >> s_lo) & one) << 4; lo.w |= ((q5.w >> s_lo) & one) << 4;
                                    hi.x |= ((q5.x >> s_hi) & one) << 4; hi.y |= ((q5.y >> s_hi) & one) << 4; hi.z |= ((q5.z >> s_hi) & one) << 4; hi.w |= ((q5.w >> s_hi) & one) << 4;
                                }
                                const uint32_t sc2 = *reinterpret_cast<const uint16_t*>(scm + sbl * 16 + j * 2);
                                const uint32_t mn2 = *reinterpret_cast<const uint16_t*>(scm + sbl * 16 + 8 + j * 2);
                                const float2 dm = __half22float2(dd[sbl]);
                                const float ds_lo = dm.x * static_cast<float>(sc2 & 0xffu), ds_hi = dm.x * static_cast<float>(sc2 >> 8);   // (d * scale), (dmin * m):
                                const float ms_lo = dm.y * static_cast<float>(mn2 & 0xffu), ms_hi = dm.y * static_cast<float>(mn2 >> 8);   // the reference's factors
                                const uint32_t e_lo = e_base + sbl * 256 + j * 64 + h * 16, e_hi = e_lo + 32;
                                const uint4 ones = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    #pragma unroll
                                for (int tk = 0; tk < kBatch; ++tk) {
                                    const uint8_t* xt = xd + static_cast<size_t>(tk) * 2 * kpad;
                                    const uint4 a1 = *reinterpret_cast<const uint4*>(xt + e_lo), b1 = *reinterpret_cast<const uint4*>(xt + e_hi);
                                    const uint4 a2 = *reinterpret_cast<const uint4*>(xt + kpad + e_lo), b2 = *reinterpret_cast<const uint4*>(xt + kpad + e_hi);
                                    const float xs_lo = xscale[static_cast<size_t>(tk) * (kpad / 32) + e_lo / 32], xs_hi = xscale[static_cast<size_t>(tk) * (kpad / 32) + e_hi / 32];
                                    const int i_lo = dot16(lo, a1) * 256 + dot16(lo, a2), i_hi = dot16(hi, b1) * 256 + dot16(hi, b2);
                                    const int s_lo = dot16(ones, a1) * 256 + dot16(ones, a2), s_hi = dot16(ones, b1) * 256 + dot16(ones, b2);
                                    float v = acc[tk];
                                    v = fmaf(ds_lo * xs_lo, static_cast<float>(i_lo), v);
                                    v = fmaf(ds_hi * xs_hi, static_cast<float>(i_hi), v);
                                    v = fmaf(-ms_lo * xs_lo, static_cast<float>(s_lo), v);
                                    v = fmaf(-ms_hi * xs_hi, static_cast<float>(s_hi), v);
                                    acc[tk] = v;
                                }
                            }
                        }
                    } else if (kFormat == kFormatQ6KCodes) {
                        // ---- Q6_K, unpacked codes: a lane owns one 16-weight group in element order; two super-blocks a pass ----
                        const uint8_t* qc = st + kq_plane_offset<kFormat>(0) + twarp * F::seg_bytes(0);
                        const int8_t* sc = reinterpret_cast<const int8_t*>(st + kq_plane_offset<kFormat>(1) + twarp * F::seg_bytes(1));
                        const __half* dd = reinterpret_cast<const __half*>(st + kq_plane_offset<kFormat>(2) + twarp * F::seg_bytes(2));
                        const uint32_t sg = lane & 15;
    #pragma unroll 4
                        for (int i = 0; i < kKqSegElems / 256 / 2; ++i) {
                            const uint32_t sbl = i * 2 + (lane >> 4);
                            if (sbl * 256 < elems) {
                                const uint4 q = *reinterpret_cast<const uint4*>(qc + sbl * 256 + sg * 16);
                                const float dsc = __half2float(dd[sbl]) * static_cast<float>(sc[sbl * 16 + sg]);
                                const uint32_t e0 = e_base + sbl * 256 + sg * 16;
    #pragma unroll
                                for (int tk = 0; tk < kBatch; ++tk) {
                                    const uint4 x1 = *reinterpret_cast<const uint4*>(xd + static_cast<size_t>(tk) * 2 * kpad + e0);
                                    const uint4 x2 = *reinterpret_cast<const uint4*>(xd + static_cast<size_t>(tk) * 2 * kpad + kpad + e0);
                                    const int isum = dot16(q, x1) * 256 + dot16(q, x2);
                                    acc[tk] = fmaf(dsc * xscale[static_cast<size_t>(tk) * (kpad / 32) + e0 / 32], static_cast<float>(isum), acc[tk]);
                                }
                            }
                        }
                    } else {
                        // ---- Q6_K: a lane owns one 16-weight scale group; a warp covers two super-blocks a pass ----
                        const uint8_t* ql = st + kq_plane_offset<kFormat>(0) + twarp * F::seg_bytes(0);
                        const uint8_t* qh = st + kq_plane_offset<kFormat>(1) + twarp * F::seg_bytes(1);
                        const int8_t* sc = reinterpret_cast<const int8_t*>(st + kq_plane_offset<kFormat>(2) + twarp * F::seg_bytes(2));
                        const __half* dd = reinterpret_cast<const __half*>(st + kq_plane_offset<kFormat>(3) + twarp * F::seg_bytes(3));
                        const uint32_t sg = lane & 15, half = sg >> 3, group = (sg >> 1) & 3, six = sg & 1;
                        const uint32_t shift4 = group >= 2 ? 4u : 0u, shift2 = group * 2;
                        // element e = half*128 + group*32 + l: ql byte half*64 + (group%2)*32 + l, qh byte half*32 + l,
                        // scale half*8 + group*2 + l/16 == sg (src/quant.cpp:500-517)
    #pragma unroll 4
                        for (int i = 0; i < kKqSegElems / 256 / 2; ++i) {
                            const uint32_t sbl = i * 2 + (lane >> 4);
                            if (sbl * 256 < elems) {
                                const uint4 l4 = *reinterpret_cast<const uint4*>(ql + sbl * 128 + half * 64 + (group & 1) * 32 + six * 16);
                                const uint4 h4 = *reinterpret_cast<const uint4*>(qh + sbl * 64 + half * 32 + six * 16);
                                uint4 q;
                                q.x = sub32_bytes(((l4.x >> shift4) & 0x0F0F0F0Fu) | (((h4.x >> shift2) & 0x03030303u) << 4));
                                q.y = sub32_bytes(((l4.y >> shift4) & 0x0F0F0F0Fu) | (((h4.y >> shift2) & 0x03030303u) << 4));
                                q.z = sub32_bytes(((l4.z >> shift4) & 0x0F0F0F0Fu) | (((h4.z >> shift2) & 0x03030303u) << 4));
                                q.w = sub32_bytes(((l4.w >> shift4) & 0x0F0F0F0Fu) | (((h4.w >> shift2) & 0x03030303u) << 4));
                                const float dsc = __half2float(dd[sbl]) * static_cast<float>(sc[sbl * 16 + sg]);  // (d * scale), the reference's order
                                const uint32_t e0 = e_base + sbl * 256 + half * 128 + group * 32 + six * 16;
    #pragma unroll
                                for (int tk = 0; tk < kBatch; ++tk) {
                                    const uint4 x1 = *reinterpret_cast<const uint4*>(xd + static_cast<size_t>(tk) * 2 * kpad + e0);
                                    const uint4 x2 = *reinterpret_cast<const uint4*>(xd + static_cast<size_t>(tk) * 2 * kpad + kpad + e0);
                                    const int isum = dot16(q, x1) * 256 + dot16(q, x2);
                                    acc[tk] = fmaf(dsc * xscale[static_cast<size_t>(tk) * (kpad / 32) + e0 / 32], static_cast<float>(isum), acc[tk]);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stage]);
            }
            if (!ok) break;
            pair_base += kTeams * p.nseg;
            if (valid) {
    #pragma unroll
                for (int tk = 0; tk < kBatch; ++tk) {
                    float v = acc[tk];
    #pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0 && t.y) t.y[static_cast<size_t>(tk) * t.rows + row] = v;
                    if (lane == 0 && p.gather.world) stash[static_cast<size_t>(tk) * n_mine + (t.first_row + row - r_first)] = v;
                }
            }
        }
    }
    if (p.gather.world) {
        asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");
        // With an input of its own the launch needs the other ranks only now: they must have finished the previous
        // launch (whose reads used the parity about to be overwritten) before anything is stored into their regions.
        bool may_push = true;
        if (p.x && !gather_wait(p.gather, lane, epoch)) {
            if (lane == 0) atomicExch(p.error_word, kErrPeerWaitTimeout);
            may_push = false;
        }
        if (may_push) gather_push(p.gather, epoch, stash, n_mine, r_first, p.total_rows, kBatch, warp, kGemvWarps, lane);
        asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");
        if (threadIdx.x == 0) gather_finish(p.gather, epoch);
    }
}

}  // namespace zk
