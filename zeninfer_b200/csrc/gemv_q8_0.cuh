// Decode-time Q8_0 matrix-vector product (batch 1..8), memory-bound by design.
//
// Replaces, on the device, what the reference does per projection in
// zen::quant::gemv / gemv_batch (src/quant.cpp:963-1163, :1441-1502) over
// gemv_q8_0_avx2_int8_prequant (kernels/avx2.cpp:562-585) when activations are
// int8 (kDigits == 1), and over gemv_q8_0_avx2 (kernels/avx2.cpp:587-641) when
// they are fp32 (kDigits == 2, two int8 digits per activation).
//
// Shape of the kernel
//   * one persistent CTA per SM owns a contiguous, byte-balanced slice of the
//     launch's rows (slice i of n covers [rows*i/n, rows*(i+1)/n), the same cut the
//     reference's ComputePool::parallel_for makes, src/compute_pool.cpp:104-106) and
//     walks it in groups of kGemvWarps rows; every consumer warp owns one row of
//     the group and keeps that row's accumulators in registers until the row is
//     finished, so no partial sums ever cross warps and the result is deterministic;
//   * one producer warp streams the group's rows through a ring of shared-memory
//     stages with 1-D TMA bulk copies (cp.async.bulk), one K-segment of
//     kGemvSegBlocks blocks at a time, each stage guarded by a full/empty
//     mbarrier pair.  Bytes in flight are set by the ring depth, not by
//     registers or occupancy;
//   * the activation vector is quantised once per CTA in the prologue (while the
//     first weight stages are already in flight) into a lane-major layout, so
//     every shared-memory read in the inner loop is a conflict-free 128-bit load;
//   * launched with programmatic stream serialisation: the weight stream of launch
//     n+1 starts while launch n drains (weights are constants), and only the
//     activation read waits for the previous grid (griddepcontrol.wait);
//   * per 32-element block: 8 dp4a per digit, one int->float conversion and one
//     fused multiply-add with the fp16 block scale times the activation scale.
//
// Algorithmic traffic is the raw GGUF size: 34 bytes per block.
#pragma once
#include <cuda_fp16.h>

#include "quantize_acts.cuh"
#include "zk_ptx.cuh"

namespace zk {

constexpr int kGemvWarps = 8;        // consumer warps == rows per row group
constexpr int kGemvSegBlocks = 64;   // 32-element blocks per K segment
constexpr int kGemvStages = 6;
constexpr int kGemvThreads = (kGemvWarps + 1) * 32;
constexpr int kMaxTasks = 8;         // projections sharing one input (zen::hip::kMaxBatch, include/zen/hip_backend.h:70)

constexpr uint32_t kQ8StageCodeBytes = kGemvWarps * kGemvSegBlocks * 32;
constexpr uint32_t kQ8StageScaleBytes = kGemvWarps * kGemvSegBlocks * 2;
constexpr uint32_t kQ8StageBytes = kQ8StageCodeBytes + kQ8StageScaleBytes;

struct GemvTask {
    const uint8_t* codes;    // [rows][K] int8
    const __half* scales;    // [rows][nbp]
    float* y;                // [batch][rows], token-major
    uint32_t rows;
    uint32_t first_row;      // index of this task's first row in the launch's concatenated row space
};

struct GemvParams {
    GemvTask task[kMaxTasks];
    uint32_t ntasks;
    uint32_t total_rows;     // over all tasks
    const float* x;          // [batch][K] fp32
    uint32_t K, nb, nbp, nseg;
    int* error_word;         // set to a zk::kErr* code when a bounded wait gives up
};

__host__ __device__ inline size_t gemv_q8_0_smem_bytes(uint32_t nseg, int batch, int digits) {
    const size_t kpad_blocks = static_cast<size_t>(nseg) * kGemvSegBlocks;
    return static_cast<size_t>(kGemvStages) * kQ8StageBytes        // weight ring
           + static_cast<size_t>(batch) * digits * kpad_blocks * 32  // activation codes
           + static_cast<size_t>(batch) * kpad_blocks * 4            // activation scales
           + 2 * kGemvStages * 8 + 16;                               // barriers + abort word
}

// The slice of the launch's concatenated row space that CTA `cta` of `n` owns.
__device__ __forceinline__ void cta_row_slice(uint32_t total_rows, uint32_t cta, uint32_t n, uint32_t& first, uint32_t& last) {
    first = static_cast<uint32_t>(static_cast<uint64_t>(total_rows) * cta / n);
    last = static_cast<uint32_t>(static_cast<uint64_t>(total_rows) * (cta + 1) / n);
}

// Walks a row slice in groups of at most kGemvWarps rows that never straddle two tasks.
struct GroupWalk {
    uint32_t r, r_end, ti;
    __device__ GroupWalk(uint32_t first, uint32_t last) : r(first), r_end(last), ti(0) {}
    __device__ bool done() const { return r >= r_end; }
    // Returns the task index and fills the group's first row within that task and its row count.
    __device__ uint32_t next(const GemvParams& p, uint32_t& row0, uint32_t& nrows) {
        while (r >= p.task[ti].first_row + p.task[ti].rows) ++ti;
        row0 = r - p.task[ti].first_row;
        nrows = min(min(static_cast<uint32_t>(kGemvWarps), p.task[ti].rows - row0), r_end - r);
        r += nrows;
        return ti;
    }
};

template <int kBatch, int kDigits>
__global__ void __launch_bounds__(kGemvThreads, (kBatch * kDigits <= 4 ? 2 : 1))
    gemv_q8_0_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t kpad_blocks = p.nseg * kGemvSegBlocks;
    uint8_t* ring = smem;
    uint4* xcodes = reinterpret_cast<uint4*>(ring + kGemvStages * kQ8StageBytes);           // [batch][digit][kpad_blocks*2]
    float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xcodes) + static_cast<size_t>(kBatch) * kDigits * kpad_blocks * 32);
    uint64_t* full = reinterpret_cast<uint64_t*>(xscale + static_cast<size_t>(kBatch) * kpad_blocks);
    uint64_t* empty = full + kGemvStages;
    volatile int* abort_word = reinterpret_cast<volatile int*>(empty + kGemvStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t r_first, r_last;
    cta_row_slice(p.total_rows, blockIdx.x, gridDim.x, r_first, r_last);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGemvWarps);
        }
        *abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Let the next launch in the stream begin: its weight stream may overlap this grid's tail.
    pdl_launch_dependents();

    if (warp == kGemvWarps) {
        // ---------------- producer warp: weights are constants, no need to wait for the previous grid ----------------
        uint32_t unit = 0;
        bool ok = true;
        GroupWalk walk(r_first, r_last);
        while (!walk.done() && ok) {
            uint32_t row0, nrows;
            const GemvTask& t = p.task[walk.next(p, row0, nrows)];
            for (uint32_t s = 0; s < p.nseg && ok; ++s, ++unit) {
                const uint32_t stage = unit % kGemvStages;
                if (unit >= kGemvStages) {
                    if (!mbar_wait(&empty[stage], ((unit / kGemvStages) - 1) & 1)) {
                        if (lane == 0) { *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); }
                        ok = false;
                    }
                }
                if (*abort_word) ok = false;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t nblk = min(static_cast<uint32_t>(kGemvSegBlocks), p.nb - s * kGemvSegBlocks);
                const uint32_t cbytes = nblk * 32, sbytes = (nblk * 2 + 15) & ~15u;
                uint8_t* st = ring + stage * kQ8StageBytes;
                if (lane == 0) mbar_arrive_expect_tx(&full[stage], nrows * (cbytes + sbytes));
                __syncwarp();
                if (lane < static_cast<int>(nrows)) {
                    bulk_g2s(st + lane * (kGemvSegBlocks * 32),
                             t.codes + static_cast<size_t>(row0 + lane) * p.K + static_cast<size_t>(s) * kGemvSegBlocks * 32, cbytes, &full[stage]);
                } else if (lane >= 16 && lane < 16 + static_cast<int>(nrows)) {
                    const int r = lane - 16;
                    bulk_g2s(st + kQ8StageCodeBytes + r * (kGemvSegBlocks * 2),
                             t.scales + static_cast<size_t>(row0 + r) * p.nbp + static_cast<size_t>(s) * kGemvSegBlocks, sbytes, &full[stage]);
                }
            }
        }
        // Nothing may still be landing in shared memory when the CTA exits: wait (bounded) for
        // the most recent phase of every stage that was armed.
        if (lane == 0) {
            const uint32_t armed = unit < static_cast<uint32_t>(kGemvStages) ? unit : kGemvStages;
            for (uint32_t k = 0; k < armed; ++k) {
                const uint32_t u = unit - 1 - k;
                if (!mbar_wait(&full[u % kGemvStages], (u / kGemvStages) & 1)) atomicExch(p.error_word, kErrDrainTimeout);
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    // The activations (and the output buffers) belong to the stream's earlier work: wait for it.
    pdl_wait();
    // Prologue: quantise the activations into the lane-major layout.  Block b = 64*s + 32*i + l is
    // read by lane l; its two 16-byte halves are stored in the order that lane loads them
    // (half ((l>>2)&1) first), which keeps both the weight and the activation loads conflict-free.
    // Four lanes share a block (eight consecutive elements each), so one pass of the eight warps
    // covers 64 blocks with two 128-bit loads per lane and the whole vector in a few passes.
    {
        const uint32_t quad = static_cast<uint32_t>(lane) >> 2, part = static_cast<uint32_t>(lane) & 3;
        for (int t = 0; t < kBatch; ++t) {
            for (uint32_t b0 = warp * 8; b0 < p.nb; b0 += kGemvWarps * 8) {  // warp-uniform trip count: the quantiser shuffles
                const uint32_t b = b0 + quad;
                const bool live = b < p.nb;
                const float4* src = reinterpret_cast<const float4*>(p.x + static_cast<size_t>(t) * p.K + b * 32 + part * 8);
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 lo = live ? __ldg(src) : zero, hi = live ? __ldg(src + 1) : zero;
                const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                uint2 c1, c2;
                const float d = quantise_block_quad(v, c1, c2);
                if (!live) continue;
                const uint32_t l = b & 31, grp = b >> 5;  // grp == 2*s + i
                const uint32_t hh = (part >> 1) ^ ((l >> 2) & 1);
                const size_t slot = (static_cast<size_t>(grp) * 2 + hh) * 32 + l;  // uint4 index
                uint2* dst = reinterpret_cast<uint2*>(xcodes + (static_cast<size_t>(t) * kDigits) * kpad_blocks * 2 + slot) + (part & 1);
                *dst = c1;
                if (kDigits == 2) dst[static_cast<size_t>(kpad_blocks) * 4] = c2;
                if (part == 0) xscale[static_cast<size_t>(t) * kpad_blocks + b] = kDigits == 2 ? d * (1.0f / 256.0f) : d;
            }
        }
    }
    // consumer-only barrier (the producer warp is already streaming)
    asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");

    uint32_t unit = 0;
    bool ok = true;
    const uint32_t h0 = (static_cast<uint32_t>(lane) >> 2) & 1;
    GroupWalk walk(r_first, r_last);
    while (!walk.done() && ok) {
        uint32_t row0, nrows;
        const GemvTask& t = p.task[walk.next(p, row0, nrows)];
        const uint32_t row = row0 + warp;
        const bool valid = static_cast<uint32_t>(warp) < nrows;
        float acc[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) acc[b] = 0.0f;

        for (uint32_t s = 0; s < p.nseg; ++s, ++unit) {
            const uint32_t stage = unit % kGemvStages;
            if (*abort_word || !mbar_wait(&full[stage], (unit / kGemvStages) & 1)) {
                if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                ok = false;
                break;
            }
            if (valid) {
                const uint8_t* st = ring + stage * kQ8StageBytes;
                const uint4* wq = reinterpret_cast<const uint4*>(st + warp * (kGemvSegBlocks * 32));
                const __half* ws = reinterpret_cast<const __half*>(st + kQ8StageCodeBytes + warp * (kGemvSegBlocks * 2));
#pragma unroll
                for (int i = 0; i < kGemvSegBlocks / 32; ++i) {
                    const uint32_t bl = i * 32 + lane;           // block within the segment
                    const uint32_t b = s * kGemvSegBlocks + bl;  // block within the row
                    if (b < p.nb) {
                        const uint4 wa = wq[bl * 2 + h0], wb = wq[bl * 2 + (h0 ^ 1)];
                        const float dw = __half2float(ws[bl]);
                        const size_t slot = (static_cast<size_t>(b >> 5) * 2) * 32 + lane;
#pragma unroll
                        for (int tk = 0; tk < kBatch; ++tk) {
                            const uint4* xc = xcodes + (static_cast<size_t>(tk) * kDigits) * kpad_blocks * 2 + slot;
                            const uint4 xa = xc[0], xb = xc[32];
                            int isum = dp4a_ss(wa.x, xa.x, 0);
                            isum = dp4a_ss(wa.y, xa.y, isum);
                            isum = dp4a_ss(wa.z, xa.z, isum);
                            isum = dp4a_ss(wa.w, xa.w, isum);
                            isum = dp4a_ss(wb.x, xb.x, isum);
                            isum = dp4a_ss(wb.y, xb.y, isum);
                            isum = dp4a_ss(wb.z, xb.z, isum);
                            isum = dp4a_ss(wb.w, xb.w, isum);
                            if (kDigits == 2) {
                                const uint4 ya = xc[kpad_blocks * 2], yb = xc[kpad_blocks * 2 + 32];
                                int lo = dp4a_ss(wa.x, ya.x, 0);
                                lo = dp4a_ss(wa.y, ya.y, lo);
                                lo = dp4a_ss(wa.z, ya.z, lo);
                                lo = dp4a_ss(wa.w, ya.w, lo);
                                lo = dp4a_ss(wb.x, yb.x, lo);
                                lo = dp4a_ss(wb.y, yb.y, lo);
                                lo = dp4a_ss(wb.z, yb.z, lo);
                                lo = dp4a_ss(wb.w, yb.w, lo);
                                isum = isum * 256 + lo;
                            }
                            const float dx = xscale[static_cast<size_t>(tk) * kpad_blocks + b];
                            acc[tk] = fmaf(dw * dx, static_cast<float>(isum), acc[tk]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
        }
        if (!ok) break;
        if (valid) {
#pragma unroll
            for (int tk = 0; tk < kBatch; ++tk) {
                float v = acc[tk];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) t.y[static_cast<size_t>(tk) * t.rows + row] = v;
            }
        }
    }
}

}  // namespace zk
