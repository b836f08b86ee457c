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
//     walks it in groups of eight rows.  Sixteen consumer warps form two teams of
//     eight; consecutive groups go to alternate teams, and inside a team every warp
//     owns one row and keeps that row's accumulators in registers until the row is
//     finished.  No partial sum ever crosses a warp, so results are deterministic;
//   * one producer warp streams the groups through a ring of shared-memory stages
//     with 1-D TMA bulk copies (cp.async.bulk), one K-segment of up to 128 blocks
//     at a time, each stage guarded by a full/empty mbarrier pair.  When a row is a
//     single segment (K <= 4096) a whole group is one contiguous 32 KB copy.
//     Bytes in flight are set by the ring depth, not by registers or occupancy;
//   * the activation vector is quantised once per CTA in the prologue (while the
//     first weight stages are already in flight) into a lane-major layout, so
//     every shared-memory read in the inner loop is a conflict-free 128-bit load;
//     for batch-1 int8 rows of at most 128 blocks it then moves into registers;
//   * launched with programmatic stream serialisation: the weight stream of launch
//     n+1 starts while launch n drains (weights are constants), and only the
//     activation read waits for the previous grid (griddepcontrol.wait);
//   * per 32-element block: 8 dp4a per digit, one int->float conversion and one
//     fused multiply-add with the fp16 block scale times the activation scale.
//
//   * with a peer gather attached (row-sharded tensor, one GPU per shard) the finishing warp
//     also stores each output into every rank's gather region and the grid's last CTA
//     publishes the launch (peer_gather.cuh): the all-gather costs no launch of its own.
//
// Algorithmic traffic is the raw GGUF size: 34 bytes per block.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "peer_gather.cuh"
#include "quantize_acts.cuh"
#include "zk_ptx.cuh"

namespace zk {

constexpr int kTeamWarps = 8;                       // warps per team == rows per row group
#ifndef ZK_GEMV_TEAMS
#define ZK_GEMV_TEAMS 2
#endif
constexpr int kTeams = ZK_GEMV_TEAMS;               // 1 or 2
constexpr int kGemvWarps = kTeamWarps * kTeams;     // consumer warps
constexpr int kGemvSegBlocks = 128;                 // 32-element blocks per K segment: four per lane
constexpr int kLaneBlocks = kGemvSegBlocks / 32;
#ifndef ZK_GEMV_STAGES
#define ZK_GEMV_STAGES 4
#endif
constexpr int kGemvStages = ZK_GEMV_STAGES;
// A parity wait is only meaningful to a waiter that has seen the barrier's previous phase complete: on a barrier still
// one phase behind, the test for the next phase's parity passes at once.  Units go to teams in turn, so the ring depth
// must be a multiple of the team count: then a stage always serves the same team, and that team observes every phase of
// the stage's barrier in order.  (With an odd depth a team met a stage whose previous phase belonged to the other team,
// could read it while its copy was still in flight and hand it back early.)
static_assert(kGemvStages % kTeams == 0, "ring depth must be a multiple of the number of consumer teams");
constexpr int kGemvThreads = (kGemvWarps + 1) * 32;
constexpr int kMaxTasks = 8;                        // projections sharing one input (zen::hip::kMaxBatch, include/zen/hip_backend.h:70)

constexpr uint32_t kQ8StageCodeBytes = kTeamWarps * kGemvSegBlocks * 32;
constexpr uint32_t kQ8StageScaleBytes = kTeamWarps * kGemvSegBlocks * 2;
constexpr uint32_t kQ8StageBytes = kQ8StageCodeBytes + kQ8StageScaleBytes;
constexpr uint32_t kL2PrefetchCap = 160 * 1024;     // bytes of the slice beyond the ring that are pulled into L2 up front

constexpr uint32_t kGemvFlagSwiglu = 1u;      // input = silu(x_gate) * x
constexpr uint32_t kGemvFlagNorm = 2u;        // input = RMSNorm(x) * norm_weight, formed in the prologue
constexpr uint32_t kGemvFlagAccumulate = 4u;  // y += W x instead of y = W x (the residual add)
constexpr uint32_t kGemvFlagWarm = 8u;        // pull the start of the next launch's tensor into L2 (producer warp only)
// Two tasks of equal shape, gate and up: row r of both is computed by the two teams of one CTA at the same time, and
// task 0's output receives silu(gate . x) * (up . x) (silu_mul, src/adapters/dense_transformer_runtime.cpp:193-199).
// The launch's row space is ONE task's rows (total_rows = rows, both first_row = 0).
constexpr uint32_t kGemvFlagPairSwiglu = 64u;
constexpr uint32_t kWarmCapBytes = 192 * 1024;   // per CTA

// Tensor maps of one resident tensor whose rows span several K segments (built on upload, kept in device memory):
// codes as [rows][K / 256][256] bytes with boxes of n rows x 16 x 256 (one segment of a row group; a tile's innermost
// extent is limited to 256 elements, hence the split of K), scales as [rows][nbp] halves with boxes of n x 128;
// n = 8, 4, 2, 1: a partial group (the end of a CTA's row slice) is fetched with the smaller boxes.
struct alignas(64) GemvTileMaps {
    CUtensorMap codes[4];
    CUtensorMap scales[4];
};

struct GemvTask {
    const uint8_t* codes;    // [rows][K] int8
    const __half* scales;    // [rows][nbp]
    float* y;                // [batch][rows], token-major
    uint32_t rows;
    uint32_t first_row;      // index of this task's first row in the launch's concatenated row space
};

// Kernel parameters live in constant memory that is cold on every SM at the start of every launch, and a warp stalls
// on each line it misses (about half a microsecond, one after the other).  So everything a single-tensor launch needs
// sits in the first 64 bytes (the scalars and task[0]; blocks per row, padded pitch and segment count are derived from
// K), and the consumer warps touch the remaining lines, one line per warp, while they wait for the previous grid.
struct GemvParams {
    const float* x;          // [batch][K] fp32; null with a gather: the vector gathered by the previous launch
    int* error_word;         // set to a zk::kErr* code when a bounded wait gives up
    uint32_t total_rows;     // over all tasks
    uint32_t ntasks;
    uint32_t K;              // columns; nb = K / 32 blocks per row, scale pitch nb rounded up to 8, nseg = ceil(nb / 128)
    uint32_t flags;          // kGemvFlag*: what happens to the input while it is quantised, and whether y accumulates
    GemvTask task[kMaxTasks];
    PeerGather gather;       // world == 0: outputs go to task[].y only
    const float* x_gate;     // [batch][K] fp32, read only with kGemvFlagSwiglu (a cold parameter line, touched by fused launches only)
    const float* norm_weight;  // [K] fp32, read only with kGemvFlagNorm
    float norm_eps;
    // kGemvFlagWarm: the tensor the stream's next product will read.  Its rows are cut like this launch's rows, and
    // every CTA's producer asks L2 for its cut once its own copies are out: the next launch then finds its first
    // stages in L2 instead of waiting a DRAM round trip for them, which is most of a small product's time.
    uint32_t warm_rows, warm_K, warm_nbp;
    const uint8_t* warm_codes;
    const __half* warm_scales;
    // Rows of several K segments: per task, the tensor maps in device memory (GemvTileMaps) through which one copy per
    // plane fetches a segment of a row group; null where a tensor has none (its rows then go one copy each).
    const GemvTileMaps* tile_maps[kMaxTasks];
#ifdef ZK_TRACE
    unsigned long long* trace;  // [grid][16] phase stamps (profiling builds only)
#endif
};

#ifdef ZK_TRACE
__device__ __forceinline__ unsigned long long zk_globaltimer() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define ZK_STAMP(slot) do { if (trace_base && threadIdx.x == 0) trace_base[blockIdx.x * 16 + (slot)] = zk_globaltimer(); } while (0)
#else
#define ZK_STAMP(slot) do {} while (0)
#endif

// Shared memory a launch with a peer gather adds: one float per (token, row of the largest CTA slice).
__host__ __device__ inline size_t gather_stash_bytes(uint32_t total_rows, uint32_t grid, int batch) {
    return static_cast<size_t>(batch) * ((total_rows + grid - 1) / grid) * sizeof(float);
}

__host__ __device__ inline size_t gemv_q8_0_smem_bytes(uint32_t nseg, int batch, int digits) {
    const size_t kpad_blocks = static_cast<size_t>(nseg) * kGemvSegBlocks;
    return static_cast<size_t>(kGemvStages) * kQ8StageBytes        // weight ring
           + static_cast<size_t>(batch) * digits * kpad_blocks * 32  // activation codes
           + static_cast<size_t>(batch) * kpad_blocks * 4            // activation scales
           + 2 * kGemvStages * 8 + 16                                // barriers + abort word
           + kMaxTasks * kGemvWarps * sizeof(double);                // per-warp sums of squares of a fused RMSNorm
}

// The slice of the launch's concatenated row space that CTA `cta` of `n` owns.
__device__ __forceinline__ void cta_row_slice(uint32_t total_rows, uint32_t cta, uint32_t n, uint32_t& first, uint32_t& last) {
    first = static_cast<uint32_t>(static_cast<uint64_t>(total_rows) * cta / n);
    last = static_cast<uint32_t>(static_cast<uint64_t>(total_rows) * (cta + 1) / n);
}

struct RowGroup {
    uint32_t task, row0, nrows;  // nrows == 0: no group (the odd tail of a pair)
};

// Walks a row slice in groups of at most kTeamWarps rows that never straddle two tasks.
struct GroupWalk {
    uint32_t r, r_end, ti;
    bool paired;   // kGemvFlagPairSwiglu: every group goes out twice in a row, for task 0 and then for task 1
    __device__ GroupWalk(uint32_t first, uint32_t last, bool paired_ = false) : r(first), r_end(last), ti(0), paired(paired_) {}
    __device__ bool done() const { return r >= r_end; }
    __device__ RowGroup next(const GemvParams& p) {
        RowGroup g{0, 0, 0};
        if (done()) return g;
        if (paired) {
            g.task = ti;
            g.row0 = r;
            g.nrows = min(static_cast<uint32_t>(kTeamWarps), r_end - r);
            if (ti) r += g.nrows;
            ti ^= 1u;
            return g;
        }
        while (r >= p.task[ti].first_row + p.task[ti].rows) ++ti;
        g.task = ti;
        g.row0 = r - p.task[ti].first_row;
        g.nrows = min(min(static_cast<uint32_t>(kTeamWarps), p.task[ti].rows - g.row0), r_end - r);
        r += g.nrows;
        return g;
    }
};

__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ int dot32(const uint4& wa, const uint4& wb, const uint4& xa, const uint4& xb) {
    int s = dp4a_ss(wa.x, xa.x, 0);
    s = dp4a_ss(wa.y, xa.y, s);
    s = dp4a_ss(wa.z, xa.z, s);
    s = dp4a_ss(wa.w, xa.w, s);
    s = dp4a_ss(wb.x, xb.x, s);
    s = dp4a_ss(wb.y, xb.y, s);
    s = dp4a_ss(wb.z, xb.z, s);
    s = dp4a_ss(wb.w, xb.w, s);
    return s;
}

#ifndef ZK_GEMV_MIN_CTAS
#define ZK_GEMV_MIN_CTAS 1
#endif
// kFuse: the launch may carry kGemvFlag* work (fused RMSNorm / SwiGLU input, accumulating store).  It is a template
// parameter because even untaken flag tests in the prologue and the store cost the plain 4096 x 4096 product 5 %.
template <int kBatch, int kDigits, bool kFuse = false>
__global__ void __launch_bounds__(kGemvThreads, (kBatch * kDigits == 1 ? ZK_GEMV_MIN_CTAS : 1))
    gemv_q8_0_kernel(const __grid_constant__ GemvParams p) {
    const uint32_t flags = kFuse ? p.flags : 0u;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t nb = p.K >> 5, nbp = (nb + 7) & ~7u, nseg = (nb + kGemvSegBlocks - 1) / kGemvSegBlocks;
    const uint32_t kpad_blocks = nseg * kGemvSegBlocks;
    uint8_t* ring = smem;
    uint4* xcodes = reinterpret_cast<uint4*>(ring + kGemvStages * kQ8StageBytes);           // [batch][digit][kpad_blocks*2]
    float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xcodes) + static_cast<size_t>(kBatch) * kDigits * kpad_blocks * 32);
    uint64_t* full = reinterpret_cast<uint64_t*>(xscale + static_cast<size_t>(kBatch) * kpad_blocks);
    uint64_t* empty = full + kGemvStages;
    volatile int* abort_word = reinterpret_cast<volatile int*>(empty + kGemvStages);
    double* norm_part = reinterpret_cast<double*>(empty + kGemvStages + 2);   // fused RMSNorm: [batch][consumer warp]
    float* stash = reinterpret_cast<float*>(norm_part + kMaxTasks * kGemvWarps);   // gather only: [batch][rows of this CTA's slice]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ZK_TRACE
    unsigned long long* const trace_base = p.trace;
#endif
    ZK_STAMP(0);
#ifdef ZK_TRACE
    if (trace_base && threadIdx.x == 0) { unsigned sm; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm)); trace_base[blockIdx.x * 16 + 13] = sm; }
#endif
    uint32_t r_first, r_last;
    cta_row_slice(p.total_rows, blockIdx.x, gridDim.x, r_first, r_last);
    const uint32_t n_mine = r_last - r_first;
    // A group of whole single-segment rows is contiguous in both planes: one copy each.
    const bool contiguous = nseg == 1 && nb == nbp;
    const uint32_t cstride = contiguous ? nb * 32 : kGemvSegBlocks * 32;  // stage row pitch of the codes, bytes
    const uint32_t sstride = contiguous ? nb : kGemvSegBlocks;             // stage row pitch of the scales, halves

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kTeamWarps);
        }
        *abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Let the next launch in the stream begin: its weight stream may overlap this grid's tail.
    pdl_launch_dependents();

    if (warp == kGemvWarps) {
        // ---------------- producer warp: weights are constants, no need to wait for the previous grid ----------------
        bool met = false;   // has the L2 prefetch of the rows beyond the ring's first fill been issued yet
        // CTA 0's producer also announces the previous launch to the other ranks, once its own first copies are out
        bool announce = p.gather.world != 0 && blockIdx.x == 0;
        uint32_t unit = 0;
        bool ok = true;
        GroupWalk walk(r_first, r_last, kFuse && (p.flags & kGemvFlagPairSwiglu));
        while (!walk.done() && ok) {
            RowGroup pair[kTeams];
#pragma unroll
            for (int m = 0; m < kTeams; ++m) pair[m] = walk.next(p);
            for (uint32_t s = 0; s < nseg && ok; ++s) {
#pragma unroll
                for (int m = 0; m < kTeams; ++m, ++unit) {
                    const uint32_t stage = unit % kGemvStages;
                    if (unit >= kGemvStages && announce) {
                        announce = false;
                        if (lane == 0) { pdl_wait(); gather_publish_pending(p.gather); }
                        __syncwarp();
                    }
                    if (unit >= kGemvStages && !met) {
                        met = true;
                        if (lane == 0) {
                            // Pull what the ring cannot hold yet into L2, so later refills do not pay DRAM latency.
                            uint32_t budget = kL2PrefetchCap;
                            GroupWalk pre(r_first + min(static_cast<uint32_t>(kGemvStages * kTeamWarps) / nseg, n_mine), r_last);
                            while (!pre.done() && budget) {
                                const RowGroup g = pre.next(p);
                                const GemvTask& t = p.task[g.task];
                                const uint32_t cb = min(g.nrows * p.K, budget);
                                l2_prefetch(t.codes + static_cast<size_t>(g.row0) * p.K, (cb + 15) & ~15u);
                                l2_prefetch(t.scales + static_cast<size_t>(g.row0) * nbp, (g.nrows * nbp * 2 + 15) & ~15u);
                                budget -= cb;
                            }
                        }
                        __syncwarp();
                    }
                    if (unit >= kGemvStages) {
                        if (!mbar_wait(&empty[stage], ((unit / kGemvStages) - 1) & 1)) {
                            if (lane == 0) { *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); }
                            ok = false;
                        }
                    }
                    if (*abort_word) ok = false;
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const RowGroup g = pair[m];  // m is a compile-time index (unrolled)
                    if (g.nrows == 0) {  // the odd tail of a pair: an empty unit keeps the ring order fixed
                        if (lane == 0) mbar_arrive(&full[stage]);
                        continue;
                    }
                    const GemvTask& t = p.task[g.task];
                    uint8_t* st = ring + stage * kQ8StageBytes;
                    if (contiguous) {
                        const uint32_t cbytes = g.nrows * p.K, sbytes = g.nrows * nb * 2;
                        if (lane == 0) {
                            mbar_arrive_expect_tx(&full[stage], cbytes + sbytes);
                            bulk_g2s(st, t.codes + static_cast<size_t>(g.row0) * p.K, cbytes, &full[stage]);
                            bulk_g2s(st + kQ8StageCodeBytes, t.scales + static_cast<size_t>(g.row0) * nbp, sbytes, &full[stage]);
#ifdef ZK_TRACE
                            if (trace_base && unit == 0) trace_base[blockIdx.x * 16 + 11] = zk_globaltimer();
#endif
                        }
                    } else if (p.tile_maps[g.task] != nullptr) {
                        // tiled copies, one per plane for a whole row group (boxes of 4, 2 and 1 rows for a partial one),
                        // instead of one copy per row and plane: sixteen small copies a stage held this path at 0.67 of the
                        // HBM rate where the contiguous one reaches 0.86.  Columns past the end of the row arrive as zeros
                        // and count as bytes like the rest of the box.
                        if (lane == 0) {
                            const GemvTileMaps* maps = p.tile_maps[g.task];
                            mbar_arrive_expect_tx(&full[stage], g.nrows * (kGemvSegBlocks * 32 + kGemvSegBlocks * 2));
                            uint32_t done_rows = 0;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const uint32_t box = 8u >> k;
                                if (g.nrows - done_rows >= box) {
                                    tma_load_3d(st + done_rows * (kGemvSegBlocks * 32), &maps->codes[k], 0, static_cast<int>(s * (kGemvSegBlocks * 32 / 256)),
                                                static_cast<int>(g.row0 + done_rows), &full[stage]);
                                    tma_load_2d(st + kQ8StageCodeBytes + done_rows * (kGemvSegBlocks * 2), &maps->scales[k], static_cast<int>(s * kGemvSegBlocks),
                                                static_cast<int>(g.row0 + done_rows), &full[stage]);
                                    done_rows += box;
                                }
                            }
                        }
                    } else {
                        const uint32_t nblk = min(static_cast<uint32_t>(kGemvSegBlocks), nb - s * kGemvSegBlocks);
                        const uint32_t cbytes = nblk * 32, sbytes = (nblk * 2 + 15) & ~15u;
                        if (lane == 0) mbar_arrive_expect_tx(&full[stage], g.nrows * (cbytes + sbytes));
                        __syncwarp();
                        if (lane < static_cast<int>(g.nrows)) {
                            bulk_g2s(st + lane * (kGemvSegBlocks * 32),
                                     t.codes + static_cast<size_t>(g.row0 + lane) * p.K + static_cast<size_t>(s) * kGemvSegBlocks * 32, cbytes, &full[stage]);
                        } else if (lane >= 16 && lane < 16 + static_cast<int>(g.nrows)) {
                            const int r = lane - 16;
                            bulk_g2s(st + kQ8StageCodeBytes + r * (kGemvSegBlocks * 2),
                                     t.scales + static_cast<size_t>(g.row0 + r) * nbp + static_cast<size_t>(s) * kGemvSegBlocks, sbytes, &full[stage]);
                        }
                    }
                }
            }
        }
        if (announce && lane == 0) { pdl_wait(); gather_publish_pending(p.gather); }
        if ((p.flags & kGemvFlagWarm) && ok && lane == 0) {
            uint32_t w_first, w_last;
            cta_row_slice(p.warm_rows, blockIdx.x, gridDim.x, w_first, w_last);
            const size_t code_bytes = min(static_cast<size_t>(w_last - w_first) * p.warm_K, static_cast<size_t>(kWarmCapBytes));
            const uint8_t* src = p.warm_codes + static_cast<size_t>(w_first) * p.warm_K;   // K is a multiple of 32: 16-byte aligned
            for (size_t off = 0; off < code_bytes; off += 32768)
                l2_prefetch(src + off, static_cast<uint32_t>((min(code_bytes - off, static_cast<size_t>(32768)) + 15) & ~static_cast<size_t>(15)));
            const uint32_t scale_rows = static_cast<uint32_t>(code_bytes / p.warm_K);
            if (scale_rows) l2_prefetch(p.warm_scales + static_cast<size_t>(w_first) * p.warm_nbp, (scale_rows * p.warm_nbp * 2 + 15) & ~15u);
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
    // While the previous grid drains: pull the parameter lines needed later into the constant cache, a different
    // 64-byte line per warp so the misses overlap (line 0, the scalars and task[0], is warm already).
    {
        uint32_t touched = 0;
        switch (warp & 7) {
        case 0: touched = p.task[1].rows; break;                                                   // bytes  64..127
        case 1: touched = p.task[3].rows; break;                                                   // bytes 128..191
        case 2: touched = p.task[5].rows; break;                                                   // bytes 192..255
        case 3: touched = p.task[7].rows; break;                                                   // bytes 256..319
        case 4: touched = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.gather.region[4])); break;   // 320..383
        case 5: touched = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.gather.flags[4])); break;    // 384..447
        case 6: touched = p.gather.world; break;                                                   // 448..
        default: break;
        }
        asm volatile("" ::"r"(touched));
    }
    // The activations (and the output buffers) belong to the stream's earlier work: wait for it.
    pdl_wait();
    ZK_STAMP(1);
    // Row-sharded launch: every rank must have published the launch before this one (its outputs are this launch's
    // input when x is null, and the slot parity written now was last read during that launch).
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
    // Prologue: quantise the activations into the lane-major layout.  Block b = 32*g + l is read by
    // lane l; its two 16-byte halves are stored in the order that lane loads them (half ((l>>2)&1)
    // first), which keeps both the weight and the activation loads conflict-free.
    // Four lanes share a block (eight consecutive elements each), so one pass of the consumer warps
    // covers 128 blocks with two 128-bit loads per lane: one pass for K = 4096.
    {
        const uint32_t quad = static_cast<uint32_t>(lane) >> 2, part = static_cast<uint32_t>(lane) & 3;
        // Fused RMSNorm (rms_norm, src/adapters/dense_transformer_runtime.cpp:117-125): a first pass over the row sums the
        // squares in double, warp by warp and then across the consumer warps in a fixed order; the quantising pass below
        // scales what it loads by inv * weight.  Every CTA repeats this for itself: the row is 16 KB in L2.
        if (kFuse && (flags & kGemvFlagNorm)) {
            for (int t = 0; t < kBatch; ++t) {
                double ss = 0.0;
                for (uint32_t b0 = warp * 8; b0 < nb; b0 += kGemvWarps * 8) {
                    const uint32_t b = b0 + quad;
                    if (b < nb) {
                        const float4* src = reinterpret_cast<const float4*>(x_src + static_cast<size_t>(t) * p.K + b * 32 + part * 8);
                        const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
                        ss += static_cast<double>(lo.x) * lo.x + static_cast<double>(lo.y) * lo.y + static_cast<double>(lo.z) * lo.z + static_cast<double>(lo.w) * lo.w
                            + static_cast<double>(hi.x) * hi.x + static_cast<double>(hi.y) * hi.y + static_cast<double>(hi.z) * hi.z + static_cast<double>(hi.w) * hi.w;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) norm_part[t * kGemvWarps + warp] = ss;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");
        }
        for (int t = 0; t < kBatch; ++t) {
            float inv_norm = 1.0f;
            if (kFuse && (flags & kGemvFlagNorm)) {
                double total = 0.0;
                for (int w = 0; w < kGemvWarps; ++w) total += norm_part[t * kGemvWarps + w];
                inv_norm = 1.0f / sqrtf(static_cast<float>(total / p.K) + p.norm_eps);
            }
            for (uint32_t b0 = warp * 8; b0 < nb; b0 += kGemvWarps * 8) {  // warp-uniform trip count: the quantiser shuffles
                const uint32_t b = b0 + quad;
                const bool live = b < nb;
                const float4* src = reinterpret_cast<const float4*>(x_src + static_cast<size_t>(t) * p.K + b * 32 + part * 8);
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                // L2 is the point of coherence for what earlier kernels and peers wrote: bypass L1
                const float4 lo = live ? __ldcg(src) : zero, hi = live ? __ldcg(src + 1) : zero;
                float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                if (kFuse && (flags & kGemvFlagNorm)) {
                    const float4* wsrc = reinterpret_cast<const float4*>(p.norm_weight + b * 32 + part * 8);
                    const float4 wlo = live ? __ldg(wsrc) : zero, whi = live ? __ldg(wsrc + 1) : zero;
                    const float nw[8] = {wlo.x, wlo.y, wlo.z, wlo.w, whi.x, whi.y, whi.z, whi.w};
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = v[e] * inv_norm * nw[e];   // x * inv * weight, the reference's order
                }
                if (kFuse && (flags & kGemvFlagSwiglu)) {
                    // SwiGLU fused into the load: silu(gate) * up, silu(z) = z / (1 + exp(-z))
                    // (silu_mul, src/adapters/dense_transformer_runtime.cpp:193-199)
                    const float4* gsrc = reinterpret_cast<const float4*>(p.x_gate + static_cast<size_t>(t) * p.K + b * 32 + part * 8);
                    const float4 glo = live ? __ldcg(gsrc) : zero, ghi = live ? __ldcg(gsrc + 1) : zero;
                    const float g[8] = {glo.x, glo.y, glo.z, glo.w, ghi.x, ghi.y, ghi.z, ghi.w};
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = (g[e] / (1.0f + expf(-g[e]))) * v[e];
                }
                uint2 c1, c2;
                const float d = quantise_block_quad(v, c1, c2);
                if (!live) continue;
                const uint32_t l = b & 31, grp = b >> 5;
                const uint32_t hh = (part >> 1) ^ ((l >> 2) & 1);
                const size_t slot = (static_cast<size_t>(grp) * 2 + hh) * 32 + l;  // uint4 index
                uint2* dst = reinterpret_cast<uint2*>(xcodes + (static_cast<size_t>(t) * kDigits) * kpad_blocks * 2 + slot) + (part & 1);
                *dst = c1;
                if (kDigits == 2) dst[static_cast<size_t>(kpad_blocks) * 4] = c2;
                if (part == 0) xscale[static_cast<size_t>(t) * kpad_blocks + b] = kDigits == 2 ? d * (1.0f / 256.0f) : d;
            }
        }
    }
    ZK_STAMP(2);
    // consumer-only barrier (the producer warp is already streaming)
    asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");
    ZK_STAMP(3);

    const int team = warp / kTeamWarps, twarp = warp % kTeamWarps;
    bool ok = *abort_word == 0;
    const uint32_t h0 = (static_cast<uint32_t>(lane) >> 2) & 1;

    // Batch-1 int8 rows of one segment (K <= 4096): a lane meets the same four activation blocks in
    // every row, so they live in registers and the inner loop reads only weights.
    constexpr bool kCanHoldX = (kBatch == 1 && kDigits == 1);
    const bool x_in_regs = kCanHoldX && nseg == 1;
    uint4 xra[kCanHoldX ? kLaneBlocks : 1], xrb[kCanHoldX ? kLaneBlocks : 1];
    float xrs[kCanHoldX ? kLaneBlocks : 1];
    if (x_in_regs) {
#pragma unroll
        for (int j = 0; j < kLaneBlocks; ++j) {
            const uint32_t b = j * 32 + lane;
            const bool live = b < nb;
            const uint4 z = make_uint4(0, 0, 0, 0);
            xra[j] = live ? xcodes[static_cast<size_t>(j) * 64 + lane] : z;
            xrb[j] = live ? xcodes[static_cast<size_t>(j) * 64 + 32 + lane] : z;
            xrs[j] = live ? xscale[b] : 0.0f;
        }
    }
    ZK_STAMP(4);

    uint32_t pair_base = 0;  // unit index of the current pair's first unit
    const bool pair_swiglu = kFuse && (flags & kGemvFlagPairSwiglu);
    float* pair_buf = reinterpret_cast<float*>(norm_part);   // [2 parities][batch][row of the group]: the prologue is done with norm_part
    uint32_t pair_parity = 0;
    GroupWalk walk(r_first, r_last, pair_swiglu);
    while (!walk.done() && ok) {
        RowGroup pair[kTeams];
#pragma unroll
        for (int m = 0; m < kTeams; ++m) pair[m] = walk.next(p);
        RowGroup g = pair[0];
        if constexpr (kTeams > 1) { if (team == 1) g = pair[kTeams - 1]; }  // no runtime-indexed local array
        const GemvTask& t = p.task[g.task];
        const uint32_t row = g.row0 + twarp;
        const bool valid = static_cast<uint32_t>(twarp) < g.nrows;
        float acc[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) acc[b] = 0.0f;
        // y += W x: fetch the old outputs now, so that their latency hides behind the row's dot products
        float y_old[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b)
            y_old[b] = (kFuse && (flags & kGemvFlagAccumulate) && valid && lane == 0 && t.y) ? __ldcg(t.y + static_cast<size_t>(b) * t.rows + row) : 0.0f;

        for (uint32_t s = 0; s < nseg; ++s) {
            const uint32_t unit = pair_base + s * kTeams + team;
            const uint32_t stage = unit % kGemvStages;
            if (*abort_word || !mbar_wait(&full[stage], (unit / kGemvStages) & 1)) {
                if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                ok = false;
                break;
            }
#ifdef ZK_TRACE
            if (team == 0 && unit < 4) ZK_STAMP(5 + 3 * (unit >> 1));
#endif
            if (valid) {
                const uint8_t* st = ring + stage * kQ8StageBytes;
                const uint4* wq = reinterpret_cast<const uint4*>(st + twarp * cstride);
                const __half* ws = reinterpret_cast<const __half*>(st + kQ8StageCodeBytes) + twarp * sstride;
                if (x_in_regs) {
#pragma unroll
                    for (int i = 0; i < kLaneBlocks; ++i) {
                        const uint32_t bl = i * 32 + lane;
                        // A lane whose block index is past the row holds zero codes; the bytes it reads are
                        // stale but inside the stage, and its term is dropped by selection (stale scale bits
                        // may be NaN, so it must not be multiplied away).
                        const uint4 wa = wq[bl * 2 + h0], wb = wq[bl * 2 + (h0 ^ 1)];
                        const float dw = __half2float(ws[bl]);
                        const int isum = dot32(wa, wb, xra[i], xrb[i]);
                        const float term = (dw * xrs[i]) * static_cast<float>(isum);
                        acc[0] += bl < nb ? term : 0.0f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < kLaneBlocks; ++i) {
                        const uint32_t bl = i * 32 + lane;           // block within the segment
                        const uint32_t b = s * kGemvSegBlocks + bl;  // block within the row
                        if (b < nb) {
                            const uint4 wa = wq[bl * 2 + h0], wb = wq[bl * 2 + (h0 ^ 1)];
                            const float dw = __half2float(ws[bl]);
                            const size_t slot = (static_cast<size_t>(b >> 5) * 2) * 32 + lane;
#pragma unroll
                            for (int tk = 0; tk < kBatch; ++tk) {
                                const uint4* xc = xcodes + (static_cast<size_t>(tk) * kDigits) * kpad_blocks * 2 + slot;
                                int isum = dot32(wa, wb, xc[0], xc[32]);
                                if (kDigits == 2) isum = isum * 256 + dot32(wa, wb, xc[kpad_blocks * 2], xc[kpad_blocks * 2 + 32]);
                                const float dx = xscale[static_cast<size_t>(tk) * kpad_blocks + b];
                                acc[tk] = fmaf(dw * dx, static_cast<float>(isum), acc[tk]);
                            }
                        }
                    }
                }
            }
#ifdef ZK_TRACE
            if (team == 0 && unit < 4) { if (acc[0] == 123.456f) trace_base[0] = 1; ZK_STAMP(6 + 3 * (unit >> 1)); }
#endif
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
        }
        if (kFuse && pair_swiglu) {
            // team 1 (up) hands its row sums to team 0 (gate) through shared memory; the barrier also agrees on failure,
            // so that no warp waits at it for one that gave up
            float v[kBatch];
#pragma unroll
            for (int tk = 0; tk < kBatch; ++tk) {
                v[tk] = acc[tk];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v[tk] += __shfl_xor_sync(0xffffffffu, v[tk], o);
            }
            float* slot = pair_buf + pair_parity * (kBatch * kTeamWarps);
            if (team == 1 && lane == 0) {
#pragma unroll
                for (int tk = 0; tk < kBatch; ++tk) slot[tk * kTeamWarps + twarp] = v[tk];
            }
            uint32_t any_failed;
            asm volatile(
                "{ .reg .pred p, q; setp.ne.u32 q, %2, 0; barrier.red.or.pred p, 2, %1, q; selp.u32 %0, 1, 0, p; }"
                : "=r"(any_failed) : "r"(kGemvWarps * 32), "r"(static_cast<uint32_t>(!ok)) : "memory");
            if (any_failed) { ok = false; break; }
            if (team == 0 && lane == 0 && valid && t.y) {
#pragma unroll
                for (int tk = 0; tk < kBatch; ++tk) {
                    const float z = v[tk];
                    t.y[static_cast<size_t>(tk) * t.rows + row] = (z / (1.0f + expf(-z))) * slot[tk * kTeamWarps + twarp];
                }
            }
            pair_parity ^= 1u;
            pair_base += kTeams * nseg;
            continue;
        }
        if (!ok) break;
#ifdef ZK_TRACE
        const uint32_t traced_unit = pair_base;
#endif
        pair_base += kTeams * nseg;
        if (valid) {
#pragma unroll
            for (int tk = 0; tk < kBatch; ++tk) {
                float v = acc[tk];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && t.y) t.y[static_cast<size_t>(tk) * t.rows + row] = kFuse ? y_old[tk] + v : v;   // y_old is zero unless accumulating
                if (lane == 0 && p.gather.world) stash[static_cast<size_t>(tk) * n_mine + (t.first_row + row - r_first)] = v;
            }
        }
#ifdef ZK_TRACE
        if (team == 0 && traced_unit < 4) ZK_STAMP(7 + 3 * (traced_unit >> 1));
#endif
    }
    ZK_STAMP(12);
    if (p.gather.world) {
        asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");   // the slice's outputs are all in the stash
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
