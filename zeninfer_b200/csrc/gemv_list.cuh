// A list of decode-time Q8_0 matrix-vector products (batch 1) in ONE persistent launch.
//
// The reference's answer to per-call overhead on a GPU is to record several products into one submission:
// ffn_residual_fused (o, residual, norm, gate|up, SwiGLU, down, residual in one command list) and
// layer_decode_pipeline (include/zen/d3d12_backend.h:289-352; the diagnosis is docs/hip_backend.md:121-125).  This is
// the same idea for gemv_q8_0_kernel (gemv_q8_0.cuh), whose single launches lose a third of their time at the launch
// boundary: a CTA owns most of an SM's shared memory, so the next launch's CTA starts only after it has left, and ring
// refill, a DRAM round trip and the prologue are paid serially per launch.
//
// One CTA per SM walks the items of the list in order.  Every item is a product as gemv_q8_0_kernel computes it (up
// to eight tensors sharing one input, optional fused RMSNorm / SwiGLU input and accumulating store):
//   * the producer warp never waits for an item boundary: weights are constants, so it streams the next item's rows
//     into the ring while the consumers still finish the current one, and the ring never drains;
//   * the consumer warps quantise the item's input while the ring is full, so the prologue is off the critical path;
//   * an item whose input (or accumulated output) is written by earlier items of the list carries kListFlagDepends:
//     its consumers wait, bounded, until every CTA has finished the item before it.  CTAs count finished items on
//     one device word; the arrival that completes the list clears the word for the next launch.  All waits are on
//     that word or on shared-memory barriers; a wait that runs out sets the error word, and the CTA still counts
//     its remaining items, so no other CTA and no later launch is left waiting.
// All CTAs must be resident at once for the dependency waits to make progress: the grid is one CTA per SM.
//
// Long rows are cut into equal K segments (K = 14336: four segments of 112 blocks), so every ring stage is filled;
// item i gives CTA c the row slice (c + 37 i) mod n of the item's rows, so the one-row imbalance of the cut does not
// fall on the same SMs in every item.  Arithmetic, per row, is gemv_q8_0_kernel's: results are bit-identical.
#pragma once
#include "gemv_q8_0.cuh"

namespace zk {

constexpr uint32_t kListFlagDepends = 16u;   // the item reads (or accumulates into) what earlier items of the list write
constexpr uint32_t kListRotate = 37u;        // slice rotation per item

struct alignas(16) GemvListItem {   // device memory, one per item
    const float* x;            // [K] fp32
    const float* x_gate;       // kGemvFlagSwiglu
    const float* norm_weight;  // kGemvFlagNorm
    float norm_eps;
    uint32_t flags;            // kGemvFlag* | kListFlagDepends
    uint32_t K, total_rows, ntasks, reserved;
    GemvTask task[kMaxTasks];
};
static_assert(sizeof(GemvListItem) % 16 == 0 && sizeof(GemvListItem) / 16 <= 32, "an item is copied to shared memory by one warp, 16 bytes per lane");

struct GemvListParams {
    const GemvListItem* items;
    uint32_t nitems;
    uint32_t kpad_blocks;      // blocks per row of the widest item, rounded up to whole 128-block segments
    unsigned int* counter;     // device word, zero between launches: finished (CTA, item) pairs of the running launch
    int* error_word;
};

__host__ __device__ inline size_t gemv_list_smem_bytes(uint32_t kpad_blocks, int digits) {
    return static_cast<size_t>(kGemvStages) * kQ8StageBytes + static_cast<size_t>(digits) * kpad_blocks * 32 + static_cast<size_t>(kpad_blocks) * 4 +
           2 * kGemvStages * 8 + 16 + kGemvWarps * sizeof(double) + 2 * sizeof(GemvListItem);
}

// Geometry of an item's rows in the ring.
struct ListShape {
    uint32_t nb, nbp, nseg, segb;   // blocks per row, scale pitch, K segments per row, blocks per segment (a multiple of 8, <= 128)
    bool contiguous;                // a group of whole rows is one copy per plane
    __device__ explicit ListShape(uint32_t K) {
        nb = K >> 5;
        nbp = (nb + 7) & ~7u;
        nseg = (nb + kGemvSegBlocks - 1) / kGemvSegBlocks;
        segb = nseg ? (((nb + nseg - 1) / nseg + 7) & ~7u) : 0;
        contiguous = nseg == 1 && nb == nbp;
    }
    __device__ uint32_t seg_blocks(uint32_t s) const { return min(segb, nb - s * segb); }
};

// Walks a row slice in groups of at most kTeamWarps rows that never straddle two tasks (tasks in shared memory).
struct ListWalk {
    const GemvTask* tasks;
    uint32_t r, r_end, ti;
    __device__ ListWalk(const GemvTask* t, uint32_t first, uint32_t last) : tasks(t), r(first), r_end(last), ti(0) {}
    __device__ bool done() const { return r >= r_end; }
    __device__ RowGroup next() {
        RowGroup g{0, 0, 0};
        if (done()) return g;
        while (r >= tasks[ti].first_row + tasks[ti].rows) ++ti;
        g.task = ti;
        g.row0 = r - tasks[ti].first_row;
        g.nrows = min(min(static_cast<uint32_t>(kTeamWarps), tasks[ti].rows - g.row0), r_end - r);
        r += g.nrows;
        return g;
    }
};

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One thread per CTA: count `n` finished items of this CTA; the arrival that completes the launch clears the word.
__device__ __forceinline__ void list_arrive(unsigned int* counter, uint32_t n, uint32_t nitems) {
    if (!n) return;
    __threadfence();   // the CTA's outputs (ordered before this thread by the CTA barrier) are visible before the count
    const unsigned int prev = atomicAdd(counter, n);
    if (prev + n == nitems * gridDim.x) atomicExch(counter, 0u);
}

template <int kDigits>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_q8_0_list_kernel(const __grid_constant__ GemvListParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t kpad_blocks = p.kpad_blocks;
    uint8_t* ring = smem;
    uint4* xcodes = reinterpret_cast<uint4*>(ring + kGemvStages * kQ8StageBytes);                  // [digit][kpad_blocks * 2]
    float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xcodes) + static_cast<size_t>(kDigits) * kpad_blocks * 32);
    uint64_t* full = reinterpret_cast<uint64_t*>(xscale + kpad_blocks);
    uint64_t* empty = full + kGemvStages;
    volatile int* abort_word = reinterpret_cast<volatile int*>(empty + kGemvStages);
    volatile int* stop_word = abort_word + 1;                                                          // the consumers' common view of abort_word, refreshed once per item
    double* norm_part = reinterpret_cast<double*>(empty + kGemvStages + 2);                         // [consumer warp]
    GemvListItem* item_prod = reinterpret_cast<GemvListItem*>(norm_part + kGemvWarps);
    GemvListItem* item_cons = item_prod + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ncta = gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kTeamWarps);
        }
        *abort_word = 0;
        *stop_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kGemvWarps) {
        // ---------------- producer warp: straight across item boundaries ----------------
        uint32_t unit = 0;
        bool ok = true;
        for (uint32_t it = 0; it < p.nitems && ok; ++it) {
            __syncwarp();
            if (lane < static_cast<int>(sizeof(GemvListItem) / 16))
                reinterpret_cast<uint4*>(item_prod)[lane] = __ldg(reinterpret_cast<const uint4*>(p.items + it) + lane);
            __syncwarp();
            const ListShape sh(item_prod->K);
            uint32_t r_first, r_last;
            cta_row_slice(item_prod->total_rows, (blockIdx.x + it * kListRotate) % ncta, ncta, r_first, r_last);
            ListWalk walk(item_prod->task, r_first, r_last);
            while (!walk.done() && ok) {
                RowGroup pair[kTeams];
#pragma unroll
                for (int m = 0; m < kTeams; ++m) pair[m] = walk.next();
                for (uint32_t s = 0; s < sh.nseg && ok; ++s) {
#pragma unroll
                    for (int m = 0; m < kTeams; ++m, ++unit) {
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
                        const RowGroup g = pair[m];
                        if (g.nrows == 0) {   // the odd tail of a pair: an empty unit keeps the ring order fixed
                            if (lane == 0) mbar_arrive(&full[stage]);
                            continue;
                        }
                        const GemvTask& t = item_prod->task[g.task];
                        uint8_t* st = ring + stage * kQ8StageBytes;
                        if (sh.contiguous) {
                            const uint32_t cbytes = g.nrows * item_prod->K, sbytes = g.nrows * sh.nb * 2;
                            if (lane == 0) {
                                mbar_arrive_expect_tx(&full[stage], cbytes + sbytes);
                                bulk_g2s(st, t.codes + static_cast<size_t>(g.row0) * item_prod->K, cbytes, &full[stage]);
                                bulk_g2s(st + kQ8StageCodeBytes, t.scales + static_cast<size_t>(g.row0) * sh.nbp, sbytes, &full[stage]);
                            }
                        } else {
                            const uint32_t nblk = sh.seg_blocks(s);
                            const uint32_t cbytes = nblk * 32, sbytes = (nblk * 2 + 15) & ~15u;
                            if (lane == 0) mbar_arrive_expect_tx(&full[stage], g.nrows * (cbytes + sbytes));
                            __syncwarp();
                            if (lane < static_cast<int>(g.nrows)) {
                                bulk_g2s(st + lane * (kGemvSegBlocks * 32),
                                         t.codes + static_cast<size_t>(g.row0 + lane) * item_prod->K + static_cast<size_t>(s) * sh.segb * 32, cbytes, &full[stage]);
                            } else if (lane >= 16 && lane < 16 + static_cast<int>(g.nrows)) {
                                const int r = lane - 16;
                                bulk_g2s(st + kQ8StageCodeBytes + r * (kGemvSegBlocks * 2),
                                         t.scales + static_cast<size_t>(g.row0 + r) * sh.nbp + static_cast<size_t>(s) * sh.segb, sbytes, &full[stage]);
                            }
                        }
                    }
                }
            }
        }
        // Nothing may still be landing in shared memory when the CTA exits.
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
    const int team = warp / kTeamWarps, twarp = warp % kTeamWarps;
    const uint32_t h0 = (static_cast<uint32_t>(lane) >> 2) & 1;
    const uint32_t quad = static_cast<uint32_t>(lane) >> 2, part = static_cast<uint32_t>(lane) & 3;
    constexpr bool kCanHoldX = kDigits == 1;
    uint32_t pair_base = 0;    // unit index of the current pair's first unit, running across items like the producer's
    uint32_t arrived = 0;      // items this CTA has counted (thread 0)
    pdl_wait();                // the first item's input and every output buffer belong to the stream's earlier work

    for (uint32_t it = 0; it < p.nitems; ++it) {
        if (warp == 0) {
            if (lane < static_cast<int>(sizeof(GemvListItem) / 16))
                reinterpret_cast<uint4*>(item_cons)[lane] = __ldg(reinterpret_cast<const uint4*>(p.items + it) + lane);
            __syncwarp();
            if (lane == 0) {
                if (it > 0 && (item_cons->flags & kListFlagDepends)) {
                    const unsigned int need = it * ncta;   // every CTA has finished items 0 .. it-1
                    if (ld_acquire_gpu_u32(p.counter) < need) {
                        const long long t0 = clock64();
                        while (ld_acquire_gpu_u32(p.counter) < need) {
                            if (clock64() - t0 > g_wait_budget_cycles) {
                                if (!*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrInputWaitTimeout); }
                                break;
                            }
                        }
                    }
                }
                *stop_word = *abort_word;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");   // A: item header, dependency and the stop decision are common
        if (*stop_word) break;

        const uint32_t flags = item_cons->flags;
        const ListShape sh(item_cons->K);
        const uint32_t nb = sh.nb;
        const float* x_src = item_cons->x;
        // ---- quantise the item's input into the lane-major layout (see gemv_q8_0_kernel) ----
        float inv_norm = 1.0f;
        if (flags & kGemvFlagNorm) {
            double ss = 0.0;
            for (uint32_t b0 = warp * 8; b0 < nb; b0 += kGemvWarps * 8) {
                const uint32_t b = b0 + quad;
                if (b < nb) {
                    const float4* src = reinterpret_cast<const float4*>(x_src + b * 32 + part * 8);
                    const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
                    ss += static_cast<double>(lo.x) * lo.x + static_cast<double>(lo.y) * lo.y + static_cast<double>(lo.z) * lo.z + static_cast<double>(lo.w) * lo.w
                        + static_cast<double>(hi.x) * hi.x + static_cast<double>(hi.y) * hi.y + static_cast<double>(hi.z) * hi.z + static_cast<double>(hi.w) * hi.w;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) norm_part[warp] = ss;
            asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");
            double total = 0.0;
            for (int w = 0; w < kGemvWarps; ++w) total += norm_part[w];
            inv_norm = 1.0f / sqrtf(static_cast<float>(total / item_cons->K) + item_cons->norm_eps);
        }
        for (uint32_t b0 = warp * 8; b0 < nb; b0 += kGemvWarps * 8) {   // warp-uniform trip count: the quantiser shuffles
            const uint32_t b = b0 + quad;
            const bool live = b < nb;
            const float4* src = reinterpret_cast<const float4*>(x_src + b * 32 + part * 8);
            const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 lo = live ? __ldcg(src) : zero, hi = live ? __ldcg(src + 1) : zero;   // L2: written by other SMs
            float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            if (flags & kGemvFlagNorm) {
                const float4* wsrc = reinterpret_cast<const float4*>(item_cons->norm_weight + b * 32 + part * 8);
                const float4 wlo = live ? __ldg(wsrc) : zero, whi = live ? __ldg(wsrc + 1) : zero;
                const float nw[8] = {wlo.x, wlo.y, wlo.z, wlo.w, whi.x, whi.y, whi.z, whi.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = v[e] * inv_norm * nw[e];
            }
            if (flags & kGemvFlagSwiglu) {
                const float4* gsrc = reinterpret_cast<const float4*>(item_cons->x_gate + b * 32 + part * 8);
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
            const size_t slot = (static_cast<size_t>(grp) * 2 + hh) * 32 + l;
            uint2* dst = reinterpret_cast<uint2*>(xcodes + slot) + (part & 1);
            *dst = c1;
            if (kDigits == 2) dst[static_cast<size_t>(kpad_blocks) * 4] = c2;
            if (part == 0) xscale[b] = kDigits == 2 ? d * (1.0f / 256.0f) : d;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");   // B: the input is quantised

        const bool x_in_regs = kCanHoldX && sh.nseg == 1;
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
        const uint32_t cstride = sh.contiguous ? nb * 32 : kGemvSegBlocks * 32;
        const uint32_t sstride = sh.contiguous ? nb : kGemvSegBlocks;

        uint32_t r_first, r_last;
        cta_row_slice(item_cons->total_rows, (blockIdx.x + it * kListRotate) % ncta, ncta, r_first, r_last);
        ListWalk walk(item_cons->task, r_first, r_last);
        bool ok = true;
        while (!walk.done() && ok) {
            RowGroup pair[kTeams];
#pragma unroll
            for (int m = 0; m < kTeams; ++m) pair[m] = walk.next();
            RowGroup g = pair[0];
            if constexpr (kTeams > 1) { if (team == 1) g = pair[kTeams - 1]; }
            const GemvTask& t = item_cons->task[g.task];
            const uint32_t row = g.row0 + twarp;
            const bool valid = static_cast<uint32_t>(twarp) < g.nrows;
            float acc = 0.0f;
            const float y_old = ((flags & kGemvFlagAccumulate) && valid && lane == 0) ? __ldcg(t.y + row) : 0.0f;

            for (uint32_t s = 0; s < sh.nseg; ++s) {
                const uint32_t unit = pair_base + s * kTeams + team;
                const uint32_t stage = unit % kGemvStages;
                if (*abort_word || !mbar_wait(&full[stage], (unit / kGemvStages) & 1)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                    ok = false;
                    break;
                }
                if (valid) {
                    const uint8_t* st = ring + stage * kQ8StageBytes;
                    const uint4* wq = reinterpret_cast<const uint4*>(st + twarp * cstride);
                    const __half* ws = reinterpret_cast<const __half*>(st + kQ8StageCodeBytes) + twarp * sstride;
                    if (x_in_regs) {
#pragma unroll
                        for (int i = 0; i < kLaneBlocks; ++i) {
                            const uint32_t bl = i * 32 + lane;
                            const uint4 wa = wq[bl * 2 + h0], wb = wq[bl * 2 + (h0 ^ 1)];
                            const float dw = __half2float(ws[bl]);
                            const int isum = dot32(wa, wb, xra[i], xrb[i]);
                            const float term = (dw * xrs[i]) * static_cast<float>(isum);
                            acc += bl < nb ? term : 0.0f;     // selected, not multiplied away: stale scale bits may be NaN
                        }
                    } else {
                        // A lane meets the blocks b of the row with b & 31 == lane, in rising order, whatever the segment length
                        // (segments start at multiples of eight blocks, which also keeps the half order h0 of the stage reads):
                        // the same blocks in the same order as gemv_q8_0_kernel, so the row sums are bit-identical to it.
                        const uint32_t nblk = sh.seg_blocks(s), b0 = s * sh.segb;
                        const uint32_t l0 = (static_cast<uint32_t>(lane) - b0) & 31u;
#pragma unroll
                        for (int i = 0; i < kLaneBlocks; ++i) {
                            const uint32_t bl = l0 + i * 32;             // block within the segment
                            const uint32_t b = b0 + bl;                  // block within the row
                            if (bl < nblk) {
                                const uint4 wa = wq[bl * 2 + h0], wb = wq[bl * 2 + (h0 ^ 1)];
                                const float dw = __half2float(ws[bl]);
                                const uint4* xc = xcodes + (static_cast<size_t>(b >> 5) * 2) * 32 + lane;
                                int isum = dot32(wa, wb, xc[0], xc[32]);
                                if (kDigits == 2) isum = isum * 256 + dot32(wa, wb, xc[kpad_blocks * 2], xc[kpad_blocks * 2 + 32]);
                                acc = fmaf(dw * xscale[b], static_cast<float>(isum), acc);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stage]);
            }
            if (!ok) break;
            pair_base += kTeams * sh.nseg;
            if (valid) {
                float v = acc;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) t.y[row] = y_old + v;   // y_old is zero unless accumulating
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kGemvWarps * 32) : "memory");   // C: this CTA's rows of the item are stored
        if (threadIdx.x == 0 && !*abort_word) { list_arrive(p.counter, 1, p.nitems); ++arrived; }
    }
    // Whatever happened, this CTA counts all its items: nobody is left waiting and the word returns to zero.
    if (threadIdx.x == 0) list_arrive(p.counter, p.nitems - arrived, p.nitems);
}

}  // namespace zk
