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
// to eight tensors sharing one input, optional fused RMSNorm / SwiGLU input and accumulating store).  Three kinds of
// warps run side by side, each in its own loop over the items, coupled only by shared-memory barriers:
//   * the producer warp never waits for an item boundary: weights are constants, so it streams the next item's rows
//     into the ring while the consumers still finish the current one, and the ring never drains; at every item
//     boundary it also asks L2 for its rows of the item after (cp.async.bulk.prefetch.L2), so HBM keeps streaming
//     while consumers wait for an item's input, and the ring refills from L2;
//   * sixteen consumer warps (two teams of eight rows) quantise the item's input, 1/16 each, into one of two
//     activation buffers and do the dot products, as in gemv_q8_0_kernel; the input of an item that does not depend
//     on the list is loaded before the previous item's rows are walked, so its latency is hidden;
//   * one service warp counts the CTA's finished items on a device word and watches that word for the consumers: an
//     item whose input (or accumulated output) is written by earlier items of the list carries kListFlagDepends and
//     starts once every CTA has counted the item before it.  The arrival that completes the list clears the word.
// Everything that needs a division (blocks per row, K segments, the CTAs' row slices) is worked out on the host when
// the list is built, and the items travel as kernel parameters (constant memory, up to kListMaxItems per launch; a
// longer list is launched in pieces): per item the device does a handful of additions on operands that cost no load,
// as gemv_q8_0_kernel does with its task table.  A wait that runs out sets the error word and
// the CTA-wide abort flag; every warp then leaves its loop (no hardware barrier is used after start-up, so nobody
// can be stranded), and the service warp still counts the CTA's remaining items, so no other CTA and no later launch
// is left waiting.  All CTAs must be resident at once for the dependency waits to make progress: the grid is one
// CTA per SM.
//
// Long rows are cut into equal K segments (K = 14336: four segments of 112 blocks), so every ring stage is filled;
// item i gives CTA c the row slice (c + 37 i) mod n of the item's rows, so the one-row imbalance of the cut does not
// fall on the same SMs in every item.  Arithmetic, per row, is gemv_q8_0_kernel's: results are bit-identical.
#pragma once
#include "gemv_q8_0.cuh"

namespace zk {

constexpr uint32_t kListFlagDepends = 16u;      // the item reads (or accumulates into) what earlier items of the list write
constexpr uint32_t kListFlagContiguous = 32u;   // a group of whole rows is one copy per plane (one K segment, no scale padding)
constexpr uint32_t kListRotate = 37u;           // slice rotation per item

struct alignas(16) GemvListItem {   // one per item, in the kernel's parameter space; geometry worked out by the host (list_create)
    const float* x;            // [K] fp32
    const float* x_gate;       // kGemvFlagSwiglu
    const float* norm_weight;  // kGemvFlagNorm
    float norm_eps;
    uint32_t flags;            // kGemvFlag* | kListFlag*
    uint32_t K, total_rows;
    uint32_t rows_q, rows_rem; // total_rows = rows_q * grid + rows_rem: slice c has rows_q + (c < rows_rem) rows
    uint32_t nb, nbp;          // blocks per row, scale pitch
    uint32_t nseg, segb;       // K segments per row, blocks per segment (a multiple of 8, at most 128)
    GemvTask task[kMaxTasks];
};
constexpr int kListMaxItems = 96;    // 96 x 320 bytes: inside the 32,764-byte limit on kernel parameters
constexpr int kListFewItems = 8;     // a second instantiation for short lists (a decoder layer's chain): 2.6 KB of parameters

constexpr int kListWarpProducer = kGemvWarps, kListWarpService = kGemvWarps + 1;
constexpr int kListThreads = (kGemvWarps + 2) * 32;
constexpr int kListMaxHoist = 4;   // passes of an input row a consumer warp loads at once (rows up to 16384 columns in one go)

template <int kItems>
struct GemvListParams {
    GemvListItem items[kItems];
    uint32_t nitems;
    uint32_t kpad_blocks;      // blocks per row of the widest item, rounded up to whole 128-block segments
    unsigned int* counter;     // device word, zero between launches: finished (CTA, item) pairs of the running launch
    int* error_word;
    uint32_t ahead_units;      // != 0: the producer asks L2 for its rows of the next item at every item boundary
#ifdef ZK_TRACE
    unsigned long long* trace; // [grid][256] time stamps, twelve per item (profiling builds only)
#endif
};

#ifdef ZK_TRACE
#define ZK_LSTAMP(item_index, slot) do { if (p.trace && (item_index) < 21) p.trace[blockIdx.x * 512 + (item_index) * 16 + (slot)] = zk_globaltimer(); } while (0)
#else
#define ZK_LSTAMP(item_index, slot) do {} while (0)
#endif

__host__ __device__ inline size_t gemv_list_smem_bytes(uint32_t kpad_blocks, int digits) {
    return static_cast<size_t>(kGemvStages) * kQ8StageBytes                                               // weight ring
           + 2 * (static_cast<size_t>(digits) * kpad_blocks * 32 + static_cast<size_t>(kpad_blocks) * 4)  // two activation buffers
           + (2 * kGemvStages + 12) * 8                                                                   // barriers, flags
           + 2 * kGemvWarps * sizeof(double)                                                              // RMSNorm partial sums, two sets
           ;
}

// Rows [first, last) of the item for the CTA whose rotated index is `slot`.
__device__ __forceinline__ void list_slice(const GemvListItem& item, uint32_t slot, uint32_t& first, uint32_t& last) {
    first = slot * item.rows_q + min(slot, item.rows_rem);
    last = first + item.rows_q + (slot < item.rows_rem ? 1u : 0u);
}

// Walks a row slice in groups of at most kTeamWarps rows that never straddle two tasks.  The bounds of the current task
// stay in registers (a task's first row is the end of the one before it), so a group costs no load unless the walk
// crosses into the next task.
struct ListWalk {
    const GemvTask* tasks;
    uint32_t r, r_end, ti, t_first, t_end;
    __device__ ListWalk(const GemvTask* t, uint32_t first, uint32_t last) : tasks(t), r(first), r_end(last), ti(0), t_first(0), t_end(0) {
        if (first < last) t_end = t[0].rows;
    }
    __device__ bool done() const { return r >= r_end; }
    __device__ RowGroup next() {
        RowGroup g{0, 0, 0};
        if (done()) return g;
        while (r >= t_end) { ++ti; t_first = t_end; t_end += tasks[ti].rows; }
        g.task = ti;
        g.row0 = r - t_first;
        g.nrows = min(min(static_cast<uint32_t>(kTeamWarps), t_end - r), r_end - r);
        r += g.nrows;
        return g;
    }
};

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait on a shared-memory barrier that also gives up as soon as another warp of the CTA has raised the abort
// flag.  A waiting warp sleeps inside the barrier test (suspend-time hint) and wakes when the phase completes.
#ifndef ZK_LIST_SLEEP_NS
#define ZK_LIST_SLEEP_NS 0
#endif
#ifndef ZK_LIST_CHECK_EVERY
#define ZK_LIST_CHECK_EVERY 1
#endif
__device__ __forceinline__ bool list_wait(uint64_t* bar, uint32_t parity, volatile int* abort_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait_hint(bar, parity, 4000)) {
        if (ZK_LIST_SLEEP_NS) __nanosleep(ZK_LIST_SLEEP_NS);
        if ((++spins % ZK_LIST_CHECK_EVERY) == 0 && (*abort_word || clock64() - t0 > g_wait_budget_cycles)) return false;
    }
    return true;
}

// Quantises the eight elements this lane holds of block b (four lanes share a block; every lane of the warp must call:
// the quantiser shuffles) and stores codes and scale in the lane-major layout of gemv_q8_0_kernel.
template <int kDigits>
__device__ __forceinline__ void list_quantise_store(const GemvListItem& I, uint32_t flags, float inv_norm, uint4* xcodes, float* xscale, uint32_t kpad_blocks,
                                                    uint32_t part, uint32_t b, bool live, const float4& lo, const float4& hi) {
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    if (flags & kGemvFlagNorm) {
        const float4* wsrc = reinterpret_cast<const float4*>(I.norm_weight + b * 32 + part * 8);
        const float4 wlo = live ? __ldg(wsrc) : zero4, whi = live ? __ldg(wsrc + 1) : zero4;
        const float nw[8] = {wlo.x, wlo.y, wlo.z, wlo.w, whi.x, whi.y, whi.z, whi.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v[e] * inv_norm * nw[e];   // x * inv * weight, the reference's order
    }
    if (flags & kGemvFlagSwiglu) {
        const float4* gsrc = reinterpret_cast<const float4*>(I.x_gate + b * 32 + part * 8);
        const float4 glo = live ? __ldcg(gsrc) : zero4, ghi = live ? __ldcg(gsrc + 1) : zero4;
        const float g[8] = {glo.x, glo.y, glo.z, glo.w, ghi.x, ghi.y, ghi.z, ghi.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (g[e] / (1.0f + expf(-g[e]))) * v[e];
    }
    uint2 c1, c2;
    const float d = quantise_block_quad(v, c1, c2);
    if (!live) return;
    const uint32_t l = b & 31, grp = b >> 5;
    const uint32_t hh = (part >> 1) ^ ((l >> 2) & 1);
    const size_t slot = (static_cast<size_t>(grp) * 2 + hh) * 32 + l;
    uint2* dst = reinterpret_cast<uint2*>(xcodes + slot) + (part & 1);
    *dst = c1;
    if (kDigits == 2) dst[static_cast<size_t>(kpad_blocks) * 4] = c2;
    if (part == 0) xscale[b] = kDigits == 2 ? d * (1.0f / 256.0f) : d;
}

__device__ __forceinline__ double list_sum_squares(const float4& lo, const float4& hi) {
    return static_cast<double>(lo.x) * lo.x + static_cast<double>(lo.y) * lo.y + static_cast<double>(lo.z) * lo.z + static_cast<double>(lo.w) * lo.w
         + static_cast<double>(hi.x) * hi.x + static_cast<double>(hi.y) * hi.y + static_cast<double>(hi.z) * hi.z + static_cast<double>(hi.w) * hi.w;
}

// Rows longer than 128 blocks: the warp meets blocks 8 warp + 128 k; kListMaxHoist passes are loaded at a time.  Kept out of
// line so that its arrays do not weigh on the registers of the common path.
__device__ __noinline__ double list_sum_squares_long(const float* x_src, uint32_t nb, uint32_t npass, uint32_t first_block, uint32_t part) {
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    double ss = 0.0;
    for (uint32_t k0 = 0; k0 < npass; k0 += kListMaxHoist) {
        float4 lo[kListMaxHoist], hi[kListMaxHoist];
#pragma unroll
        for (int j = 0; j < kListMaxHoist; ++j) {
            const uint32_t b = (k0 + j) * kGemvSegBlocks + first_block;
            const float4* src = reinterpret_cast<const float4*>(x_src + b * 32 + part * 8);
            lo[j] = b < nb ? __ldcg(src) : zero4;
            hi[j] = b < nb ? __ldcg(src + 1) : zero4;
        }
#pragma unroll
        for (int j = 0; j < kListMaxHoist; ++j)
            if ((k0 + j) * kGemvSegBlocks + first_block < nb) ss += list_sum_squares(lo[j], hi[j]);
    }
    return ss;
}
template <int kDigits>
__device__ __noinline__ void list_quantise_long(const GemvListItem& I, uint32_t flags, float inv_norm, uint4* xcodes, float* xscale, uint32_t kpad_blocks,
                                                uint32_t npass, uint32_t first_block, uint32_t part) {
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint32_t nb = I.nb;
    for (uint32_t k0 = 0; k0 < npass; k0 += kListMaxHoist) {
        float4 lo[kListMaxHoist], hi[kListMaxHoist];
#pragma unroll
        for (int j = 0; j < kListMaxHoist; ++j) {
            const uint32_t b = (k0 + j) * kGemvSegBlocks + first_block;
            const float4* src = reinterpret_cast<const float4*>(I.x + b * 32 + part * 8);
            lo[j] = b < nb ? __ldcg(src) : zero4;
            hi[j] = b < nb ? __ldcg(src + 1) : zero4;
        }
#pragma unroll
        for (int j = 0; j < kListMaxHoist; ++j) {
            const uint32_t b = (k0 + j) * kGemvSegBlocks + first_block;
            if (k0 + j < npass) list_quantise_store<kDigits>(I, flags, inv_norm, xcodes, xscale, kpad_blocks, part, b, b < nb, lo[j], hi[j]);   // warp-uniform
        }
    }
}

template <int kDigits, int kItems>
__global__ void __launch_bounds__(kListThreads, 1) gemv_q8_0_list_kernel(const __grid_constant__ GemvListParams<kItems> p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t kpad_blocks = p.kpad_blocks;
    const size_t xbuf_bytes = static_cast<size_t>(kDigits) * kpad_blocks * 32 + static_cast<size_t>(kpad_blocks) * 4;   // codes, then scales
    uint8_t* ring = smem;
    uint8_t* xbuf = ring + kGemvStages * kQ8StageBytes;                                       // [2][codes | scales]
    uint64_t* full = reinterpret_cast<uint64_t*>(xbuf + 2 * xbuf_bytes);
    uint64_t* empty = full + kGemvStages;
    uint64_t* x_ready = empty + kGemvStages;     // [2] every consumer warp has written its share of the quantised input of its item
    uint64_t* norm_bar = x_ready + 2;            // [2] every consumer warp has written its partial sum of squares
    uint64_t* item_done = norm_bar + 2;          // [4] every consumer warp has stored its rows of item j: barrier j & 3
    uint64_t* dep_ready = item_done + 4;         // the service warp has seen every CTA count the item before a dependent one
    volatile int* abort_word = reinterpret_cast<volatile int*>(dep_ready + 2);                      // 2 * kGemvStages + 10 barrier words so far
    double* norm_part = reinterpret_cast<double*>(dep_ready + 4);                                   // [2][consumer warp]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ncta = gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kTeamWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&x_ready[b], kGemvWarps);
            mbar_init(&norm_bar[b], kGemvWarps);
        }
        for (int b = 0; b < 4; ++b) mbar_init(&item_done[b], kGemvWarps);
        mbar_init(dep_ready, 1);
        *abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kListWarpProducer) {
        // ---------------- producer warp: straight across item boundaries ----------------
        // Everything the inner loop needs sits in registers: the item's geometry is read from its shared-memory copy once, a
        // row group's two base addresses once per pair, and a unit then costs a barrier test, an address addition and the copy.
        uint32_t unit = 0, rot = blockIdx.x;
        bool ok = true;
        for (uint32_t it = 0; it < p.nitems && ok; ++it) {
            const GemvListItem& I = p.items[it];
            const uint32_t K = I.K, nb = I.nb, nbp = I.nbp, nseg = I.nseg, segb = I.segb;
            const bool contiguous = (I.flags & kListFlagContiguous) != 0;
            uint32_t r_first, r_last;
            list_slice(I, rot, r_first, r_last);
            rot += kListRotate;
            while (rot >= ncta) rot -= ncta;
            // Ask L2 for the start of this CTA's rows of the NEXT item now (at most ahead_units ring stages' worth): HBM keeps
            // working while the consumers wait for an item's input, and the ring's first refill of that item comes from L2.
            if (p.ahead_units && it + 1 < p.nitems && lane < static_cast<int>(kMaxTasks)) {     // lane t: the part of the slice that falls into task t
                const GemvListItem& N = p.items[it + 1];
                uint32_t nfirst, nlast;
                list_slice(N, rot, nfirst, nlast);
                nlast = min(nlast, nfirst + p.ahead_units * kTeamWarps);
                const GemvTask& t = N.task[lane];
                const uint32_t a = max(nfirst, t.first_row), b = min(nlast, t.first_row + t.rows);
                if (a < b && t.rows) {
                    const size_t bytes = static_cast<size_t>(b - a) * N.K;
                    const uint8_t* src = t.codes + static_cast<size_t>(a - t.first_row) * N.K;
                    for (size_t off = 0; off < bytes; off += 32768)
                        l2_prefetch(src + off, static_cast<uint32_t>(min(bytes - off, static_cast<size_t>(32768))));
                    l2_prefetch(t.scales + static_cast<size_t>(a - t.first_row) * N.nbp, ((b - a) * N.nbp * 2 + 15) & ~15u);
                }
            }
            ListWalk walk(I.task, r_first, r_last);
            uint32_t cached_task = 0xffffffffu;
            const uint8_t* task_codes = nullptr;
            const __half* task_scales = nullptr;
            while (!walk.done() && ok) {
                RowGroup pair[kTeams];
                const uint8_t* codes[kTeams];
                const __half* scales[kTeams];
#pragma unroll
                for (int m = 0; m < kTeams; ++m) {
                    pair[m] = walk.next();
                    if (pair[m].nrows && pair[m].task != cached_task) {   // the task's planes: read again only when the walk changes task
                        cached_task = pair[m].task;
                        task_codes = I.task[cached_task].codes;
                        task_scales = I.task[cached_task].scales;
                    }
                    codes[m] = task_codes + static_cast<size_t>(pair[m].row0) * K;
                    scales[m] = task_scales + static_cast<size_t>(pair[m].row0) * nbp;
                }
                for (uint32_t s = 0; s < nseg && ok; ++s) {
#pragma unroll
                    for (int m = 0; m < kTeams; ++m, ++unit) {
                        const uint32_t stage = unit % kGemvStages;
                        if (unit >= kGemvStages) {
                            if (!list_wait(&empty[stage], ((unit / kGemvStages) - 1) & 1, abort_word)) {
                                if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrEmptyWaitTimeout); }
                                ok = false;
                            }
                        }
                        if (*abort_word) ok = false;
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
#ifdef ZK_TRACE
                        if (lane == 0 && p.trace && it < 21) { unsigned long long* tr = p.trace + blockIdx.x * 512 + it * 16; if (!tr[0]) tr[0] = zk_globaltimer(); tr[1] = zk_globaltimer(); }
#endif
                        const uint32_t nrows = pair[m].nrows;
                        if (nrows == 0) {   // the odd tail of a pair: an empty unit keeps the ring order fixed
                            if (lane == 0) mbar_arrive(&full[stage]);
                            continue;
                        }
                        uint8_t* st = ring + stage * kQ8StageBytes;
                        if (contiguous) {
                            const uint32_t cbytes = nrows * K, sbytes = nrows * nb * 2;
                            if (lane == 0) {
                                mbar_arrive_expect_tx(&full[stage], cbytes + sbytes);
                                bulk_g2s(st, codes[m], cbytes, &full[stage]);
                                bulk_g2s(st + kQ8StageCodeBytes, scales[m], sbytes, &full[stage]);
                            }
                        } else {
                            const uint32_t nblk = min(segb, nb - s * segb);
                            const uint32_t cbytes = nblk * 32, sbytes = (nblk * 2 + 15) & ~15u;
                            if (lane == 0) mbar_arrive_expect_tx(&full[stage], nrows * (cbytes + sbytes));
                            __syncwarp();
                            if (lane < static_cast<int>(nrows)) {
                                bulk_g2s(st + lane * (kGemvSegBlocks * 32), codes[m] + static_cast<size_t>(lane) * K + static_cast<size_t>(s) * segb * 32, cbytes, &full[stage]);
                            } else if (lane >= 16 && lane < 16 + static_cast<int>(nrows)) {
                                const int r = lane - 16;
                                bulk_g2s(st + kQ8StageCodeBytes + r * (kGemvSegBlocks * 2), scales[m] + static_cast<size_t>(r) * nbp + static_cast<size_t>(s) * segb, sbytes, &full[stage]);
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

    if (warp == kListWarpService) {
        // ---------------- service warp (one lane): the device word ----------------
        // For every item in turn: if it depends on the list, watch the word until every CTA has counted the item before it
        // and tell the consumers; then wait for the consumers to finish the item and count it.  This CTA's own count of
        // item j - 1 always precedes its watch for item j, so the two duties never wait for each other.
        if (lane != 0) return;
        pdl_wait();     // the word is cleared by the previous launch's last arrival
        uint32_t arrived = 0;
        const unsigned int total = p.nitems * ncta;
        auto count_in = [&](uint32_t n) {
            if (!n) return;
            __threadfence();   // cumulative: the consumers' outputs, observed through the item's barrier, are visible before the count
            const unsigned int prev = atomicAdd(p.counter, n);
            if (prev + n == total) atomicExch(p.counter, 0u);
        };
        for (uint32_t it = 0; it < p.nitems; ++it) {
            if (it > 0 && (p.items[it].flags & kListFlagDepends)) {
                const unsigned int need = it * ncta;   // every CTA has counted items 0 .. it-1
                bool ok = true;
                if (ld_acquire_gpu_u32(p.counter) < need) {
                    const long long t0 = clock64();
                    while (ld_acquire_gpu_u32(p.counter) < need) {
                        if (*abort_word) { ok = false; break; }
                        if (clock64() - t0 > g_wait_budget_cycles) {
                            *abort_word = 1; atomicExch(p.error_word, kErrInputWaitTimeout);
                            ok = false; break;
                        }
                    }
                }
                if (!ok) break;
                __threadfence();           // what the other CTAs wrote before they counted is ordered before the consumers' reads
                mbar_arrive(dep_ready);
            }
            // Four barriers in turn: the consumers would have to finish four more items before this lane has looked at one
            // for a phase to be missed.
            if (!list_wait(&item_done[it & 3], (it >> 2) & 1, abort_word)) break;   // the flag is up, or this wait ran out (then others did, too, and reported)
            ZK_LSTAMP(it, 8);
            count_in(1);
            ++arrived;
            ZK_LSTAMP(it, 9);
        }
        count_in(p.nitems - arrived);   // whatever happened, this CTA counts all its items: nobody is left waiting and the word returns to zero
        return;
    }

    // ---------------- consumer warps ----------------
    const int team = warp / kTeamWarps, twarp = warp % kTeamWarps;
    const uint32_t h0 = (static_cast<uint32_t>(lane) >> 2) & 1;
    const uint32_t quad = static_cast<uint32_t>(lane) >> 2, part = static_cast<uint32_t>(lane) & 3;
    constexpr bool kCanHoldX = kDigits == 1;
    uint32_t pair_base = 0;    // unit index of the current pair's first unit, running across items like the producer's
    uint32_t rot = blockIdx.x, dep_uses = 0, norm_uses = 0;
    pdl_wait();                // inputs and output buffers belong to the stream's earlier work
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 pre_lo = zero4, pre_hi = zero4;     // this lane's share of the NEXT item's input, when that item does not depend on the list
    bool pre_valid = false;

    for (uint32_t it = 0; it < p.nitems; ++it) {
        if (warp == 0 && lane == 0) ZK_LSTAMP(it, 2);
        const GemvListItem& I = p.items[it];
        const uint32_t flags = I.flags, nb = I.nb, nseg = I.nseg, buf = it & 1;
        uint4* xcodes = reinterpret_cast<uint4*>(xbuf + buf * xbuf_bytes);
        float* xscale = reinterpret_cast<float*>(xbuf + buf * xbuf_bytes + static_cast<size_t>(kDigits) * kpad_blocks * 32);
        if (*abort_word) break;
        if (it > 0 && (flags & kListFlagDepends)) {
            if (!list_wait(dep_ready, dep_uses & 1, abort_word)) {
                if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrInputWaitTimeout); }
                break;
            }
            ++dep_uses;
        }
        if (warp == 0 && lane == 0) ZK_LSTAMP(it, 3);

        // ---- this warp's sixteenth of the input: load, (norm,) quantise into the item's activation buffer ----
        const float* x_src = I.x;
        const uint32_t npass = (nb + kGemvSegBlocks - 1) / kGemvSegBlocks;    // passes of 128 blocks: 1 for K <= 4096, at most a handful
        float inv_norm = 1.0f;
        bool ok = true;
        // Meets the other consumer warps once every partial sum of squares is written; sets inv_norm.
        auto finish_norm = [&](double ss) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            double* part_sums = norm_part + (norm_uses & 1) * kGemvWarps;   // two sets in turn: the next use cannot overwrite sums still being added up
            if (lane == 0) { part_sums[warp] = ss; mbar_arrive(&norm_bar[norm_uses & 1]); }
            if (!list_wait(&norm_bar[norm_uses & 1], (norm_uses >> 1) & 1, abort_word)) {
                if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                return false;
            }
            ++norm_uses;
            double total = 0.0;
            for (int w = 0; w < kGemvWarps; ++w) total += part_sums[w];
            inv_norm = 1.0f / sqrtf(static_cast<float>(total / I.K) + I.norm_eps);
            return true;
        };
        if (npass == 1) {
            const uint32_t b = warp * 8 + quad;
            const bool live = b < nb;
            float4 lo = pre_lo, hi = pre_hi;
            if (!pre_valid) {
                const float4* src = reinterpret_cast<const float4*>(x_src + b * 32 + part * 8);
                lo = live ? __ldcg(src) : zero4;       // L2: written by other SMs
                hi = live ? __ldcg(src + 1) : zero4;
            }
            if (flags & kGemvFlagNorm) ok = finish_norm(live ? list_sum_squares(lo, hi) : 0.0);
            if (ok) list_quantise_store<kDigits>(I, flags, inv_norm, xcodes, xscale, kpad_blocks, part, b, live, lo, hi);
        } else {
            if (flags & kGemvFlagNorm) ok = finish_norm(list_sum_squares_long(x_src, nb, npass, warp * 8 + quad, part));
            if (ok) list_quantise_long<kDigits>(I, flags, inv_norm, xcodes, xscale, kpad_blocks, npass, warp * 8 + quad, part);
        }
        if (!ok) break;
        __syncwarp();
        if (warp == 0 && lane == 0) ZK_LSTAMP(it, 4);
        if (lane == 0) mbar_arrive(&x_ready[buf]);
        // The next item's input, if it was complete before the launch (no dependence on the list) and is one pass long: load it
        // now, so that it is in registers when this item's rows are done.
        pre_valid = false;
#ifndef ZK_LIST_NO_PRE
        if (it + 1 < p.nitems) {
            const GemvListItem& N = p.items[it + 1];
            if (!(N.flags & kListFlagDepends) && N.nb <= static_cast<uint32_t>(kGemvSegBlocks)) {
                const uint32_t b = warp * 8 + quad;
                const float4* src = reinterpret_cast<const float4*>(N.x + b * 32 + part * 8);
                pre_lo = b < N.nb ? __ldcg(src) : zero4;
                pre_hi = b < N.nb ? __ldcg(src + 1) : zero4;
                pre_valid = true;
            }
        }
#endif
        if (!list_wait(&x_ready[buf], (it >> 1) & 1, abort_word)) {
            if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
            break;
        }
        if (warp == 0 && lane == 0) ZK_LSTAMP(it, 5);
#ifdef ZK_TRACE
        const long long ck0 = clock64();
#endif

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
#ifdef ZK_TRACE
        const long long ck1 = clock64();
#endif
        const bool contiguous = (flags & kListFlagContiguous) != 0;
        const uint32_t cstride = contiguous ? nb * 32 : kGemvSegBlocks * 32;
        const uint32_t sstride = contiguous ? nb : kGemvSegBlocks;

        uint32_t r_first, r_last;
        list_slice(I, rot, r_first, r_last);
        rot += kListRotate;
        while (rot >= ncta) rot -= ncta;
        ListWalk walk(I.task, r_first, r_last);
        const uint32_t segb = I.segb;
        uint32_t cached_task = 0xffffffffu;
        float* task_y = nullptr;
        while (!walk.done() && ok) {
            RowGroup pair[kTeams];
#pragma unroll
            for (int m = 0; m < kTeams; ++m) pair[m] = walk.next();
            RowGroup g = pair[0];
            if constexpr (kTeams > 1) { if (team == 1) g = pair[kTeams - 1]; }
            if (g.nrows && g.task != cached_task) { cached_task = g.task; task_y = I.task[cached_task].y; }   // read again only when the walk changes task
            const uint32_t row = g.row0 + twarp;
            const bool valid = static_cast<uint32_t>(twarp) < g.nrows;
            float acc = 0.0f;
            const float y_old = ((flags & kGemvFlagAccumulate) && valid && lane == 0) ? __ldcg(task_y + row) : 0.0f;
#ifdef ZK_TRACE
            const long long ck2 = clock64();
#endif

            for (uint32_t s = 0; s < nseg; ++s) {
                const uint32_t unit = pair_base + s * kTeams + team;
                const uint32_t stage = unit % kGemvStages;
                if (*abort_word || !list_wait(&full[stage], (unit / kGemvStages) & 1, abort_word)) {
                    if (lane == 0 && !*abort_word) { *abort_word = 1; atomicExch(p.error_word, kErrFullWaitTimeout); }
                    ok = false;
                    break;
                }
#ifdef ZK_TRACE
                if (warp == 0 && lane == 0 && p.trace && it < 21) { unsigned long long* tr = p.trace + blockIdx.x * 512 + it * 16; if (!tr[6]) { tr[6] = zk_globaltimer();
                    tr[12] = static_cast<unsigned long long>(ck1 - ck0); tr[13] = static_cast<unsigned long long>(ck2 - ck1); tr[14] = static_cast<unsigned long long>(clock64() - ck2); } }
#endif
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
                        const uint32_t nblk = min(segb, nb - s * segb), b0 = s * segb;
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
#ifdef ZK_TRACE
                if (warp == 0 && lane == 0 && p.trace && it < 21) { unsigned long long* tr = p.trace + blockIdx.x * 512 + it * 16; if (!tr[10]) tr[10] = zk_globaltimer(); tr[11] = zk_globaltimer(); }
#endif
            }
            if (!ok) break;
            pair_base += kTeams * nseg;
            if (valid) {
                float v = acc;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) task_y[row] = y_old + v;   // y_old is zero unless accumulating
            }
        }
        if (!ok) break;
        __syncwarp();
        if (warp == 0 && lane == 0) ZK_LSTAMP(it, 7);
        if (lane == 0) mbar_arrive(&item_done[it & 3]);   // release: this warp's outputs are ordered before its arrival
    }
}

}  // namespace zk
