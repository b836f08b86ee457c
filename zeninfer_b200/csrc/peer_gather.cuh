// Output all-gather fused into the decode kernels, over peer memory (NVLink / NVSwitch).
//
// A projection is sharded by output rows, one shard per GPU (one process per GPU).  Instead of
// running the product and then a separate collective, the product kernel itself delivers its
// outputs: a CTA collects the outputs of its row slice in shared memory and, when the slice is
// done, copies the run into the same slot of every rank's gather region with coalesced peer
// stores.  The launch's number is published into every rank's flag array by the NEXT kernel on
// the gather object (one idle thread of it, as soon as the launch has ended), off every critical
// path.  A kernel that consumes the gathered vector (the next launch in the chain, or
// gather_fetch_kernel) waits, with a clock budget, until all ranks' flags have reached the
// number it needs.  No host round trip, no extra launch, and the next launch's weight stream
// overlaps the link latency.  The reference drives one device and has no counterpart of this
// file; the row cut it mirrors is ComputePool::parallel_for's (src/compute_pool.cpp:104-106).
//
// Region layout in each rank's memory (allocated once, zero-filled, shared through CUDA IPC):
//     float  data[2][world][slot_floats]      two parities: launch L writes parity L & 1
//     u64    flags[kMaxPeers]                 flags[r] = number of launches rank r has published here
// Launch L (1-based) of a rank may only start writing once every rank has published L-1, so a
// rank is never more than one launch ahead of any other and the parity it overwrites (that of
// launch L-2) is no longer being read by anyone.
//
// Ordering, and why it looks the way it does: a fence at system scope costs this GPU tens of
// nanoseconds that do not overlap with other such fences, so a launch may afford one, not one per
// CTA or per warp (148 of them were measured at about 10 us per launch).  Writers of a CTA meet
// at a CTA barrier after their peer stores; one thread then counts the CTA in with an atomic, and
// the thread that completes the count advances the rank's launch counter (no fence: see below).
// The publishing thread of the next kernel starts after that grid has completed, fences ONCE at
// system scope -- fences are cumulative, so this covers every store of the completed grid, and
// by then their acknowledgements are mostly in, so the fence is short -- and stores the flags.
// Readers poll their own (local) flags with relaxed system-scope loads and
// read the data through L2 (never L1), the point where peer stores to local memory land.
// Only loads of local memory ever spin.
#pragma once
#include <cstdint>

#include "zk_ptx.cuh"

namespace zk {

constexpr int kMaxPeers = 8;
enum : int { kErrPeerWaitTimeout = 5 };

struct PeerGather {
    float* region[kMaxPeers];                 // data base of every rank's region (own entry = local memory)
    unsigned long long* flags[kMaxPeers];     // flag array of every rank's region
    float* local_region;
    const unsigned long long* local_flags;
    unsigned long long* epoch;                // local: launches this rank has completed
    unsigned int* arrive;                     // local: CTAs of the running launch that have finished
    unsigned long long* published;            // local: launches whose number has been stored into the ranks' flags
    uint32_t world, rank, slot_floats;        // world == 0: no gather, the kernel writes its ordinary outputs only
    uint32_t grid;                            // CTAs of every gather launch on this object, the same on all ranks
};

__host__ __device__ inline size_t peer_region_data_bytes(size_t world, size_t slot_floats) { return 2 * world * slot_floats * sizeof(float); }
__host__ __device__ inline size_t peer_region_flag_offset(size_t world, size_t slot_floats) {
    return ((peer_region_data_bytes(world, slot_floats) + 255) / 256) * 256;
}
__host__ __device__ inline size_t peer_region_bytes(size_t world, size_t slot_floats) {
    return peer_region_flag_offset(world, slot_floats) + static_cast<size_t>(kMaxPeers) * sizeof(unsigned long long);
}

__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// The number of launches this rank has completed so far (the running launch is number epoch + 1).  Valid once the
// previous grid in the stream has completed.
__device__ __forceinline__ unsigned long long gather_epoch(const PeerGather& g) {
    return *reinterpret_cast<volatile unsigned long long*>(g.epoch);
}

// Warp-wide: waits until every rank has published `epoch` launches; false (warp-uniform) when the clock budget ran out
// first.  A launch calls it before it reads gathered data and, at the latest, before it stores into other ranks' regions.
__device__ __forceinline__ bool gather_wait(const PeerGather& g, int lane, unsigned long long epoch) {
    bool ok = true;
    if (lane < static_cast<int>(g.world) && lane != static_cast<int>(g.rank)) {   // own outputs are local and complete
        const unsigned long long* f = g.local_flags + lane;
        if (ld_relaxed_sys(f) < epoch) {
            const long long t0 = clock64();
            while (ld_relaxed_sys(f) < epoch)
                if (clock64() - t0 > g_wait_budget_cycles) { ok = false; break; }
        }
    }
    __threadfence();   // GPU scope: nothing that follows is satisfied from before the flags were seen
    return __all_sync(0xffffffffu, ok);
}

// Where launch (epoch + 1) of this rank puts element `off` of its slot, in rank `peer`'s region.
__device__ __forceinline__ float* gather_slot(const PeerGather& g, unsigned long long epoch, uint32_t peer, uint32_t off) {
    const size_t parity = static_cast<size_t>((epoch + 1) & 1);
    return g.region[peer] + (parity * g.world + g.rank) * g.slot_floats + off;
}
// The vector gathered by the launch before this one (what a chained launch reads as its input), in local memory.
__device__ __forceinline__ const float* gather_previous(const PeerGather& g, unsigned long long epoch) {
    return g.local_region + static_cast<size_t>(epoch & 1) * g.world * g.slot_floats;
}

// Copies a CTA's finished outputs -- stash[token][n_mine], rows [r_first, r_first + n_mine) of the launch's row space
// -- into every rank's region.  Jobs (rank, token) are dealt to warps; a warp stores 32 consecutive floats at a time.
__device__ __forceinline__ void gather_push(const PeerGather& g, unsigned long long epoch, const float* stash, uint32_t n_mine,
                                            uint32_t r_first, uint32_t total_rows, uint32_t tokens, int warp, int nwarps, int lane) {
    for (uint32_t job = warp; job < g.world * tokens; job += nwarps) {
        const uint32_t peer = job % g.world, tk = job / g.world;
        float* dst = gather_slot(g, epoch, peer, tk * total_rows + r_first);
        const float* src = stash + static_cast<size_t>(tk) * n_mine;
        for (uint32_t i = lane; i < n_mine; i += 32) dst[i] = src[i];
    }
}

// One thread per CTA, after every writer of the CTA has passed a CTA barrier: count the CTA in; the thread that
// completes the count advances the rank's own launch counter.
__device__ __forceinline__ void gather_finish(const PeerGather& g, unsigned long long epoch) {
    // No fence here: the counter only numbers the launches.  What orders the peer stores before the flags is the end of
    // this grid followed by the publishing thread's fence; a fence in every CTA would keep the CTA resident until its
    // peer stores are acknowledged and hold back the next launch's weight stream on this SM.
    const unsigned int prev = atomicAdd(g.arrive, 1u);
    if (prev == gridDim.x - 1) {
        *reinterpret_cast<volatile unsigned int*>(g.arrive) = 0;  // the next launch counts again only after this grid has ended
        *reinterpret_cast<volatile unsigned long long*>(g.epoch) = epoch + 1;
    }
}

// One thread of a kernel, once the previous grid in the stream has completed: tell every rank about the launches this
// rank has finished but not announced yet.  This holds the one system-scope fence a launch costs.
__device__ __forceinline__ void gather_publish_pending(const PeerGather& g) {
    const unsigned long long done = *reinterpret_cast<volatile unsigned long long*>(g.epoch);
    if (*reinterpret_cast<volatile unsigned long long*>(g.published) < done) {
        fence_acq_rel_sys();
        for (uint32_t p = 0; p < g.world; ++p) st_relaxed_sys(g.flags[p] + g.rank, done);
        *reinterpret_cast<volatile unsigned long long*>(g.published) = done;
    }
}

// Waits until the latest launch of every rank has landed here, then copies the gathered vector
// ([world][slot_floats], the parity of the latest launch) to `out`.  One CTA per 1024 floats.
__global__ void __launch_bounds__(256) gather_fetch_kernel(const PeerGather g, float* __restrict__ out, int* error_word) {
    const int lane = threadIdx.x & 31;
    if (blockIdx.x == 0 && threadIdx.x == 0) gather_publish_pending(g);   // the last launch has no successor to do it
    const unsigned long long epoch = gather_epoch(g);
    if (!gather_wait(g, lane, epoch)) {
        if (threadIdx.x == 0) atomicExch(error_word, kErrPeerWaitTimeout);
        return;
    }
    if (!out) return;
    const float* src = gather_previous(g, epoch);
    const size_t n = static_cast<size_t>(g.world) * g.slot_floats;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        out[i] = __ldcv(src + i);   // written by peers: never through a stale non-coherent line
}

// A plain all-gather of device vectors over the same regions and flags, for the vectors no product kernel produces
// (attention output, SwiGLU activation) or whose producer also folds other work in: every rank's `piece` (n floats, a
// multiple of 4) ends up in every rank's `whole` at [rank * n, (rank + 1) * n).  One CTA: it copies the piece into its
// slot of every rank's region (peer stores), meets at a CTA barrier, one thread fences once at system scope and raises
// this launch's number in every rank's flags; warp 0 then waits (bounded) for all ranks' flags and the CTA copies the
// other ranks' slots from the local region to `whole`.  The launch number is a device counter, so a captured launch can
// be replayed.  A rank starts launch L only after its launch L-1 has seen every rank's L-1, i.e. after every rank has
// finished reading launch L-2, whose parity launch L overwrites.  An object used by this kernel is not used by the
// product kernels' fused gather (they number launches differently).
__global__ void __launch_bounds__(1024) allgather_kernel(const PeerGather g, const float* __restrict__ piece, uint32_t n, float* __restrict__ whole,
                                                         int* error_word) {
    __shared__ int wait_ok;
    pdl_launch_dependents();     // the next launch may stream its weights meanwhile; it reads `whole` only after its own wait
    pdl_wait();
    const unsigned long long launch = gather_epoch(g) + 1;
    const uint32_t n4 = n / 4;
    for (uint32_t peer = 0; peer < g.world; ++peer) {
        float4* dst = reinterpret_cast<float4*>(gather_slot(g, launch - 1, peer, 0));
        const float4* src = reinterpret_cast<const float4*>(piece);
        for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        fence_acq_rel_sys();
        for (uint32_t p = 0; p < g.world; ++p) st_relaxed_sys(g.flags[p] + g.rank, launch);
    }
    if (threadIdx.x < 32) {
        const bool ok = gather_wait(g, static_cast<int>(threadIdx.x), launch);
        if (threadIdx.x == 0) wait_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned long long*>(g.epoch) = launch;   // counted even when the wait gave up
    if (!wait_ok) {
        if (threadIdx.x == 0) atomicExch(error_word, kErrPeerWaitTimeout);
        return;
    }
    const float* local = gather_previous(g, launch);    // the parity launch `launch` wrote
    for (uint32_t r = 0; r < g.world; ++r) {
        float4* dst = reinterpret_cast<float4*>(whole + static_cast<size_t>(r) * n);
        if (r == g.rank) {
            if (reinterpret_cast<const float*>(dst) != piece)
                for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = reinterpret_cast<const float4*>(piece)[i];
            continue;
        }
        const float4* src = reinterpret_cast<const float4*>(local + static_cast<size_t>(r) * g.slot_floats);
        for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = __ldcv(src + i);   // written by a peer: never through a stale line
    }
}

// The all-reduce that goes with a column cut: inout[i] += partial_0[i] + partial_1[i] + ... , the ranks' partial products
// added in rank order on every rank, so that all ranks hold the same sums bit for bit.  Same regions, flags, launch
// counter and parities as allgather_kernel (the two may alternate on one object); a rank's own partial is read from
// `partial` and not sent to itself.
__global__ void __launch_bounds__(1024) allreduce_add_kernel(const PeerGather g, const float* __restrict__ partial, uint32_t n, float* __restrict__ inout,
                                                             int* error_word) {
    __shared__ int wait_ok;
    pdl_launch_dependents();
    pdl_wait();
    const unsigned long long launch = gather_epoch(g) + 1;
    const uint32_t n4 = n / 4;
    const float4* mine = reinterpret_cast<const float4*>(partial);
    for (uint32_t peer = 0; peer < g.world; ++peer) {
        if (peer == g.rank) continue;
        float4* dst = reinterpret_cast<float4*>(gather_slot(g, launch - 1, peer, 0));
        for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = mine[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        fence_acq_rel_sys();
        for (uint32_t p = 0; p < g.world; ++p) st_relaxed_sys(g.flags[p] + g.rank, launch);
    }
    if (threadIdx.x < 32) {
        const bool ok = gather_wait(g, static_cast<int>(threadIdx.x), launch);
        if (threadIdx.x == 0) wait_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned long long*>(g.epoch) = launch;
    if (!wait_ok) {
        if (threadIdx.x == 0) atomicExch(error_word, kErrPeerWaitTimeout);
        return;
    }
    const float* local = gather_previous(g, launch);
    float4* io = reinterpret_cast<float4*>(inout);
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 acc = io[i];
        for (uint32_t r = 0; r < g.world; ++r) {
            const float4 v = r == g.rank ? mine[i] : __ldcv(reinterpret_cast<const float4*>(local + static_cast<size_t>(r) * g.slot_floats) + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        io[i] = acc;
    }
}

}  // namespace zk
