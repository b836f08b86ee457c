// Greedy token pick over fp32 logits: per token row, the index of the first maximum among the finite
// entries, -1 when the row has none.
//
// This is the greedy branch of the reference's sampler (sample_logits,
// src/adapters/dense_transformer_runtime.cpp:391-418): candidates are the finite logits in ascending
// index order, a candidate replaces the best only when it is strictly greater, so the lowest index wins
// ties and -0.0 ties with +0.0.
//
// A row of logits may be laid out in up to eight segments (the gathered shards of a row-sharded
// lm_head: [rank][token][shard rows]); a segment carries the index of its first entry.  Every
// candidate is packed into one 64-bit key, (order-preserving bits of the value) << 32 | (2^32-1 - index),
// so that an unsigned maximum is exactly the reference's rule; key 0 means "no candidate".  CTAs
// reduce their share in registers and shared memory and merge with one atomicMax per CTA, so the
// result does not depend on the order in which CTAs run.
#pragma once
#include <cstdint>

#include "zk_ptx.cuh"

namespace zk {

constexpr int kPickMaxSegments = 8;
constexpr int kPickThreads = 256;

struct PickSegment {
    const float* base;       // first entry of token 0
    uint32_t len;            // entries per token
    uint32_t first_index;    // index of the segment's first entry within the row
    uint32_t token_stride;   // floats between consecutive tokens
    uint32_t pad;
};

struct PickParams {
    PickSegment seg[kPickMaxSegments];
    uint32_t nseg;
    uint32_t ctas_per_segment;
    unsigned long long* keys;  // [tokens], zeroed before the launch; finished in place by pick_finish_kernel
};

__device__ __forceinline__ unsigned long long pick_key(float v, uint32_t index) {
    v += 0.0f;  // -0.0 -> +0.0: the reference compares values, and the two zeros are equal
    const uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7f800000u) == 0x7f800000u) return 0ull;  // infinities and NaNs are never candidates
    const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - index);
}

// grid = (nseg * ctas_per_segment, tokens)
__global__ void __launch_bounds__(kPickThreads) pick_scan_kernel(const __grid_constant__ PickParams p) {
    pdl_launch_dependents();
    pdl_wait();   // the logits, and the cleared keys, come from earlier launches
    const uint32_t s = blockIdx.x / p.ctas_per_segment, part = blockIdx.x % p.ctas_per_segment;
    const PickSegment& sg = p.seg[s];
    const float* row = sg.base + static_cast<size_t>(blockIdx.y) * sg.token_stride;
    unsigned long long best = 0ull;
    for (uint32_t i = part * kPickThreads + threadIdx.x; i < sg.len; i += p.ctas_per_segment * kPickThreads) {
        const unsigned long long k = pick_key(__ldcg(row + i), sg.first_index + i);  // L2: the producer may be a peer's store
        best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    __shared__ unsigned long long warp_best[kPickThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < kPickThreads / 32; ++w) best = warp_best[w] > best ? warp_best[w] : best;
        if (best) atomicMax(p.keys + blockIdx.y, best);
    }
}

// keys[t] -> picked index as a signed 64-bit integer, in place.
__global__ void pick_finish_kernel(unsigned long long* keys, uint32_t tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    const unsigned long long k = keys[t];
    reinterpret_cast<long long*>(keys)[t] = k ? static_cast<long long>(0xffffffffu - static_cast<uint32_t>(k)) : -1ll;
}

}  // namespace zk
