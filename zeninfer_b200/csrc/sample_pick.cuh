// Temperature / top-k / top-p sampling on the device: the non-greedy branch of the reference's sampler
// (sampling_distribution + sample_distribution, src/adapters/dense_transformer_runtime.cpp:349-390; the greedy branch is
// greedy_pick.cuh).  The logits stay in HBM; one CTA
//   1. finds the k highest finite logits with a four-pass radix select over order-preserving keys (k = top_k, at most
//      kSampleMaxCandidates; ties at the threshold go to the lowest indices),
//   2. sorts them by value (descending; equal values by index) and forms p_i = exp((v_i - max) / temperature) in double,
//      normalised over the candidates, as the reference does over its sorted `order`,
//   3. applies the top-p cut: the shortest prefix whose cumulative probability reaches top_p (at least one token), and
//      renormalises over it,
//   4. draws from the kept tokens IN TOKEN-ID ORDER with a uniform number the host supplies: the first token whose
//      cumulative probability reaches u.  That is the inverse-CDF walk std::discrete_distribution does over the
//      reference's id-indexed probability vector, so a host that feeds u from its own generator gets the reference's
//      choice up to the rounding of the partial sums; the generator itself stays on the host.
// The kept ids and their probabilities can be written out as well, for a host that prefers to draw itself.
//
// Limit: at most kSampleMaxCandidates tokens are kept.  With top_k == 0 (no top-k cut) or a larger top_k the reference
// normalises over, and may keep, more tokens than that: the probabilities are then still normalised over everything the
// reference would sort (one more pass over the logits), so the top-p cut falls where the reference's does whenever its
// nucleus has at most 1024 tokens; when it has more, the 1024 most likely are kept and `truncated` reports it.
#pragma once
#include <cstdint>

#include "zk_ptx.cuh"

namespace zk {

constexpr int kSampleThreads = 1024;
constexpr uint32_t kSampleMaxCandidates = 1024;

struct SampleParams {
    const float* logits;      // [n]
    uint32_t n;
    float temperature;        // > 0
    uint32_t top_k;           // 0: no cut (then the kSampleMaxCandidates most likely tokens are considered)
    float top_p;              // in (0, 1]; >= 1: no cut
    double u;                 // uniform in [0, 1)
    long long* pick;          // token id, -1 when no logit is finite
    int* kept_ids;            // optional [kSampleMaxCandidates]: kept token ids in ascending order
    double* kept_probs;       // optional [kSampleMaxCandidates]: their probabilities (sum 1)
    int* kept_count;          // optional
    int* truncated;           // optional: 1 when the candidates' cumulative probability stayed below top_p
};

// Order-preserving key of a finite float (larger float, larger key); 0 for a non-finite one (never a candidate).
__device__ __forceinline__ uint32_t sample_key(float v) {
    const uint32_t b = __float_as_uint(v);
    if ((b & 0x7f800000u) == 0x7f800000u) return 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(kSampleThreads) sample_top_kernel(const SampleParams p) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t cand_key[kSampleMaxCandidates];
    __shared__ uint32_t cand_idx[kSampleMaxCandidates];
    __shared__ double prob[kSampleMaxCandidates];
    __shared__ double scan[kSampleMaxCandidates];
    __shared__ uint32_t s_count, s_prefix, s_remaining, s_keep, s_ties_taken;
    const uint32_t tid = threadIdx.x;
    pdl_wait();     // the logits belong to the stream's earlier work

    // ---- how many finite logits there are
    if (tid == 0) s_count = 0;
    __syncthreads();
    uint32_t mine = 0;
    for (uint32_t i = tid; i < p.n; i += kSampleThreads) mine += sample_key(__ldcg(p.logits + i)) != 0u;
    mine = __reduce_add_sync(0xffffffffu, mine);
    if ((tid & 31) == 0 && mine) atomicAdd(&s_count, mine);
    __syncthreads();
    const uint32_t finite = s_count;
    if (finite == 0) {
        if (tid == 0) {
            *p.pick = -1;
            if (p.kept_count) *p.kept_count = 0;
            if (p.truncated) *p.truncated = 0;
        }
        return;
    }
    const uint32_t k = min(min(p.top_k ? p.top_k : kSampleMaxCandidates, kSampleMaxCandidates), finite);

    // ---- radix select: the key T of the k-th largest, and how many keys equal to T are still needed
    if (tid == 0) { s_prefix = 0; s_remaining = k; }
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (uint32_t i = tid; i < p.n; i += kSampleThreads) {
            const uint32_t key = sample_key(__ldcg(p.logits + i));
            if (key && (key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t remaining = s_remaining;
            int d = 255;
            for (; d > 0; --d) {
                if (hist[d] >= remaining) break;
                remaining -= hist[d];
            }
            s_prefix = prefix | (static_cast<uint32_t>(d) << shift);
            s_remaining = remaining;
            s_count = hist[d];     // after the last pass: the number of keys equal to T
        }
        __syncthreads();
        mask |= 255u << shift;
    }
    const uint32_t threshold = s_prefix, need_ties = s_remaining, ties = s_count;

    // ---- collect: everything above T, and of the keys equal to T the `need_ties` lowest indices
    if (tid == 0) { s_count = 0; s_ties_taken = 0; }
    __syncthreads();
    for (uint32_t i = tid; i < p.n; i += kSampleThreads) {
        const uint32_t key = sample_key(__ldcg(p.logits + i));
        if (key > threshold || (key == threshold && ties == need_ties)) {
            const uint32_t slot = atomicAdd(&s_count, 1u);
            if (slot < kSampleMaxCandidates) { cand_key[slot] = key; cand_idx[slot] = i; }
        }
    }
    __syncthreads();
    if (ties != need_ties) {
        // more keys equal to T than are needed (rare): walk the vocabulary in index order, 1024 at a time, and rank them
        for (uint32_t base = 0; base < p.n; base += kSampleThreads) {
            const uint32_t i = base + tid;
            const bool tie = i < p.n && sample_key(__ldcg(p.logits + i)) == threshold;
            const uint32_t ballot = __ballot_sync(0xffffffffu, tie);
            if ((tid & 31) == 0) hist[tid >> 5] = __popc(ballot);
            __syncthreads();
            uint32_t before = s_ties_taken;
            for (uint32_t w = 0; w < (tid >> 5); ++w) before += hist[w];
            const uint32_t rank = before + __popc(ballot & ((1u << (tid & 31)) - 1u));
            if (tie && rank < need_ties) {
                const uint32_t slot = atomicAdd(&s_count, 1u);
                if (slot < kSampleMaxCandidates) { cand_key[slot] = threshold; cand_idx[slot] = i; }
            }
            __syncthreads();
            if (tid == 0) { uint32_t total = 0; for (uint32_t w = 0; w < kSampleThreads / 32; ++w) total += hist[w]; s_ties_taken += total; }
            __syncthreads();
            if (s_ties_taken >= need_ties) break;
        }
        __syncthreads();
    }
    // k candidates are in cand_*[0, k) in no particular order; pad the rest so that the sort leaves them at the end
    if (tid >= k) { cand_key[tid] = 0u; cand_idx[tid] = 0xffffffffu; }
    __syncthreads();

    // ---- bitonic sort, descending by key, equal keys ascending by index
    auto before = [](uint32_t ka, uint32_t ia, uint32_t kb, uint32_t ib) { return ka > kb || (ka == kb && ia < ib); };
    for (uint32_t size = 2; size <= kSampleMaxCandidates; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            const uint32_t partner = tid ^ stride;
            if (partner > tid) {
                const bool up = (tid & size) == 0;     // this pair is to end in `before` order
                const uint32_t ka = cand_key[tid], ia = cand_idx[tid], kb = cand_key[partner], ib = cand_idx[partner];
                if (before(kb, ib, ka, ia) == up) { cand_key[tid] = kb; cand_idx[tid] = ib; cand_key[partner] = ka; cand_idx[partner] = ia; }
            }
            __syncthreads();
        }
    }

    // ---- p_i = exp((v_i - max) / temperature), normalised over the candidates (double, as the reference)
    const double maxv = static_cast<double>(__ldcg(p.logits + cand_idx[0]));
    double pi = 0.0;
    if (tid < k) pi = exp((static_cast<double>(__ldcg(p.logits + cand_idx[tid])) - maxv) / static_cast<double>(p.temperature));
    // inclusive prefix sums in sorted order (Hillis-Steele over shared memory, the same order of additions for every run)
    scan[tid] = pi;
    __syncthreads();
    for (uint32_t off = 1; off < kSampleMaxCandidates; off <<= 1) {
        const double add = tid >= off ? scan[tid - off] : 0.0;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
    }
    double total = scan[kSampleMaxCandidates - 1];
    const uint32_t k_wanted = p.top_k ? min(p.top_k, finite) : finite;     // how many tokens the reference normalises over
    if (k_wanted > k) {
        // the reference's sum runs over more tokens than the candidates: add the rest up over the whole vocabulary (with
        // top_k beyond the limit this takes in tokens the reference would cut, a mass below that of 1024 more likely ones)
        double part = 0.0;
        for (uint32_t i = tid; i < p.n; i += kSampleThreads) {
            const float v = __ldcg(p.logits + i);
            if (sample_key(v)) part += exp((static_cast<double>(v) - maxv) / static_cast<double>(p.temperature));
        }
        __syncthreads();
        prob[tid] = part;
        __syncthreads();
        for (uint32_t off = kSampleMaxCandidates / 2; off > 0; off >>= 1) {
            if (tid < off) prob[tid] += prob[tid + off];
            __syncthreads();
        }
        total = prob[0];
        __syncthreads();
    }
    // ---- top-p: the shortest prefix whose cumulative probability reaches top_p (at least one token)
    if (tid == 0) s_keep = k;
    __syncthreads();
    if (p.top_p > 0.0f && p.top_p < 1.0f && tid < k) {
        const double cum = scan[tid] / total, prev = tid ? scan[tid - 1] / total : 0.0;
        if (cum >= static_cast<double>(p.top_p) && !(tid && prev >= static_cast<double>(p.top_p))) s_keep = tid + 1;   // exactly one thread: the first crossing
    }
    __syncthreads();
    const uint32_t keep = max(1u, s_keep);
    const double kept_total = scan[keep - 1];
    // the reference would have kept more than the candidates: no top-p cut among more than 1024 wanted tokens, or a cut
    // the candidates' cumulative probability never reaches
    if (tid == 0 && p.truncated)
        *p.truncated = (k_wanted > k && (!(p.top_p > 0.0f && p.top_p < 1.0f) || scan[k - 1] / total < static_cast<double>(p.top_p))) ? 1 : 0;
    prob[tid] = tid < keep ? pi / kept_total : 0.0;
    // ---- the kept tokens in token-id order: sort (index, probability) ascending by index; dropped slots go last
    if (tid >= keep) cand_idx[tid] = 0xffffffffu;
    __syncthreads();
    for (uint32_t size = 2; size <= kSampleMaxCandidates; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            const uint32_t partner = tid ^ stride;
            if (partner > tid) {
                const bool up = (tid & size) == 0;
                const uint32_t ia = cand_idx[tid], ib = cand_idx[partner];
                if ((ib < ia) == up) {
                    const double pa = prob[tid], pb = prob[partner];
                    cand_idx[tid] = ib; cand_idx[partner] = ia; prob[tid] = pb; prob[partner] = pa;
                }
            }
            __syncthreads();
        }
    }
    // ---- draw: the first kept token (ascending id) whose cumulative probability reaches u
    scan[tid] = prob[tid];
    __syncthreads();
    for (uint32_t off = 1; off < kSampleMaxCandidates; off <<= 1) {
        const double add = tid >= off ? scan[tid - off] : 0.0;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
    }
    if (tid == 0) s_count = keep - 1;    // rounding may leave the last cumulative sum a hair below u: then the last kept token
    __syncthreads();
    if (tid < keep && scan[tid] >= p.u && !(tid && scan[tid - 1] >= p.u)) s_count = tid;
    __syncthreads();
    if (tid == 0) {
        *p.pick = static_cast<long long>(cand_idx[s_count]);
        if (p.kept_count) *p.kept_count = static_cast<int>(keep);
    }
    if (p.kept_ids && tid < keep) p.kept_ids[tid] = static_cast<int>(cand_idx[tid]);
    if (p.kept_probs && tid < keep) p.kept_probs[tid] = prob[tid];
}

}  // namespace zk
