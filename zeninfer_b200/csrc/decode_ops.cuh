// The decode-step operators that sit between the quantised projections of a dense Llama-style layer, so that a
// whole token step stays in HBM on one stream: embedding row fetch, RMSNorm (with the residual add fused in),
// rotary embedding + KV-cache append, grouped-query attention over an fp32 KV cache, SwiGLU.
//
// Each follows the arithmetic of the reference's host loop in DenseTransformerRuntime::forward
// (src/adapters/dense_transformer_runtime.cpp): rms_norm :117-125 (sum of squares in double), rope :300-329 with
// the host-built cos/sin table contract of rope_table :264-276 (the device never computes an angle), the attention
// block :4284-4337 (scores * 1/sqrt(D), max-subtracted exp, denominator summed in double, a = score * (1/denominator),
// out += a * v), silu_mul :193-199.  The position of the token in flight is read from device memory, so one captured
// launch sequence serves every step.
//
// Every kernel here is launched with programmatic stream serialisation: it lets the next launch start at once (the
// projection kernels stream their weights before they need this kernel's output) and waits for the previous grid
// before it touches memory.  Each grid waits for its predecessor before it can finish, so completion is transitive
// along the stream.
#pragma once
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "zk_ptx.cuh"

namespace zk {

// x[e] = code[token][e] * d[token][e / 32]: one row of a resident Q8_0 tensor as fp32 (the reference decodes the
// embedding row with its Q8_0 decoder, src/quant.cpp:410-416).  A token id outside [0, rows) yields a zero row and
// sets the error word.
__global__ void embed_row_q8_0_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, uint32_t rows, uint32_t K, uint32_t nbp,
                                      const long long* __restrict__ token, float* __restrict__ out, int* error_word) {
    pdl_launch_dependents();
    pdl_wait();
    const long long id = *token;
    const bool ok = id >= 0 && id < static_cast<long long>(rows);
    if (!ok && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(error_word, kErrBadToken);
    for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < K; e += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (ok) v = static_cast<float>(codes[static_cast<size_t>(id) * K + e]) * __half2float(scales[static_cast<size_t>(id) * nbp + (e >> 5)]);
        out[e] = v;
    }
}

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < nwarp; ++w) total += scratch[w];   // same order in every thread
    __syncthreads();
    return total;
}

// One CTA per row.  If `delta` is given the row is first updated in place, x += delta (the residual add that
// precedes every norm but the first), then y = x * inv * weight with inv = 1 / sqrt(float(sum x^2 / n) + eps).
// weight == nullptr: only the residual add.  Rows whose length is a multiple of four move as 16-byte words, one or a
// few per thread, so a 4096-wide row is two short round trips to L2.
constexpr int kNormThreads = 1024;
__global__ void __launch_bounds__(kNormThreads) residual_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                                         const float* __restrict__ weight, float* __restrict__ y, uint32_t n, float eps) {
    __shared__ double scratch[kNormThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    float* xr = x + static_cast<size_t>(blockIdx.x) * n;
    const float* dr = delta ? delta + static_cast<size_t>(blockIdx.x) * n : nullptr;
    float* yr = y ? y + static_cast<size_t>(blockIdx.x) * n : nullptr;
    const bool vec = (n & 3u) == 0;
    double ss = 0.0;
    if (vec) {
        for (uint32_t i = threadIdx.x; i < n / 4; i += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(xr)[i];
            if (dr) {
                const float4 dl = reinterpret_cast<const float4*>(dr)[i];
                v.x += dl.x; v.y += dl.y; v.z += dl.z; v.w += dl.w;
                reinterpret_cast<float4*>(xr)[i] = v;
            }
            ss += static_cast<double>(v.x) * v.x + static_cast<double>(v.y) * v.y + static_cast<double>(v.z) * v.z + static_cast<double>(v.w) * v.w;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
            float v = xr[i];
            if (dr) { v += dr[i]; xr[i] = v; }
            ss += static_cast<double>(v) * v;
        }
    }
    if (!weight) return;
    const double total = block_sum_double(ss, scratch);
    const float inv = 1.0f / sqrtf(static_cast<float>(total / n) + eps);
    if (vec) {
        for (uint32_t i = threadIdx.x; i < n / 4; i += blockDim.x) {   // a thread re-reads what it wrote itself
            const float4 v = reinterpret_cast<const float4*>(xr)[i], w = reinterpret_cast<const float4*>(weight)[i];
            reinterpret_cast<float4*>(yr)[i] = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = xr[i] * inv * weight[i];
    }
}

// Rotates q (heads x D) and k (kv_heads x D) in place with the cos/sin row of the current position, then appends k
// and v to the layer's cache at that position.  Table: [positions][pairs]; adjacent: pairs (x[2i], x[2i+1]), else
// (x[i], x[i + pairs]).  Dimensions past 2 * pairs are left alone.  ONE CTA (the append follows the rotation behind a
// block barrier); a thread takes (head, pair) items in turn.
__global__ void __launch_bounds__(1024) rope_kv_append_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v,
                                                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                              const int* __restrict__ pos_ptr, uint32_t heads, uint32_t kv_heads, uint32_t D, uint32_t pairs,
                                                              int adjacent, float* __restrict__ k_cache, float* __restrict__ v_cache, uint32_t max_positions,
                                                              int* error_word) {
    pdl_launch_dependents();
    pdl_wait();
    const int pos = *pos_ptr;
    if (pos < 0 || static_cast<uint32_t>(pos) >= max_positions) {
        if (threadIdx.x == 0) atomicExch(error_word, kErrBadPosition);
        return;
    }
    const uint32_t kw = kv_heads * D;
    const uint32_t total = (heads + kv_heads) * pairs;
    const float* c = cos_t + static_cast<size_t>(pos) * pairs;
    const float* s = sin_t + static_cast<size_t>(pos) * pairs;
    for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
        const uint32_t h = i / pairs, pr = i % pairs;
        float* vec = h < heads ? q + static_cast<size_t>(h) * D : k + static_cast<size_t>(h - heads) * D;
        const uint32_t ia = adjacent ? 2 * pr : pr, ib = adjacent ? 2 * pr + 1 : pr + pairs;
        const float a = vec[ia], b = vec[ib], cc = c[pr], sn = s[pr];
        vec[ia] = a * cc - b * sn;
        vec[ib] = a * sn + b * cc;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kw; i += blockDim.x) {
        k_cache[static_cast<size_t>(pos) * kw + i] = k[i];
        v_cache[static_cast<size_t>(pos) * kw + i] = v[i];
    }
}

// Grouped-query attention for one new token.  A cluster of kAttnSplit CTAs serves one query head: CTA `rank` takes
// positions first + rank, first + rank + kAttnSplit, ...; inside a CTA a warp takes a position at a time, four dimensions
// per lane, kAttnUnroll positions in flight.  At a few hundred positions the kernel is bound by memory latency, not
// bandwidth, so it is built to pay as few dependent round trips as possible: the key AND value rows of a warp's
// positions are requested together, and every warp keeps a running maximum m, denominator l and output accumulator
// (the streaming form of the softmax: when a new maximum arrives, l and the accumulator are rescaled by
// exp(m_old - m_new)), so nothing waits for a block-wide maximum between the keys and the values.  Eight warps x four
// positions x eight CTAs cover 256 positions per round (kWide: head dimensions above 128, eight floats per lane).
// Resources are part of the design: the kernel runs between two projection launches that overlap with it, so a CTA
// stays at 256 threads and at most 85 registers.  Measured inside a Llama-3-8B layer at position 575: 8.5 us with four
// positions per warp and 85 registers; 11.2 us with eight positions and 128 registers although that version is the
// faster one when timed alone (6.8 against 8.6 us); 512 threads ran the clusters in two waves (19 us); builds that
// spill to reach 48 or 64 registers lose more than they gain.  The warps' (m, l, accumulator) are merged in shared memory,
// rank 0 merges the CTAs' shares through distributed shared memory:
// out = sum_r w_r out_r / sum_r w_r l_r with w_r = exp(m_r - max m), which is exp(score - max) / denominator applied
// to v, the reference's formula (src/adapters/dense_transformer_runtime.cpp:4284-4337); denominators are kept in double as there.
// D must be a multiple of 4 and at most 256.
constexpr int kAttnThreads = 256;
constexpr int kAttnSplit = 8;
constexpr int kAttnMaxD = 256;

struct AttnShare {          // one CTA's contribution, read by rank 0 of the cluster
    float out[kAttnMaxD];
    float max_score;
    double sum;
};

// One rotation of an adjacent pair, with every product and the sum rounded on its own as in the reference's scalar
// loop (a fused multiply-add here would make a cached key differ in the last bit from the one used in its own step).
__device__ __forceinline__ void rope_pair(float& a, float& b, float c, float s) {
    const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    a = ra; b = rb;
}
// dimensions base .. base+3 of a head vector: pairs base/2 and base/2 + 1 (adjacent pairing)
__device__ __forceinline__ void rope_quad(float4& v, uint32_t base, uint32_t pairs, const float* __restrict__ c, const float* __restrict__ s) {
    const uint32_t pr = base >> 1;
    if (pr < pairs) rope_pair(v.x, v.y, c[pr], s[pr]);
    if (pr + 1 < pairs) rope_pair(v.z, v.w, c[pr + 1], s[pr + 1]);
}

// kFused: q, k_new, v_new are the raw projections of the token in flight; the kernel applies the adjacent-pair rotary
// embedding (host-built table rows of *pos_ptr) to q and k_new in registers, attends to the cache for earlier
// positions and to k_new / v_new for the current one, and the cluster of each KV group's first query head appends the
// rotated key and the value to the caches.  This is the reference's attention_block contract
// (include/zen/d3d12_backend.h:247).  Other clusters never read the cache at the current position, so the append
// races with nothing.
template <bool kFused, bool kWide>
__global__ void __cluster_dims__(kAttnSplit, 1, 1) __launch_bounds__(kAttnThreads, kWide ? 2 : 3)
    attention_decode_kernel(const float* __restrict__ q, const float* __restrict__ k_cache_in, const float* __restrict__ v_cache_in,
                            const int* __restrict__ pos_ptr, float* __restrict__ out, uint32_t heads, uint32_t kv_heads, uint32_t D, float scale,
                            uint32_t window, uint32_t max_positions, int* error_word, const float* __restrict__ k_new, const float* __restrict__ v_new,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, uint32_t pairs, float* k_cache_out, float* v_cache_out) {
    const float* k_cache = kFused ? k_cache_out : k_cache_in;   // fused: the caches are also written here, so no read-only promise
    const float* v_cache = kFused ? v_cache_out : v_cache_in;
    namespace cg = cooperative_groups;
    constexpr int kWarps = kAttnThreads / 32, kAttnUnroll = 4;
    __shared__ AttnShare share;
    __shared__ __align__(16) float partial[kWarps * kAttnMaxD];   // [warp][dimension]: the warps' accumulators
    __shared__ float warp_max[kWarps];
    __shared__ double warp_sum[kWarps];
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t h = blockIdx.y, kh = h / (heads / kv_heads), kw = kv_heads * D;
    const bool lo_on = 4u * lane < D, hi_on = kWide && 128u + 4u * lane < D;   // !kWide: the compiler drops the upper halves
    pdl_launch_dependents();
    pdl_wait();
    // the first round trip: the position, and beside it everything whose address does not depend on it
    const int pos = *pos_ptr;
    const float* qh = q + static_cast<size_t>(h) * D;
    float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
    if (lo_on) q0 = __ldcg(reinterpret_cast<const float4*>(qh + 4 * lane));      // q, k_new, v_new: written by the launch before this one
    if (hi_on) q1 = __ldcg(reinterpret_cast<const float4*>(qh + 128 + 4 * lane));
    const float* knew = kFused ? k_new + static_cast<size_t>(kh) * D : nullptr;
    const float* vnew = kFused ? v_new + static_cast<size_t>(kh) * D : nullptr;
    float4 kn0 = make_float4(0.f, 0.f, 0.f, 0.f), kn1 = kn0, vn0 = kn0, vn1 = kn0;   // the token in flight, every warp's copy
    if (kFused) {
        if (lo_on) { kn0 = __ldcg(reinterpret_cast<const float4*>(knew + 4 * lane)); vn0 = __ldcg(reinterpret_cast<const float4*>(vnew + 4 * lane)); }
        if (hi_on) { kn1 = __ldcg(reinterpret_cast<const float4*>(knew + 128 + 4 * lane)); vn1 = __ldcg(reinterpret_cast<const float4*>(vnew + 128 + 4 * lane)); }
    }
    const bool bad = pos < 0 || static_cast<uint32_t>(pos) >= max_positions;
    if (bad && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicExch(error_word, kErrBadPosition);
    const uint32_t first = (window && static_cast<uint32_t>(pos) + 1 > window) ? static_cast<uint32_t>(pos) + 1 - window : 0u;
    const uint32_t count = bad ? 0u : static_cast<uint32_t>(pos) + 1 - first;                 // positions attended by the head
    const uint32_t mine = count > rank ? (count - rank + kAttnSplit - 1) / kAttnSplit : 0u;   // ... by this CTA
    const float* kbase = k_cache + static_cast<size_t>(first + rank) * kw + static_cast<size_t>(kh) * D;
    const float* vbase = v_cache + static_cast<size_t>(first + rank) * kw + static_cast<size_t>(kh) * D;
    const size_t step = static_cast<size_t>(kAttnSplit) * kw;     // floats between this CTA's consecutive positions
    const uint32_t last = count ? count - 1 : 0;                  // index of the current position among the attended ones

    float run_max = -INFINITY;
    double run_sum = 0.0;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    bool rotated = false;
    for (uint32_t i0 = warp; i0 < mine; i0 += kWarps * kAttnUnroll) {
        // the second round trip: keys and values of this round's positions together (and, the first time, the cos/sin row)
        float4 ka[kAttnUnroll], kb[kAttnUnroll], va[kAttnUnroll], vb[kAttnUnroll];
        bool fresh[kAttnUnroll];
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) {
            const uint32_t i = i0 + u * kWarps;
            ka[u] = kb[u] = va[u] = vb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            fresh[u] = kFused && i < mine && rank + i * kAttnSplit == last;     // the token in flight: not in the cache yet
            if (i < mine && !fresh[u]) {
                const float* kt = kbase + static_cast<size_t>(i) * step;
                const float* vt = vbase + static_cast<size_t>(i) * step;
                if (lo_on) { ka[u] = __ldcg(reinterpret_cast<const float4*>(kt + 4 * lane)); va[u] = __ldcg(reinterpret_cast<const float4*>(vt + 4 * lane)); }
                if (hi_on) { kb[u] = __ldcg(reinterpret_cast<const float4*>(kt + 128 + 4 * lane)); vb[u] = __ldcg(reinterpret_cast<const float4*>(vt + 128 + 4 * lane)); }
            }
        }
        if (kFused && !rotated && !bad) {   // rotate q and the new key once (table rows of the current position)
            const float* cs = cos_t + static_cast<size_t>(pos) * pairs;
            const float* sn = sin_t + static_cast<size_t>(pos) * pairs;
            if (lo_on) { rope_quad(q0, 4u * lane, pairs, cs, sn); rope_quad(kn0, 4u * lane, pairs, cs, sn); }
            if (hi_on) { rope_quad(q1, 128u + 4u * lane, pairs, cs, sn); rope_quad(kn1, 128u + 4u * lane, pairs, cs, sn); }
            rotated = true;
        }
        float sc[kAttnUnroll];
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) {
            if (fresh[u]) { ka[u] = kn0; kb[u] = kn1; va[u] = vn0; vb[u] = vn1; }
            float acc = q0.x * ka[u].x + q0.y * ka[u].y + q0.z * ka[u].z + q0.w * ka[u].w + q1.x * kb[u].x + q1.y * kb[u].y + q1.z * kb[u].z + q1.w * kb[u].w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            sc[u] = i0 + u * kWarps < mine ? acc * scale : -INFINITY;
        }
        float new_max = run_max;
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) new_max = fmaxf(new_max, sc[u]);
        // i0 < mine, so at least sc[0] is a real score; a non-finite maximum (NaN or +inf scores) is caught by the final check
        const float corr = run_max == -INFINITY ? 0.0f : expf(run_max - new_max);
        a0.x *= corr; a0.y *= corr; a0.z *= corr; a0.w *= corr;
        a1.x *= corr; a1.y *= corr; a1.z *= corr; a1.w *= corr;
        double add = 0.0;
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) {
            const float e = sc[u] == -INFINITY ? 0.0f : expf(sc[u] - new_max);
            add += e;
            a0.x += e * va[u].x; a0.y += e * va[u].y; a0.z += e * va[u].z; a0.w += e * va[u].w;
            a1.x += e * vb[u].x; a1.y += e * vb[u].y; a1.z += e * vb[u].z; a1.w += e * vb[u].w;
        }
        run_sum = run_sum * static_cast<double>(corr) + add;
        run_max = new_max;
    }
    // append: the cluster of the KV group's first query head, the CTA that owns the current position
    if (kFused && !bad && h % (heads / kv_heads) == 0 && rank == last % kAttnSplit && threadIdx.x < D) {
        const float* cs = cos_t + static_cast<size_t>(pos) * pairs;
        const float* sn = sin_t + static_cast<size_t>(pos) * pairs;
        const uint32_t dd = threadIdx.x, pr = dd >> 1;
        float a = __ldcg(knew + (dd & ~1u)), b = __ldcg(knew + (dd | 1u));
        if (pr < pairs) rope_pair(a, b, cs[pr], sn[pr]);
        k_cache_out[static_cast<size_t>(pos) * kw + static_cast<size_t>(kh) * D + dd] = (dd & 1u) ? b : a;
        v_cache_out[static_cast<size_t>(pos) * kw + static_cast<size_t>(kh) * D + dd] = __ldcg(vnew + dd);
    }
    // merge the warps: this CTA's (maximum, denominator, output share)
    if (lo_on) *reinterpret_cast<float4*>(&partial[warp * kAttnMaxD + 4 * lane]) = a0;
    if (hi_on) *reinterpret_cast<float4*>(&partial[warp * kAttnMaxD + 128 + 4 * lane]) = a1;
    if (lane == 0) { warp_max[warp] = run_max; warp_sum[warp] = run_sum; }
    __syncthreads();
    float cta_max = warp_max[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) cta_max = fmaxf(cta_max, warp_max[w]);
    if (threadIdx.x < D) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float wm = warp_max[w];
            if (wm != -INFINITY) total += expf(wm - cta_max) * partial[w * kAttnMaxD + threadIdx.x];
        }
        share.out[threadIdx.x] = total;
    }
    if (threadIdx.x == 0) {
        double sum = 0.0;
        for (int w = 0; w < kWarps; ++w)
            if (warp_max[w] != -INFINITY) sum += static_cast<double>(expf(warp_max[w] - cta_max)) * warp_sum[w];
        share.max_score = cta_max;
        share.sum = sum;
    }
    cluster.sync();                                   // every CTA's share is complete and visible
    if (rank == 0 && !bad) {
        float m = -INFINITY;
        for (uint32_t r = 0; r < kAttnSplit; ++r) m = fmaxf(m, cluster.map_shared_rank(&share, r)->max_score);
        double denom = 0.0;
        float w[kAttnSplit];
        for (uint32_t r = 0; r < kAttnSplit; ++r) {
            const AttnShare* sh = cluster.map_shared_rank(&share, r);
            w[r] = sh->max_score == -INFINITY ? 0.0f : expf(sh->max_score - m);   // a CTA without positions contributes nothing
            denom += static_cast<double>(w[r]) * sh->sum;
        }
        if (!(denom > 0.0) || !isfinite(denom)) {
            if (threadIdx.x == 0) atomicExch(error_word, kErrNonFinite);
        } else if (threadIdx.x < D) {
            const float inv = 1.0f / static_cast<float>(denom);
            float total = 0.0f;
            for (uint32_t r = 0; r < kAttnSplit; ++r) total += w[r] * cluster.map_shared_rank(&share, r)->out[threadIdx.x];
            out[static_cast<size_t>(h) * D + threadIdx.x] = total * inv;
        }
    }
    cluster.sync();                                   // nobody leaves while rank 0 still reads its shared memory
}

// ---- prefill: the same operators over a block of T tokens at positions pos0 .. pos0 + T - 1 ------------------------------
// (DenseTransformerRuntime::forward_batch, src/adapters/dense_transformer_runtime.cpp:2296-3664: embedding gather
// :2315-2319, rope tables once :2380-2398, then per layer norm rows, batched projections, rope, attention, FFN.)

// out[t][e] = row tokens[t] of a resident Q8_0 tensor; grid (ceil(K / 256), T).
__global__ void embed_rows_q8_0_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, uint32_t rows, uint32_t K, uint32_t nbp,
                                       const long long* __restrict__ tokens, float* __restrict__ out, int* error_word) {
    pdl_launch_dependents();
    pdl_wait();
    const long long id = tokens[blockIdx.y];
    const bool ok = id >= 0 && id < static_cast<long long>(rows);
    if (!ok && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(error_word, kErrBadToken);
    const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= K) return;
    float v = 0.0f;
    if (ok) v = static_cast<float>(codes[static_cast<size_t>(id) * K + e]) * __half2float(scales[static_cast<size_t>(id) * nbp + (e >> 5)]);
    out[static_cast<size_t>(blockIdx.y) * K + e] = v;
}

// One CTA per token: rotate q [T][heads*D] and k [T][kv_heads*D] in place (adjacent pairs, or half-split) with the
// table row of position *pos_ptr + t, then append k and v to the caches there.
__global__ void __launch_bounds__(1024) rope_kv_append_rows_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v,
                                                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                                   const int* __restrict__ pos_ptr, uint32_t heads, uint32_t kv_heads, uint32_t D,
                                                                   uint32_t pairs, int adjacent, float* __restrict__ k_cache, float* __restrict__ v_cache,
                                                                   uint32_t max_positions, int* error_word) {
    pdl_launch_dependents();
    pdl_wait();
    const long long pos = static_cast<long long>(*pos_ptr) + blockIdx.x;
    if (pos < 0 || pos >= static_cast<long long>(max_positions)) {
        if (threadIdx.x == 0) atomicExch(error_word, kErrBadPosition);
        return;
    }
    const uint32_t kw = kv_heads * D, qw = heads * D;
    float* qt = q + static_cast<size_t>(blockIdx.x) * qw;
    float* kt = k + static_cast<size_t>(blockIdx.x) * kw;
    const float* vt = v + static_cast<size_t>(blockIdx.x) * kw;
    const float* c = cos_t + static_cast<size_t>(pos) * pairs;
    const float* s = sin_t + static_cast<size_t>(pos) * pairs;
    for (uint32_t i = threadIdx.x; i < (heads + kv_heads) * pairs; i += blockDim.x) {
        const uint32_t h = i / pairs, pr = i % pairs;
        float* vec = h < heads ? qt + static_cast<size_t>(h) * D : kt + static_cast<size_t>(h - heads) * D;
        const uint32_t ia = adjacent ? 2 * pr : pr, ib = adjacent ? 2 * pr + 1 : pr + pairs;
        float a = vec[ia], b = vec[ib];
        rope_pair(a, b, c[pr], s[pr]);
        vec[ia] = a;
        vec[ib] = b;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kw; i += blockDim.x) {
        k_cache[static_cast<size_t>(pos) * kw + i] = kt[i];
        v_cache[static_cast<size_t>(pos) * kw + i] = vt[i];
    }
}

// Causal grouped-query attention for a block of T new tokens whose keys and values are already in the caches.
// A CTA takes kPfTokens consecutive tokens, one KV head and R query heads of that KV head's group (R = 4, 2 or 1, the
// largest that divides the group and keeps the rows in registers).  A token is held by kPfLanes threads; thread `part`
// owns the float4 columns part, part + kPfLanes, ... of the head and keeps them for all R heads, so a key or value word
// read from shared memory feeds R multiply-adds (shared-memory bandwidth, 128 bytes per clock per SM, bounds this
// kernel otherwise) and the token's threads read consecutive 16-byte words (no bank conflict).  Products and
// accumulations are packed fp32 pairs (fma.rn.f32x2: each half is an IEEE fused multiply-add).  Keys and values come
// through shared memory in blocks of kPfBlock positions; the softmax is the running-maximum form (out and denominator
// rescaled when the maximum moves), which equals the reference's two-pass form up to rounding (attention rows of
// forward_batch, :3041-3570).  Token t attends positions [first, pos0 + t], first = the sliding-window start or 0.
// The grid is one-dimensional and ordered by work: the tiles of the last tokens (the longest key ranges) take the low
// block indices and start first.
#ifndef ZK_PF_STEP
#define ZK_PF_STEP 4
#endif
constexpr int kPfTokens = 16, kPfLanes = 8, kPfBlock = 32, kPfThreads = kPfTokens * kPfLanes, kPfStep = ZK_PF_STEP;
static_assert(kPfBlock % kPfStep == 0, "a round of positions must not straddle two staged blocks");
// 16-byte asynchronous copy global -> shared (bypassing L1); `bytes` = 16, or 0 for a zero fill.
__device__ __forceinline__ void cp_async_16(float* smem_dst, const float* gmem_src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }
__device__ __forceinline__ uint64_t pf_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void pf_unpack(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t pf_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t pf_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// The lane (within a token's kPfLanes) that ends the score reduction with head r's sum and keeps that row's softmax state.
template <int R>
__device__ __forceinline__ constexpr int pf_owner(int r) { return R == 4 ? ((r >> 1) * 4 + (r & 1) * 2) : R == 2 ? r * 4 : 0; }
template <int D, int R>   // head dimension (64, 128 or 256) and query heads per thread: compile-time, so the rows stay in registers
__global__ void __launch_bounds__(kPfThreads) attention_prefill_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                        const float* __restrict__ v_cache, const int* __restrict__ pos_ptr,
                                                                        float* __restrict__ out, uint32_t tokens, uint32_t heads, uint32_t kv_heads,
                                                                        float scale, uint32_t window, uint32_t max_positions, int* error_word) {
    extern __shared__ __align__(16) float kv_smem[];      // two buffers of [2][kPfBlock][D]: keys, then values
    pdl_launch_dependents();
    pdl_wait();
    const int pos0 = *pos_ptr;
    if (pos0 < 0 || static_cast<uint32_t>(pos0) + tokens > max_positions) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(error_word, kErrBadPosition);
        return;
    }
    const uint32_t group = heads / kv_heads, passes = group / R, kw = kv_heads * D, qw = heads * D;
    const uint32_t per_tile = kv_heads * passes, n_tiles = gridDim.x / per_tile;
    const uint32_t tile = n_tiles - 1 - blockIdx.x / per_tile, rem = blockIdx.x % per_tile;
    const uint32_t kh = rem / passes, h0 = kh * group + (rem % passes) * R;      // this CTA's heads: h0 .. h0 + R - 1
    constexpr int per4 = D / (4 * kPfLanes);                          // float4 columns per thread and head
    const uint32_t t0 = tile * kPfTokens;
    const uint32_t t_end = min(tokens, t0 + kPfTokens);
    // the span of positions any token of this CTA attends
    const uint32_t last_pos = static_cast<uint32_t>(pos0) + t_end - 1;
    const uint32_t first_any = (window && static_cast<uint32_t>(pos0) + t0 + 1 > window) ? static_cast<uint32_t>(pos0) + t0 + 1 - window : 0u;
    const uint32_t t = t0 + threadIdx.x / kPfLanes, part = threadIdx.x % kPfLanes;
    const bool live = t < t_end;
    const uint32_t my_last = static_cast<uint32_t>(pos0) + t;
    const uint32_t my_first = (window && my_last + 1 > window) ? my_last + 1 - window : 0u;
    uint64_t q01[R][per4], q23[R][per4], a01[R][per4], a23[R][per4];
    // The softmax state of a row lives in one lane: the score reduction below leaves the token's lane `part` with the
    // full sum of one head (head ((part >> 2) << 1 | ((part >> 1) & 1)) for R == 4, part >> 2 for R == 2), and that lane
    // keeps the row's running maximum and denominator.
    float m = -INFINITY;
    double l = 0.0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int i = 0; i < per4; ++i) { q01[r][i] = q23[r][i] = a01[r][i] = a23[r][i] = pf_pack(0.0f, 0.0f); }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float4* qrow = reinterpret_cast<const float4*>(q + static_cast<size_t>(t) * qw + static_cast<size_t>(h0 + r) * D) + part;
#pragma unroll
            for (int i = 0; i < per4; ++i) {
                const float4 v = qrow[i * kPfLanes];
                q01[r][i] = pf_pack(v.x, v.y);
                q23[r][i] = pf_pack(v.z, v.w);
            }
        }
    }
    // Blocks of kPfBlock positions go through two shared-memory buffers: the asynchronous copies of block b + 1 are in
    // flight while block b is consumed.  Rows past last_pos are filled with zeros (a copy of source size 0).
    auto stage = [&](uint32_t p0, uint32_t buf) {
        float* kd = kv_smem + buf * (2 * kPfBlock * D);
        float* vd = kd + kPfBlock * D;
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < kPfBlock * D / 4; i += kPfThreads) {
            const uint32_t row = i / (D / 4), col = i % (D / 4), pos = min(p0 + row, last_pos);
            const uint32_t bytes = p0 + row <= last_pos ? 16u : 0u;
            const size_t off = static_cast<size_t>(pos) * kw + static_cast<size_t>(kh) * D + col * 4;
            cp_async_16(kd + i * 4, k_cache + off, bytes);
            cp_async_16(vd + i * 4, v_cache + off, bytes);
        }
        cp_async_commit();
    };
    stage(first_any, 0);
    uint32_t buf = 0;
    for (uint32_t p0 = first_any; p0 <= last_pos; p0 += kPfBlock, buf ^= 1u) {
        const bool more = p0 + kPfBlock <= last_pos;
        if (more) stage(p0 + kPfBlock, buf ^ 1u);       // its buffer was read during the previous block, which ended with a barrier
        if (more) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        const float* ks = kv_smem + buf * (2 * kPfBlock * D);
        const float* vs = ks + kPfBlock * D;
        const uint32_t j_end = min(static_cast<uint32_t>(kPfBlock), last_pos - p0 + 1);
        // kPfStep positions per round: their score chains, reductions and exponentials are independent of one another, which
        // is what hides the arithmetic and shuffle latencies at the two or three warps per scheduler the row registers allow.
        // Rows of the staged block past last_pos are zeros and fall outside every token's range.
        for (uint32_t j = 0; j < j_end; j += kPfStep) {
            bool in_range[kPfStep];
            bool any = false;
#pragma unroll
            for (int u = 0; u < kPfStep; ++u) {
                const uint32_t pos = p0 + j + u;
                in_range[u] = live && pos >= my_first && pos <= my_last;      // uniform over the token's kPfLanes threads
                any |= in_range[u];
            }
            if (!__any_sync(0xffffffffu, any)) continue;                          // none of this warp's tokens attends these positions
            const float4* krow = reinterpret_cast<const float4*>(ks + j * D) + part;
            uint64_t d[kPfStep][R];
#pragma unroll
            for (int u = 0; u < kPfStep; ++u) {
#pragma unroll
                for (int r = 0; r < R; ++r) d[u][r] = pf_pack(0.0f, 0.0f);
            }
#pragma unroll
            for (int i = 0; i < per4; ++i) {
#pragma unroll
                for (int u = 0; u < kPfStep; ++u) {
                    const float4 kk = krow[u * (D / 4) + i * kPfLanes];
                    const uint64_t k01 = pf_pack(kk.x, kk.y), k23 = pf_pack(kk.z, kk.w);
#pragma unroll
                    for (int r = 0; r < R; ++r) d[u][r] = pf_fma(q23[r][i], k23, pf_fma(q01[r][i], k01, d[u][r]));
                }
            }
            // Sum over the token's eight lanes, halving the rows a lane carries at each exchange: lane `part` ends with
            // the full score of its head (R + 1 or 3 shuffles, where one reduction per row would take 3 R).
            float sc[kPfStep];
#pragma unroll
            for (int u = 0; u < kPfStep; ++u) {
                float dot[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float d0, d1;
                    pf_unpack(d[u][r], d0, d1);
                    dot[r] = d0 + d1;
                }
                float red;
                if constexpr (R == 4) {
                    const bool hi = part & 4, hi2 = part & 2;
                    float k0 = hi ? dot[2] : dot[0], k1 = hi ? dot[3] : dot[1];
                    k0 += __shfl_xor_sync(0xffffffffu, hi ? dot[0] : dot[2], 4);
                    k1 += __shfl_xor_sync(0xffffffffu, hi ? dot[1] : dot[3], 4);
                    red = (hi2 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, hi2 ? k0 : k1, 2);
                } else if constexpr (R == 2) {
                    const bool hi = part & 4;
                    red = (hi ? dot[1] : dot[0]) + __shfl_xor_sync(0xffffffffu, hi ? dot[0] : dot[1], 4);
                    red += __shfl_xor_sync(0xffffffffu, red, 2);
                } else {
                    red = dot[0] + __shfl_xor_sync(0xffffffffu, dot[0], 4);
                    red += __shfl_xor_sync(0xffffffffu, red, 2);
                }
                red += __shfl_xor_sync(0xffffffffu, red, 1);
                sc[u] = red * scale;
            }
            float m_new = m;
#pragma unroll
            for (int u = 0; u < kPfStep; ++u) m_new = in_range[u] ? fmaxf(m_new, sc[u]) : m_new;
            const bool moved = m_new > m;
            if (__any_sync(0xffffffffu, moved)) {                   // a maximum moves: rescale what has been summed (rare after the first positions)
                const float f = moved ? expf(m - m_new) : 1.0f;     // exp(-inf) = 0 on the first position
                l *= f;
                m = m_new;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float fr = __shfl_sync(0xffffffffu, f, pf_owner<R>(r), kPfLanes);
                    const uint64_t f2 = pf_pack(fr, fr);
#pragma unroll
                    for (int i = 0; i < per4; ++i) { a01[r][i] = pf_mul(a01[r][i], f2); a23[r][i] = pf_mul(a23[r][i], f2); }
                }
            }
            uint64_t e2[kPfStep][R];
            float e_sum = 0.0f;                                         // the round's terms in fp32, one double addition per round
#pragma unroll
            for (int u = 0; u < kPfStep; ++u) {
                const float e = in_range[u] ? expf(sc[u] - m) : 0.0f;   // a token that does not attend the position adds 0 x value
                e_sum += e;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float er = __shfl_sync(0xffffffffu, e, pf_owner<R>(r), kPfLanes);
                    e2[u][r] = pf_pack(er, er);
                }
            }
            l += e_sum;
            const float4* vrow = reinterpret_cast<const float4*>(vs + j * D) + part;
#pragma unroll
            for (int i = 0; i < per4; ++i) {
#pragma unroll
                for (int u = 0; u < kPfStep; ++u) {
                    const float4 vv = vrow[u * (D / 4) + i * kPfLanes];
                    const uint64_t v01 = pf_pack(vv.x, vv.y), v23 = pf_pack(vv.z, vv.w);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        a01[r][i] = pf_fma(e2[u][r], v01, a01[r][i]);
                        a23[r][i] = pf_fma(e2[u][r], v23, a23[r][i]);
                    }
                }
            }
        }
        __syncthreads();                                    // the block's rows are no longer read: the next copies may land in this buffer
    }
    // every lane of the warp takes part in the exchanges below; only live tokens store
    const bool bad = live && (!(l > 0.0) || !isfinite(l));
    const float inv_mine = (live && !bad) ? 1.0f / static_cast<float>(l) : 0.0f;
    if (bad) atomicExch(error_word, kErrNonFinite);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float inv = __shfl_sync(0xffffffffu, inv_mine, pf_owner<R>(r), kPfLanes);
        if (live && inv != 0.0f) {
            float4* orow = reinterpret_cast<float4*>(out + static_cast<size_t>(t) * qw + static_cast<size_t>(h0 + r) * D) + part;
#pragma unroll
            for (int i = 0; i < per4; ++i) {
                float4 o;
                pf_unpack(a01[r][i], o.x, o.y);
                pf_unpack(a23[r][i], o.z, o.w);
                o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
                orow[i * kPfLanes] = o;
            }
        }
    }
}

// out = silu(gate) * up, silu(z) = z / (1 + exp(-z)).
__global__ void silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float z = gate[i];
        out[i] = (z / (1.0f + expf(-z))) * up[i];
    }
}

__global__ void advance_position_kernel(int* pos, int delta) {
    pdl_launch_dependents();
    pdl_wait();
    *pos += delta;
}

}  // namespace zk
