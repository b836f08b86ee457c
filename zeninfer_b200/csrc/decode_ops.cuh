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
// weight == nullptr: only the residual add.
__global__ void __launch_bounds__(256) residual_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ weight,
                                                                float* __restrict__ y, uint32_t n, float eps) {
    __shared__ double scratch[8];
    pdl_launch_dependents();
    pdl_wait();
    float* xr = x + static_cast<size_t>(blockIdx.x) * n;
    const float* dr = delta ? delta + static_cast<size_t>(blockIdx.x) * n : nullptr;
    float* yr = y ? y + static_cast<size_t>(blockIdx.x) * n : nullptr;
    double ss = 0.0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        if (dr) { v += dr[i]; xr[i] = v; }
        ss += static_cast<double>(v) * v;
    }
    if (!weight) return;
    const double total = block_sum_double(ss, scratch);
    const float inv = 1.0f / sqrtf(static_cast<float>(total / n) + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = xr[i] * inv * weight[i];
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

// Grouped-query attention for one new token: one CTA per query head (four warps).  Warps take positions in turn
// and compute q . k[t] with four dimensions per lane; scores wait in shared memory; after the max and the
// denominator (double) thread d accumulates out[d] = sum_t a[t] * v[t][d] over coalesced rows of V.
// D must be a multiple of 4 and at most 4 * 32 * 2; scores for up to `max_positions` fit the dynamic shared memory.
constexpr int kAttnThreads = 128;
__global__ void __launch_bounds__(kAttnThreads) attention_decode_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                          const float* __restrict__ v_cache, const int* __restrict__ pos_ptr,
                                                                          float* __restrict__ out, uint32_t heads, uint32_t kv_heads, uint32_t D, float scale,
                                                                          uint32_t window, uint32_t max_positions, int* error_word) {
    extern __shared__ float scores[];
    __shared__ float red[kAttnThreads / 32];
    __shared__ double scratch[8];
    pdl_launch_dependents();
    pdl_wait();
    const int pos = *pos_ptr;
    if (pos < 0 || static_cast<uint32_t>(pos) >= max_positions) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(error_word, kErrBadPosition);
        return;
    }
    const uint32_t h = blockIdx.x, kh = h / (heads / kv_heads), kw = kv_heads * D;
    const uint32_t first = (window && static_cast<uint32_t>(pos) + 1 > window) ? static_cast<uint32_t>(pos) + 1 - window : 0u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* qh = q + static_cast<size_t>(h) * D;
    // q for this lane: dimensions 4 * lane + {0..3} (+ 128 when D > 128)
    float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
    if (4u * lane < D) q0 = *reinterpret_cast<const float4*>(qh + 4 * lane);
    if (128u + 4u * lane < D) q1 = *reinterpret_cast<const float4*>(qh + 128 + 4 * lane);
    float local_max = -INFINITY;
    for (uint32_t t = first + warp; t <= static_cast<uint32_t>(pos); t += kAttnThreads / 32) {
        const float* kt = k_cache + static_cast<size_t>(t) * kw + static_cast<size_t>(kh) * D;
        float acc = 0.0f;
        if (4u * lane < D) {
            const float4 kk = *reinterpret_cast<const float4*>(kt + 4 * lane);
            acc = q0.x * kk.x + q0.y * kk.y + q0.z * kk.z + q0.w * kk.w;
        }
        if (128u + 4u * lane < D) {
            const float4 kk = *reinterpret_cast<const float4*>(kt + 128 + 4 * lane);
            acc += q1.x * kk.x + q1.y * kk.y + q1.z * kk.z + q1.w * kk.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        const float sc = acc * scale;
        if (lane == 0) scores[t - first] = sc;
        local_max = fmaxf(local_max, sc);
    }
    if (lane == 0) red[warp] = local_max;
    __syncthreads();
    float max_score = red[0];
#pragma unroll
    for (int w = 1; w < kAttnThreads / 32; ++w) max_score = fmaxf(max_score, red[w]);
    const uint32_t count = static_cast<uint32_t>(pos) + 1 - first;
    double part = 0.0;
    for (uint32_t i = threadIdx.x; i < count; i += kAttnThreads) {
        const float e = expf(scores[i] - max_score);
        scores[i] = e;
        part += e;
    }
    const double denom = block_sum_double(part, scratch);   // also orders the score writes before the reads below
    if (!(denom > 0.0) || !isfinite(denom)) {
        if (threadIdx.x == 0) atomicExch(error_word, kErrNonFinite);
        return;
    }
    const float inv = 1.0f / static_cast<float>(denom);
    for (uint32_t d = threadIdx.x; d < D; d += kAttnThreads) {
        const float* vcol = v_cache + static_cast<size_t>(first) * kw + static_cast<size_t>(kh) * D + d;
        float acc = 0.0f;
        for (uint32_t i = 0; i < count; ++i) acc += (scores[i] * inv) * vcol[static_cast<size_t>(i) * kw];
        out[static_cast<size_t>(h) * D + d] = acc;
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
