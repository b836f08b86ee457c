// zen/cuda_backend.h -- the B200 backend in the shape ZenInfer binds its GPU backends: free functions in a namespace,
// plain scalar/pointer signatures, no vendor header in sight (the rule of include/zen/hip_backend.h:8-13).  Every function
// forwards to the C-ABI of libzen_cuda.so (zen_cuda.h).  Same surface as zen::hip (include/zen/hip_backend.h:46-83) plus the
// Q6_K / Q4_0 / K-quant / release entry points of zen::d3d12 (include/zen/d3d12_backend.h:75-97,169).
//
// This backend has no CPU route behind it: where zen::hip returns false to let the caller try its next route, a false here
// is a failed call, and zen::cuda::last_error() says why.
#pragma once
#include <cstddef>
#include <cstdint>

#include "../zen_cuda.h"

namespace zen::cuda {
using AdapterInfo = zen_cuda_adapter_info;
using Stats = zen_cuda_stats;
using GemvTask = zen_cuda_gemv_task;   // {weights, y, rows, columns}: zen::hip::GemvTask
using GemmTask = zen_cuda_gemm_task;   // {weights, y, rows}: zen::d3d12::GemmTask
constexpr std::size_t kMaxBatch = ZEN_CUDA_MAX_BATCH;

inline bool enabled() noexcept { return zen_cuda_enabled() != 0; }
inline bool init() noexcept { return zen_cuda_init() != 0; }
inline void shutdown() noexcept { zen_cuda_shutdown(); }
inline bool info(AdapterInfo& out) noexcept { return zen_cuda_info(&out) != 0; }
inline Stats stats() noexcept { Stats s{}; zen_cuda_get_stats(&s); return s; }
inline const char* last_error() noexcept { return zen_cuda_last_error(); }

inline bool gemv_q8_0(const std::uint8_t* w, const float* x, float* y, std::size_t rows, std::size_t cols) noexcept {
    return zen_cuda_gemv_q8_0(w, x, y, rows, cols) != 0;
}
inline bool gemm_q8_0(const std::uint8_t* w, const float* in, float* out, std::size_t tokens, std::size_t rows, std::size_t cols) noexcept {
    return zen_cuda_gemm_q8_0(w, in, out, tokens, rows, cols) != 0;
}
inline bool gemv_q8_0_batch(const float* x, const GemvTask* tasks, std::size_t count) noexcept { return zen_cuda_gemv_q8_0_batch(x, tasks, count) != 0; }
inline bool gemm_q8_0_batch(const float* x, const GemmTask* tasks, std::size_t count, std::size_t tokens, std::size_t cols) noexcept {
    return zen_cuda_gemm_q8_0_batch(x, tasks, count, tokens, cols) != 0;
}
inline bool gemm_q6_k(const std::uint8_t* w, const float* in, float* out, std::size_t tokens, std::size_t rows, std::size_t cols) noexcept {
    return zen_cuda_gemm_q6_k(w, in, out, tokens, rows, cols) != 0;
}
inline bool gemm_q4_0(const std::uint8_t* w, const float* in, float* out, std::size_t tokens, std::size_t rows, std::size_t cols) noexcept {
    return zen_cuda_gemm_q4_0(w, in, out, tokens, rows, cols) != 0;
}
inline bool gemm_kquant(const std::uint8_t* w, const float* in, float* out, std::size_t tokens, std::size_t rows, std::size_t cols, bool q5) noexcept {
    return zen_cuda_gemm_kquant(w, in, out, tokens, rows, cols, q5 ? 1 : 0) != 0;
}
inline bool rms_norm(const float* x, const float* weight, float* y, std::size_t rows, std::size_t cols, float epsilon) noexcept {
    return zen_cuda_rms_norm(x, weight, y, rows, cols, epsilon) != 0;
}
inline bool gemv_q8_0_ffn(const std::uint8_t* gate, const std::uint8_t* up, const std::uint8_t* down, const float* x, float* y,
                          std::size_t ffn_rows, std::size_t cols, std::size_t out_rows) noexcept {
    return zen_cuda_gemv_q8_0_ffn(gate, up, down, x, y, ffn_rows, cols, out_rows) != 0;
}
inline void release_weights(const std::uint8_t* w) noexcept { zen_cuda_release_weights(w); }
}  // namespace zen::cuda
