// ref_shim.cpp -- C-ABI doorway into the UNMODIFIED reference, compiled from
// its own sources where they lie (see oracle/Makefile; nothing is copied).
//
// TEST INFRASTRUCTURE ONLY.  libzenref.so exists to (1) validate the plain-C
// restatement in zen_oracle.c bit for bit and (2) time the reference's own
// CPU path beside the GPU numbers.  The product never loads it.
//
// Each wrapper forwards to the reference's public entry point named in its
// comment and adds no arithmetic of its own.
#include "zen/compute_pool.h"
#include "zen/kernels.h"
#include "zen/quant.h"

#include <cstddef>
#include <cstdint>

namespace {
const zen::quant::Format* format_for(int ggml_type) {
    switch (ggml_type) {
    case 8: return zen::quant::find("Q8_0");
    case 2: return zen::quant::find("Q4_0");
    case 14: return zen::quant::find("Q6_K");
    case 12: return zen::quant::find("Q4_K");
    case 13: return zen::quant::find("Q5_K");
    default: return nullptr;
    }
}
}  // namespace

extern "C" {

// zen::quant::row_bytes, include/zen/quant.h:107
std::size_t zr_row_bytes(int fmt, std::size_t columns) {
    const auto* f = format_for(fmt);
    return f ? zen::quant::row_bytes(*f, columns) : 0;
}

// zen::quant::dequantize, include/zen/quant.h:25
int zr_dequantize(int fmt, const std::uint8_t* src, std::size_t n, float* dst) {
    const auto* f = format_for(fmt);
    return f && zen::quant::dequantize(*f, src, n, dst) ? 1 : 0;
}

// zen::quant::encode_fp16 / decode_fp16, include/zen/quant.h:23-24
int zr_encode_fp16(const float* src, std::uint16_t* dst, std::size_t n) { return zen::quant::encode_fp16(src, dst, n) ? 1 : 0; }
int zr_decode_fp16(const std::uint16_t* src, float* dst, std::size_t n) { return zen::quant::decode_fp16(src, dst, n) ? 1 : 0; }

// zen::quant::gemv, include/zen/quant.h:28 (route order src/quant.cpp:963-1163).
// Set ZEN_CPU_Q8_ACT=1 in the environment BEFORE the first call to take the
// int8-activation route; the reference latches that switch on first use.
int zr_gemv(int fmt, const std::uint8_t* w, const float* x, float* y, std::size_t rows, std::size_t cols, unsigned workers) {
    const auto* f = format_for(fmt);
    return f && zen::quant::gemv(*f, w, x, y, rows, cols, 1.0f, workers) ? 1 : 0;
}

// zen::quant::gemm, include/zen/quant.h:32
int zr_gemm(int fmt, const std::uint8_t* w, const float* in, float* out, std::size_t tokens, std::size_t rows,
            std::size_t cols, unsigned workers) {
    const auto* f = format_for(fmt);
    return f && zen::quant::gemm(*f, w, in, out, tokens, rows, cols, 1.0f, workers) ? 1 : 0;
}

// zen::quant::gemv_batch, include/zen/quant.h:84
int zr_gemv_batch(int fmt, const std::uint8_t* const* w, const float* x, float* const* ys, const std::size_t* rows,
                  std::size_t cols, std::size_t count, unsigned workers) {
    const auto* f = format_for(fmt);
    return f && zen::quant::gemv_batch(*f, w, x, ys, rows, cols, count, 1.0f, workers) ? 1 : 0;
}

// zen::gemv_q8_0_avx2 (fp32 activations unless ZEN_CPU_Q8_ACT=1), include/zen/kernels.h:26
int zr_gemv_q8_0_avx2(const std::uint8_t* w, const float* x, float* y, std::size_t rows, std::size_t cols) {
    return zen::gemv_q8_0_avx2(w, x, y, rows, cols) ? 1 : 0;
}

// zen::gemv_q8_0_avx2_int8_prequant, include/zen/kernels.h:63-67
int zr_gemv_q8_0_i8_prequant(const std::uint8_t* w, const std::int8_t* xq, const float* xsc, float* y,
                             std::size_t rows, std::size_t cols) {
    return zen::gemv_q8_0_avx2_int8_prequant(w, xq, xsc, y, rows, cols) ? 1 : 0;
}

// zen::gemv_q6k_avx2, include/zen/kernels.h:56
int zr_gemv_q6k_avx2(const std::uint8_t* w, const float* x, float* y, std::size_t rows, std::size_t cols) {
    return zen::gemv_q6k_avx2(w, x, y, rows, cols) ? 1 : 0;
}

// zen::gemm_q8_0_avx2 / gemm_q8_0_kblk_avx2 / gemm_q6k_kblk_avx2, include/zen/kernels.h:73,85,163
int zr_gemm_q8_0_avx2(const std::uint8_t* w, const float* in, float* out, std::size_t t, std::size_t rows, std::size_t cols) {
    return zen::gemm_q8_0_avx2(w, in, out, t, rows, cols, rows) ? 1 : 0;
}
int zr_gemm_q8_0_kblk_avx2(const std::uint8_t* w, const float* in, float* out, std::size_t t, std::size_t rows, std::size_t cols) {
    return zen::gemm_q8_0_kblk_avx2(w, in, out, t, rows, cols, rows) ? 1 : 0;
}
int zr_gemm_q6k_kblk_avx2(const std::uint8_t* w, const float* in, float* out, std::size_t t, std::size_t rows, std::size_t cols) {
    return zen::gemm_q6k_kblk_avx2(w, in, out, t, rows, cols, rows) ? 1 : 0;
}

// zen::cpu_has_avx2_fma, include/zen/kernels.h:165; ComputePool::worker_count, include/zen/compute_pool.h:13
int zr_cpu_has_avx2_fma() { return zen::cpu_has_avx2_fma() ? 1 : 0; }
unsigned zr_pool_workers() { return zen::ComputePool::instance().worker_count(); }

}  // extern "C"
