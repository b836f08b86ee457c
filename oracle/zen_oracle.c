/*
 * zen_oracle.c -- CPU restatement of ZenInfer's block-quantised GEMV/GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against; nothing in the product path links, loads or calls it.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may load liboracle.
 *
 * Every function restates one reference routine in plain C and names the
 * reference file:line it follows.  Where the reference is AVX2 code, the
 * eight vector lanes are emulated with an explicit float[8] and fmaf(), so
 * that results are bit-identical to the compiled reference (the test-suite
 * checks exactly that against oracle/_ref when it is built).
 *
 * Parity is pinned: the known-answer vectors of the reference's own tests
 * (tests/core_tests.cpp:263-309, tests/q6k_gemm_tests.cpp:16-45,
 * tests/support/quant_fixture.h:12-14) are replayed against this file by
 * tests/test_oracle_golden.py.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ZO_API __attribute__((visibility("default")))

enum { ZO_Q8_0 = 8, ZO_Q4_0 = 2, ZO_Q6_K = 14, ZO_Q4_K = 12, ZO_Q5_K = 13 }; /* GGML type ids */

/* ---- binary16 <-> binary32: src/quant.cpp:80-122 ------------------------ */

ZO_API float zo_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 31u, mant = h & 1023u, out = 0;
    if (exp == 0) {
        if (mant == 0) out = sign;
        else {
            int e = -14;
            while ((mant & 1024u) == 0) { mant <<= 1; --e; }
            mant &= 1023u;
            out = sign | ((uint32_t)(e + 127) << 23) | (mant << 13);
        }
    } else if (exp == 31) out = sign | 0x7f800000u | (mant << 13);
    else out = sign | ((exp + 112u) << 23) | (mant << 13);
    float f; memcpy(&f, &out, 4); return f;
}

static uint32_t rounded_shift(uint32_t x, unsigned shift) {
    if (shift == 0) return x;
    if (shift >= 32) return 0;
    const uint32_t q = x >> shift, mask = ((uint32_t)1 << shift) - 1u;
    const uint32_t rem = x & mask, halfway = (uint32_t)1 << (shift - 1);
    return q + ((rem > halfway || (rem == halfway && (q & 1u))) ? 1u : 0u);
}

ZO_API uint16_t zo_float_to_half(float value) {
    uint32_t bits; memcpy(&bits, &value, 4);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    const uint32_t exp = (bits >> 23) & 0xffu, mant = bits & 0x7fffffu;
    if (exp == 0xffu) {
        if (mant == 0) return (uint16_t)(sign | 0x7c00u);
        uint16_t payload = (uint16_t)(mant >> 13);
        if (payload == 0) payload = 1;
        return (uint16_t)(sign | 0x7c00u | payload);
    }
    if (exp == 0) return sign;
    const int e = (int)exp - 127;
    if (e > 15) return (uint16_t)(sign | 0x7c00u);
    const uint32_t significand = 0x800000u | mant;
    if (e >= -14) {
        uint32_t hm = rounded_shift(mant, 13);
        int he = e + 15;
        if (hm == 0x400u) { hm = 0; ++he; }
        if (he >= 31) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | ((uint16_t)he << 10) | (uint16_t)hm);
    }
    const unsigned shift = (unsigned)(-e - 1);
    return (uint16_t)(sign | (uint16_t)rounded_shift(significand, shift));
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ---- format table rows: src/quant.cpp:253,257,259 and :894-943 ---------- */

ZO_API size_t zo_block_elements(int fmt) {
    return (fmt == ZO_Q6_K || fmt == ZO_Q4_K || fmt == ZO_Q5_K) ? 256 : (fmt == ZO_Q8_0 || fmt == ZO_Q4_0) ? 32 : 0;
}
ZO_API size_t zo_block_bytes(int fmt) {   /* Q4_K, Q5_K: src/quant.cpp:273-274 */
    return fmt == ZO_Q8_0 ? 34 : fmt == ZO_Q4_0 ? 18 : fmt == ZO_Q6_K ? 210 : fmt == ZO_Q4_K ? 144 : fmt == ZO_Q5_K ? 176 : 0;
}

/* The 6-bit scale and minimum of sub-block j (0..7) of a Q4_K / Q5_K super-block, from its 12 packed bytes:
 * src/quant.cpp:133-141. */
static inline void k_scale_min(unsigned j, const uint8_t* q, unsigned* scale, unsigned* min) {
    if (j < 4) {
        *scale = q[j] & 63u;
        *min = q[j + 4] & 63u;
    } else {
        *scale = (q[j + 4] & 15u) | ((unsigned)(q[j - 4] >> 6) << 4);
        *min = (unsigned)(q[j + 4] >> 4) | ((unsigned)(q[j] >> 6) << 4);
    }
}
ZO_API size_t zo_row_bytes(int fmt, size_t columns) {
    const size_t be = zo_block_elements(fmt);
    if (!be || columns % be) return 0;
    return (columns / be) * zo_block_bytes(fmt);
}

/* ---- dequantisers: src/quant.cpp:391-397 (Q4_0), :410-416 (Q8_0),
 *      :500-517 (Q6_K) ---------------------------------------------------- */

ZO_API int zo_dequantize(int fmt, const uint8_t* src, size_t n, float* dst) {
    if (!src || !dst) return 0;
    if (fmt == ZO_Q8_0) {
        if (n % 32) return 0;
        for (size_t b = 0; b < n / 32; ++b) {
            const uint8_t* p = src + b * 34; const float d = zo_half_to_float(rd16(p));
            for (unsigned j = 0; j < 32; ++j) dst[b * 32 + j] = (float)(int8_t)p[2 + j] * d;
        }
        return 1;
    }
    if (fmt == ZO_Q4_0) {
        if (n % 32) return 0;
        for (size_t b = 0; b < n / 32; ++b) {
            const uint8_t* p = src + b * 18; const float d = zo_half_to_float(rd16(p));
            for (unsigned j = 0; j < 16; ++j) {
                const uint8_t q = p[2 + j];
                dst[b * 32 + j] = (float)((int)(q & 15) - 8) * d;
                dst[b * 32 + j + 16] = (float)((int)(q >> 4) - 8) * d;
            }
        }
        return 1;
    }
    if (fmt == ZO_Q4_K || fmt == ZO_Q5_K) {   /* src/quant.cpp:439-457 and :458-476: y = (d * sc) * q - dmin * m */
        const int q5 = fmt == ZO_Q5_K;
        if (n % 256) return 0;
        for (size_t b = 0; b < n / 256; ++b) {
            const uint8_t* p = src + b * (q5 ? 176 : 144);
            const float d = zo_half_to_float(rd16(p)), dmin = zo_half_to_float(rd16(p + 2));
            const uint8_t* scales = p + 4; const uint8_t* qh = p + 16; const uint8_t* ql = p + (q5 ? 48 : 16);
            size_t out = b * 256;
            for (unsigned pair = 0; pair < 4; ++pair) {     /* 64 values: low nibbles, then high nibbles, of 32 bytes */
                unsigned sc, m;
                k_scale_min(2 * pair, scales, &sc, &m);
                const float d1 = d * (float)sc, m1 = dmin * (float)m;
                k_scale_min(2 * pair + 1, scales, &sc, &m);
                const float d2 = d * (float)sc, m2 = dmin * (float)m;
                const unsigned u1 = 1u << (2 * pair), u2 = 2u << (2 * pair);
                for (unsigned l = 0; l < 32; ++l) dst[out++] = d1 * (float)((ql[l] & 15u) + ((q5 && (qh[l] & u1)) ? 16u : 0u)) - m1;
                for (unsigned l = 0; l < 32; ++l) dst[out++] = d2 * (float)((unsigned)(ql[l] >> 4) + ((q5 && (qh[l] & u2)) ? 16u : 0u)) - m2;
                ql += 32;
            }
        }
        return 1;
    }
    if (fmt == ZO_Q6_K) {
        if (n % 256) return 0;
        for (size_t b = 0; b < n / 256; ++b) {
            const uint8_t* p = src + b * 210; const uint8_t* ql = p; const uint8_t* qh = p + 128;
            const int8_t* sc = (const int8_t*)(p + 192); const float d = zo_half_to_float(rd16(p + 208));
            for (unsigned n128 = 0; n128 < 256; n128 += 128) {
                for (unsigned l = 0; l < 32; ++l) {
                    const unsigned is = l / 16;
                    const int q1 = (int)((ql[l] & 15u) | (((qh[l] >> 0) & 3u) << 4)) - 32;
                    const int q2 = (int)((ql[l + 32] & 15u) | (((qh[l] >> 2) & 3u) << 4)) - 32;
                    const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3u) << 4)) - 32;
                    const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3u) << 4)) - 32;
                    const size_t base = b * 256 + n128 + l;
                    dst[base + 0]  = d * (float)sc[is + 0] * (float)q1;
                    dst[base + 32] = d * (float)sc[is + 2] * (float)q2;
                    dst[base + 64] = d * (float)sc[is + 4] * (float)q3;
                    dst[base + 96] = d * (float)sc[is + 6] * (float)q4;
                }
                ql += 64; qh += 32; sc += 8;
            }
        }
        return 1;
    }
    return 0;
}

/* ---- activation quantiser: kernels/avx2.cpp:502-524 (twin of
 *      src/quant.cpp:1094-1113).  fp32 scale, round half away from zero. --- */

ZO_API void zo_quantise_acts_q8_0(const float* x, size_t columns, int8_t* q, float* sc) {
    const size_t blocks = columns / 32;
    for (size_t b = 0; b < blocks; ++b) {
        const float* xb = x + b * 32;
        float amax = 0.0f;
        for (unsigned i = 0; i < 32; ++i) { const float a = fabsf(xb[i]); amax = a > amax ? a : amax; }
        const float d = amax > 0.0f ? amax / 127.0f : 0.0f;
        const float inv = d > 0.0f ? 1.0f / d : 0.0f;
        sc[b] = d;
        for (unsigned i = 0; i < 32; ++i) {
            float v = xb[i] * inv;
            v = v > 127.0f ? 127.0f : (v < -127.0f ? -127.0f : v);
            q[b * 32 + i] = (int8_t)lroundf(v);
        }
    }
}

/* horizontal sum used by every fused AVX2 GEMV: kernels/avx2.cpp:95-102.
 * (lo+hi), then two hadd passes: ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)). */
static inline float hsum8(const float* l) {
    const float s0 = l[0] + l[4], s1 = l[1] + l[5], s2 = l[2] + l[6], s3 = l[3] + l[7];
    return (s0 + s1) + (s2 + s3);
}

/* ---- Q8_0 GEMV, fp32 activations (the reference default):
 *      kernels/avx2.cpp:608-640 ------------------------------------------- */

ZO_API int zo_gemv_q8_0_f32(const uint8_t* weights, const float* x, float* y, size_t rows, size_t columns) {
    if (!weights || !x || !y || !rows || !columns || columns % 32) return 0;
    const size_t blocks = columns / 32, row_bytes = blocks * 34;
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t* row = weights + r * row_bytes;
        float acc[8] = {0};
        for (size_t b = 0; b < blocks; ++b) {
            const uint8_t* p = row + b * 34;
            const float d = zo_half_to_float(rd16(p));
            float a[4][8];
            for (unsigned chunk = 0; chunk < 4; ++chunk)
                for (unsigned j = 0; j < 8; ++j)
                    a[chunk][j] = fmaf((float)(int8_t)p[2 + chunk * 8 + j], x[b * 32 + chunk * 8 + j], 0.0f);
            for (unsigned j = 0; j < 8; ++j) {
                const float s = (a[0][j] + a[1][j]) + (a[2][j] + a[3][j]);
                acc[j] = fmaf(d, s, acc[j]);
            }
        }
        y[r] = hsum8(acc);
    }
    return 1;
}

/* ---- Q8_0 GEMV, int8 activations quantised once (ZEN_CPU_Q8_ACT=1):
 *      kernels/avx2.cpp:562-585.  maddubs+madd leave lane j holding the
 *      exact int32 sum of bytes 4j..4j+3. -------------------------------- */

ZO_API int zo_gemv_q8_0_i8_prequant(const uint8_t* weights, const int8_t* xq, const float* xsc,
                                    float* y, size_t rows, size_t columns) {
    if (!weights || !xq || !xsc || !y || !rows || !columns || columns % 32) return 0;
    const size_t blocks = columns / 32, row_bytes = blocks * 34;
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t* row = weights + r * row_bytes;
        float acc[8] = {0};
        for (size_t b = 0; b < blocks; ++b) {
            const uint8_t* p = row + b * 34;
            const float d = zo_half_to_float(rd16(p)) * xsc[b];
            for (unsigned j = 0; j < 8; ++j) {
                int32_t s = 0;
                for (unsigned k = 0; k < 4; ++k)
                    s += (int32_t)(int8_t)p[2 + j * 4 + k] * (int32_t)xq[b * 32 + j * 4 + k];
                acc[j] = fmaf(d, (float)s, acc[j]);
            }
        }
        y[r] = hsum8(acc);
    }
    return 1;
}

/* quantise + sweep: kernels/avx2.cpp:531-558 and src/quant.cpp:1088-1123 */
ZO_API int zo_gemv_q8_0_i8(const uint8_t* weights, const float* x, float* y, size_t rows, size_t columns) {
    if (!weights || !x || !y || !rows || !columns || columns % 32) return 0;
    int8_t* xq = (int8_t*)malloc(columns); float* xsc = (float*)malloc((columns / 32) * sizeof(float));
    if (!xq || !xsc) { free(xq); free(xsc); return 0; }
    zo_quantise_acts_q8_0(x, columns, xq, xsc);
    const int ok = zo_gemv_q8_0_i8_prequant(weights, xq, xsc, y, rows, columns);
    free(xq); free(xsc);
    return ok;
}

/* ---- fp32 row dot used by the generic route: kernels/avx2.cpp:16-40 ----- */

static float dot_gemv_avx2(const float* row, const float* x, size_t k) {
    float s[4][8] = {{0}};
    size_t p = 0;
    for (; p + 31 < k; p += 32)
        for (unsigned c = 0; c < 4; ++c)
            for (unsigned j = 0; j < 8; ++j)
                s[c][j] = fmaf(row[p + c * 8 + j], x[p + c * 8 + j], s[c][j]);
    float sum[8];
    for (unsigned j = 0; j < 8; ++j) sum[j] = (s[0][j] + s[1][j]) + (s[2][j] + s[3][j]);
    for (; p + 7 < k; p += 8)
        for (unsigned j = 0; j < 8; ++j) sum[j] = fmaf(row[p + j], x[p + j], sum[j]);
    float total = sum[0] + sum[1] + sum[2] + sum[3] + sum[4] + sum[5] + sum[6] + sum[7];
    for (; p < k; ++p) total += row[p] * x[p];
    return total;
}

/* kernels/avx2.cpp:696-711 -- the tail dot of the batched kernels */
static float dot_f32(const float* a, const float* b, size_t n) {
    float s0[8] = {0}, s1[8] = {0};
    size_t i = 0;
    for (; i + 15 < n; i += 16)
        for (unsigned j = 0; j < 8; ++j) {
            s0[j] = fmaf(a[i + j], b[i + j], s0[j]);
            s1[j] = fmaf(a[i + 8 + j], b[i + 8 + j], s1[j]);
        }
    float s[8];
    for (unsigned j = 0; j < 8; ++j) s[j] = s0[j] + s1[j];
    for (; i + 7 < n; i += 8)
        for (unsigned j = 0; j < 8; ++j) s[j] = fmaf(a[i + j], b[i + j], s[j]);
    float t = s[0] + s[1] + s[2] + s[3] + s[4] + s[5] + s[6] + s[7];
    for (; i < n; ++i) t += a[i] * b[i];
    return t;
}

/* ---- generic route (what Q4_0 takes): src/quant.cpp:1135-1162 (GEMV) and
 *      :1743-1773 (GEMM).  Dequantise the row, then one full-row dot per
 *      token. ------------------------------------------------------------- */

ZO_API int zo_gemm_generic(int fmt, const uint8_t* weights, const float* input, float* output,
                           size_t tokens, size_t rows, size_t columns) {
    const size_t rb = zo_row_bytes(fmt, columns);
    if (!weights || !input || !output || !tokens || !rows || !columns || !rb) return 0;
    float* rowbuf = (float*)malloc(columns * sizeof(float));
    if (!rowbuf) return 0;
    for (size_t r = 0; r < rows; ++r) {
        if (!zo_dequantize(fmt, weights + r * rb, columns, rowbuf)) { free(rowbuf); return 0; }
        for (size_t t = 0; t < tokens; ++t)
            output[t * rows + r] = dot_gemv_avx2(rowbuf, input + t * columns, columns);
    }
    free(rowbuf);
    return 1;
}

/* ---- Q6_K fused GEMV: kernels/avx2.cpp:380-422.  Weight order (d*scale)*q,
 *      accumulator index = lane/8, final add (s0+s1)+(s2+s3) then hsum. --- */

static inline float q6k_weight(const uint8_t* p, unsigned half, unsigned group, unsigned lane, float d) {
    const uint8_t low = p[half * 64 + (group % 2) * 32 + lane];
    const uint8_t high = p[128 + half * 32 + lane];
    const unsigned nib = group >= 2 ? (unsigned)(low >> 4) : (unsigned)(low & 15u);
    const int q = (int)(nib | (((high >> (group * 2)) & 3u) << 4)) - 32;
    const int8_t* scales = (const int8_t*)(p + 192);
    const float ds = d * (float)scales[half * 8 + group * 2 + lane / 16];
    return ds * (float)q;
}

ZO_API int zo_gemv_q6k_f32(const uint8_t* weights, const float* x, float* y, size_t rows, size_t columns) {
    if (!weights || !x || !y || !rows || !columns || columns % 256) return 0;
    const size_t blocks = columns / 256;
    for (size_t r = 0; r < rows; ++r) {
        float sums[4][8] = {{0}};
        for (size_t b = 0; b < blocks; ++b) {
            const uint8_t* p = weights + (r * blocks + b) * 210;
            const float d = zo_half_to_float(rd16(p + 208));
            for (unsigned half = 0; half < 2; ++half)
                for (unsigned group = 0; group < 4; ++group)
                    for (unsigned lane = 0; lane < 32; ++lane) {
                        const float w = q6k_weight(p, half, group, lane, d);
                        const float xv = x[b * 256 + half * 128 + group * 32 + lane];
                        float* s = &sums[lane / 8][lane % 8];
                        *s = fmaf(w, xv, *s);
                    }
        }
        float t[8];
        for (unsigned j = 0; j < 8; ++j) t[j] = (sums[0][j] + sums[1][j]) + (sums[2][j] + sums[3][j]);
        y[r] = hsum8(t);
    }
    return 1;
}

/* ---- Q4_K / Q5_K GEMV, fp32 activations: kernels/avx2.cpp:329-378 (route src/quant.cpp:1020-1031, columns % 256 == 0).
 *      Per sub-block of 32: ds = d * sc, ms = dmin * m; chunk c (8 lanes) of the sub-block goes to accumulator c:
 *      w = ds * float(q) - ms (a multiply, then a subtract), acc[c] = fma(w, x, acc[c]); the four accumulators are added
 *      pairwise and summed across lanes at the end of the row. ----------------------------------------------------- */

ZO_API int zo_gemv_q4k_q5k_f32(const uint8_t* weights, const float* x, float* y, size_t rows, size_t columns, int q5) {
    if (!weights || !x || !y || !rows || !columns || columns % 256) return 0;
    const size_t block_bytes = q5 ? 176 : 144, blocks = columns / 256;
    for (size_t r = 0; r < rows; ++r) {
        float acc[4][8] = {{0}};
        for (size_t b = 0; b < blocks; ++b) {
            const uint8_t* p = weights + (r * blocks + b) * block_bytes;
            const float d = zo_half_to_float(rd16(p)), dm = zo_half_to_float(rd16(p + 2));
            const uint8_t* scales = p + 4; const uint8_t* qh = p + 16; const uint8_t* ql = p + (q5 ? 48 : 16);
            for (unsigned group = 0; group < 8; ++group) {
                unsigned sc, mn;
                k_scale_min(group, scales, &sc, &mn);
                const float ds = d * (float)sc, ms = dm * (float)mn;
                const unsigned shift = (group & 1u) * 4;
                for (unsigned chunk = 0; chunk < 4; ++chunk)
                    for (unsigned j = 0; j < 8; ++j) {
                        const unsigned l = chunk * 8 + j;
                        unsigned q = ((unsigned)ql[(group / 2) * 32 + l] >> shift) & 15u;
                        if (q5) q |= (((unsigned)qh[l] >> group) & 1u) << 4;
                        const float prod = ds * (float)q;       /* rounded before the subtraction, as mul_ps then sub_ps */
                        const float w = prod - ms;
                        acc[chunk][j] = fmaf(w, x[b * 256 + group * 32 + l], acc[chunk][j]);
                    }
            }
        }
        float t[8];
        for (unsigned j = 0; j < 8; ++j) t[j] = (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]);
        y[r] = hsum8(t);
    }
    return 1;
}

/* ---- batched kernels.  Main block of kernels/avx2.cpp:772-840 (Q8_0, two
 *      rows x four tokens) and of gemm_kblk_impl :1470-1545 (Q6_K, Kc=256):
 *      the row is dequantised to fp32, one 8-lane FMA chain runs over
 *      c = 0, 8, 16, ..., and the lanes are added in index order.  Token and
 *      row tails of the reference go through dot_f32 (:696-711) instead;
 *      `tail_rows`/`tail_tokens` select it so the result is bit-identical
 *      for every shape. --------------------------------------------------- */

static float dot_lane_chain(const float* w, const float* x, size_t columns) {
    float a[8] = {0};
    size_t c = 0;
    for (; c + 8 <= columns; c += 8)
        for (unsigned j = 0; j < 8; ++j) a[j] = fmaf(w[c + j], x[c + j], a[j]);
    float total = a[0] + a[1] + a[2] + a[3] + a[4] + a[5] + a[6] + a[7];
    for (; c < columns; ++c) total += w[c] * x[c];
    return total;
}

static void dequant_row_q8_0(const uint8_t* row, size_t columns, float* dst) {
    for (size_t b = 0; b < columns / 32; ++b) {
        const uint8_t* p = row + b * 34; const float d = zo_half_to_float(rd16(p));
        for (unsigned j = 0; j < 32; ++j) dst[b * 32 + j] = (float)(int8_t)p[2 + j] * d;
    }
}

/* fp32-activation Q8_0 GEMM, the legacy row-pair kernel: kernels/avx2.cpp:772-840 */
ZO_API int zo_gemm_q8_0_f32(const uint8_t* weights, const float* input, float* output,
                            size_t tokens, size_t rows, size_t columns) {
    if (!weights || !input || !output || !tokens || !rows || !columns || columns % 32) return 0;
    const size_t rb = (columns / 32) * 34;
    float* w = (float*)malloc(columns * sizeof(float));
    if (!w) return 0;
    const size_t rows_paired = rows & ~(size_t)1, tokens_main = tokens & ~(size_t)3;
    for (size_t r = 0; r < rows; ++r) {
        dequant_row_q8_0(weights + r * rb, columns, w);
        for (size_t t = 0; t < tokens; ++t) {
            const float* x = input + t * columns;
            const int main_block = r < rows_paired && t < tokens_main;
            output[t * rows + r] = main_block ? dot_lane_chain(w, x, columns) : dot_f32(w, x, columns);
        }
    }
    free(w);
    return 1;
}

/* K-blocked Q8_0 GEMM (what config-size prefill takes: tokens*cols >= 131072,
 * src/quant.cpp:1188-1192): kernels/avx2.cpp:878-1070.  Partials stay 8-lane
 * vectors across K panels, so every (row,token) of the 4-row main block is
 * the plain c = 0,8,16,... chain; rows beyond the last multiple of four use
 * dot_f32. */
ZO_API int zo_gemm_q8_0_f32_kblk(const uint8_t* weights, const float* input, float* output,
                                 size_t tokens, size_t rows, size_t columns) {
    if (!weights || !input || !output || !tokens || !rows || !columns || columns % 32) return 0;
    const size_t rb = (columns / 32) * 34, rows_main = (rows / 4) * 4;
    float* w = (float*)malloc(columns * sizeof(float));
    if (!w) return 0;
    for (size_t r = 0; r < rows; ++r) {
        dequant_row_q8_0(weights + r * rb, columns, w);
        for (size_t t = 0; t < tokens; ++t) {
            const float* x = input + t * columns;
            output[t * rows + r] = r < rows_main ? dot_lane_chain(w, x, columns) : dot_f32(w, x, columns);
        }
    }
    free(w);
    return 1;
}

/* int8-activation GEMM.  The reference has no batched int8 CPU kernel; its
 * int8 arithmetic is the per-token sweep of kernels/avx2.cpp:562-585, which
 * the D3D12 int8 prefill shader (shaders/q8_0_gemm_i8.hlsl:249-257) restates
 * per (row, token, block).  Output is token-major [tokens][rows]. */
ZO_API int zo_gemm_q8_0_i8(const uint8_t* weights, const float* input, float* output,
                           size_t tokens, size_t rows, size_t columns) {
    if (!weights || !input || !output || !tokens || !rows || !columns || columns % 32) return 0;
    for (size_t t = 0; t < tokens; ++t)
        if (!zo_gemv_q8_0_i8(weights, input + t * columns, output + t * rows, rows, columns)) return 0;
    return 1;
}

/* Q6_K GEMM: gemm_q6k_kblk_avx2, kernels/avx2.cpp:1762-1770 over
 * gemm_kblk_impl :1470-1545 (MR=4, Kc=256). */
ZO_API int zo_gemm_q6k_f32(const uint8_t* weights, const float* input, float* output,
                           size_t tokens, size_t rows, size_t columns) {
    if (!weights || !input || !output || !tokens || !rows || !columns || columns % 256) return 0;
    const size_t rb = (columns / 256) * 210, rows_main = (rows / 4) * 4;
    float* w = (float*)malloc(columns * sizeof(float));
    if (!w) return 0;
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t* row = weights + r * rb;
        for (size_t c = 0; c < columns; ++c) {
            const size_t idx = c % 256;
            w[c] = q6k_weight(row + (c / 256) * 210, (unsigned)(idx / 128), (unsigned)((idx % 128) / 32),
                              (unsigned)(idx % 32), zo_half_to_float(rd16(row + (c / 256) * 210 + 208)));
        }
        for (size_t t = 0; t < tokens; ++t) {
            const float* x = input + t * columns;
            output[t * rows + r] = r < rows_main ? dot_lane_chain(w, x, columns) : dot_f32(w, x, columns);
        }
    }
    free(w);
    return 1;
}

/* ---- format-level entry points mirroring zen::quant::gemv / gemm
 *      (src/quant.cpp:963-1163, :1613-1777) with the route the CPU build
 *      takes for each of the three formats.  q8_int8_acts selects the
 *      ZEN_CPU_Q8_ACT=1 arithmetic for Q8_0. ------------------------------ */

/* Q4_K / Q5_K batched: gemm_q4k_kblk_avx2 / gemm_q5k_kblk_avx2 (kernels/avx2.cpp:1605-1628) are gemm_kblk_impl
 * (:1470-1545) over panel dequantisers whose values equal zo_dequantize's (multiply, then subtract: :1352-1366,
 * :1410-1432); the panel width does not enter the arithmetic (the lane accumulators live across panels).  So, as for
 * Q6_K: the decoded row, one 8-lane FMA chain over the columns for rows in whole groups of four, dot_f32 for the
 * remaining rows. */
ZO_API int zo_gemm_q4k_q5k_f32(int fmt, const uint8_t* weights, const float* input, float* output,
                               size_t tokens, size_t rows, size_t columns) {
    if ((fmt != ZO_Q4_K && fmt != ZO_Q5_K) || !weights || !input || !output || !tokens || !rows || !columns || columns % 256) return 0;
    const size_t rb = zo_row_bytes(fmt, columns), rows_main = (rows / 4) * 4;
    float* w = (float*)malloc(columns * sizeof(float));
    if (!w) return 0;
    for (size_t r = 0; r < rows; ++r) {
        zo_dequantize(fmt, weights + r * rb, columns, w);
        for (size_t t = 0; t < tokens; ++t) {
            const float* x = input + t * columns;
            output[t * rows + r] = r < rows_main ? dot_lane_chain(w, x, columns) : dot_f32(w, x, columns);
        }
    }
    free(w);
    return 1;
}

ZO_API int zo_gemv(int fmt, const uint8_t* w, const float* x, float* y, size_t rows, size_t columns, int q8_int8_acts) {
    if (fmt == ZO_Q8_0) return q8_int8_acts ? zo_gemv_q8_0_i8(w, x, y, rows, columns) : zo_gemv_q8_0_f32(w, x, y, rows, columns);
    if (fmt == ZO_Q6_K) return zo_gemv_q6k_f32(w, x, y, rows, columns);
    if (fmt == ZO_Q4_0) return zo_gemm_generic(fmt, w, x, y, 1, rows, columns);
    if (fmt == ZO_Q4_K || fmt == ZO_Q5_K) return zo_gemv_q4k_q5k_f32(w, x, y, rows, columns, fmt == ZO_Q5_K);
    return 0;
}

ZO_API int zo_gemm(int fmt, const uint8_t* w, const float* in, float* out, size_t tokens, size_t rows, size_t columns, int q8_int8_acts) {
    if (fmt == ZO_Q8_0 && q8_int8_acts) return zo_gemm_q8_0_i8(w, in, out, tokens, rows, columns);
    /* every fused batched kernel is gated on tokens >= 2 (src/quant.cpp:1660,1726); a
     * one-token quant::gemm call lands on the generic route.  (The runtime never makes
     * that call: tensor_gemm sends tokens == 1 to gemv, dense_transformer_runtime.cpp:513.) */
    if (tokens == 1) return zo_gemm_generic(fmt, w, in, out, 1, rows, columns);
    if (fmt == ZO_Q8_0) {
        return tokens * columns >= 131072 ? zo_gemm_q8_0_f32_kblk(w, in, out, tokens, rows, columns)
                                          : zo_gemm_q8_0_f32(w, in, out, tokens, rows, columns);
    }
    if (fmt == ZO_Q6_K) return zo_gemm_q6k_f32(w, in, out, tokens, rows, columns);
    if (fmt == ZO_Q4_0) return zo_gemm_generic(fmt, w, in, out, tokens, rows, columns);
    if (fmt == ZO_Q4_K || fmt == ZO_Q5_K) return zo_gemm_q4k_q5k_f32(fmt, w, in, out, tokens, rows, columns);
    return 0;
}

/* ---- greedy pick: src/adapters/dense_transformer_runtime.cpp:407-415.
 *      Lowest index wins a tie; non-finite logits never win; -1 when no
 *      finite logit exists. ----------------------------------------------- */

ZO_API int64_t zo_argmax(const float* logits, size_t n) {
    int64_t best = -1; float best_v = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float v = logits[i];
        if (!isfinite(v)) continue;
        if (best < 0 || v > best_v) { best = (int64_t)i; best_v = v; }
    }
    return best;
}

/* ---- row slicing of ComputePool::parallel_for: src/compute_pool.cpp:104-106.
 *      Slice i of `workers` covers [count*i/workers, count*(i+1)/workers). -- */

ZO_API void zo_row_slice(size_t count, unsigned workers, unsigned i, size_t* first, size_t* last) {
    *first = count * i / workers; *last = count * (i + 1) / workers;
}
