/*
 * larql_oracle.c — CPU restatement of the reference's vindex FFN walk arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker for the CUDA
 * library and the timed CPU baseline.  Nothing in the product path may link,
 * import or call it; the CUDA path fails loudly when its extension is missing
 * instead of falling back to this code.
 *
 * Every function cites the reference file:line (paths relative to the
 * reference repository root) whose arithmetic it restates.  The restatement
 * pins the NON-aarch64 scalar arms of the reference (what it runs on x86).
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared -pthread
 * (contraction must stay off: Rust never fuses a*b+c, so an FMA here would
 * change bits).
 *
 * Parity status: pinned against the reference's own golden vectors
 * (ggml k-quant golden JSON, Q8_0 ggml golden blocks, codec known-answer
 * tests, top-k and router tie cases) and against the reference's importable
 * Python verifier for the Q8_0 gemv.  The MXFP4 gemv has no CPU-backend
 * implementation in the reference ("parity unpinned" for that one function);
 * it follows the reference's test device loop.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* Rust f32::round(): half away from zero. C roundf has the same rule. */
static inline float rs_round(float v) { return roundf(v); }
static inline float rs_clamp(float v, float lo, float hi) {
    /* f32::clamp: NaN stays NaN; callers cast afterwards (`as u8` saturates, NaN -> 0). */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}
static inline uint8_t rs_as_u8(float v) {
    if (!(v == v)) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 255.0f) return 255;
    return (uint8_t)v;
}
static inline int8_t rs_as_i8(float v) {
    if (!(v == v)) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}

/* ------------------------------------------------------------------ f16 -- */

/* crates/larql-models/src/quant/half.rs:14-35 (f16_to_f32); the twin in
 * crates/larql-compute/src/cpu/ops/q4_common/f16.rs:60-102 is bit-equal. */
ORC_API float orc_f16_to_f32(uint16_t bits) {
    uint32_t sign = ((uint32_t)(bits >> 15)) << 31;
    uint32_t exp = (bits >> 10) & 0x1F;
    uint32_t mant = bits & 0x3FF;
    if (exp == 0) {
        if (mant == 0) return u2f(sign);
        uint32_t e = 1, m = mant;
        while ((m & 0x400) == 0) { m <<= 1; e += 1; }
        return u2f(sign | ((114 - e) << 23) | ((m & 0x3FF) << 13));
    }
    if (exp == 31) return u2f(sign | (0xFFu << 23) | (mant << 13));
    return u2f(sign | ((exp + 127 - 15) << 23) | (mant << 13));
}

/* crates/larql-compute/src/cpu/ops/q4_common/f16.rs:10-41 — TRUNCATING
 * encoder that keeps subnormals; used by the Q4_K quantiser only. */
ORC_API uint16_t orc_f32_to_f16_trunc(float val) {
    uint32_t bits = f2u(val);
    uint32_t sign = (bits >> 16) & 0x8000;
    int32_t exp = (int32_t)((bits >> 23) & 0xFF);
    uint32_t mant = bits & 0x7FFFFF;
    if (exp == 0) return (uint16_t)sign;
    if (exp == 255) return (uint16_t)(sign | 0x7C00 | (mant >> 13));
    int32_t new_exp = exp - 127 + 15;
    if (new_exp >= 31) return (uint16_t)(sign | 0x7C00);
    if (new_exp <= 0) {
        int32_t shift = 1 - new_exp;
        if (13 + (uint32_t)shift >= 24) return (uint16_t)sign;
        uint32_t sub_mant = (mant | 0x800000) >> (13 + (uint32_t)shift);
        return (uint16_t)(sign | sub_mant);
    }
    return (uint16_t)(sign | ((uint32_t)new_exp << 10) | (mant >> 13));
}

/* crates/larql-models/src/quant/half.rs:70-104 — IEEE round-to-nearest-even,
 * subnormals kept; used by the Q8_0 quantiser. */
ORC_API uint16_t orc_f32_to_f16_nearest(float value) {
    uint32_t bits = f2u(value);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
    int32_t exp = (int32_t)((bits >> 23) & 0xFF);
    uint32_t mant = bits & 0x007FFFFF;
    if (exp == 255) return sign | (mant == 0 ? 0x7C00 : 0x7E00);
    int32_t exp16 = exp - 127 + 15;
    if (exp16 >= 31) return sign | 0x7C00;
    uint32_t significand, shift;
    if (exp16 >= 1) { significand = mant; shift = 13; }
    else if (exp == 0 || exp16 < -10) return sign;
    else { significand = mant | 0x00800000; shift = (uint32_t)(14 - exp16); }
    uint32_t magnitude = significand >> shift;
    uint32_t remainder = significand & ((1u << shift) - 1);
    uint32_t half = 1u << (shift - 1);
    if (remainder > half || (remainder == half && (magnitude & 1) == 1)) magnitude += 1;
    if (exp16 >= 1) magnitude += ((uint32_t)exp16) << 10;
    return sign | (uint16_t)magnitude;
}

/* --------------------------------------------------------- fp8 / fp4 ---- */

/* crates/larql-models/src/quant/fp8.rs:33-56 (e4m3_bits_to_f32_compute). */
ORC_API float orc_e4m3_to_f32(uint8_t byte) {
    uint32_t sign = (byte >> 7) & 1, exp = (byte >> 3) & 0x0F, mant = byte & 0x07;
    if (exp == 0x0F && mant == 0x07) return NAN;
    float mag;
    if (exp == 0) mag = (float)mant * (1.0f / 8.0f) * ldexpf(1.0f, -6);
    else {
        float frac = 1.0f + (float)mant / 8.0f;
        mag = frac * ldexpf(1.0f, (int)exp - 7);
    }
    return sign ? -mag : mag;
}

/* crates/larql-models/src/quant/fp8.rs:141-153 (round_ties_to_even). */
static float round_ties_to_even_rs(float x) {
    float r = rs_round(x);
    if (fabsf(x - truncf(x)) == 0.5f) {
        if (((int32_t)r) % 2 != 0) return r - copysignf(1.0f, r);
        return r;
    }
    return r;
}

/* crates/larql-models/src/quant/fp8.rs:63-139 (f32_to_e4m3). */
ORC_API uint8_t orc_f32_to_e4m3(float value) {
    if (value != value) return signbit(value) ? 0xFF : 0x7F;
    uint8_t sign_bit = signbit(value) ? 0x80 : 0x00;
    float mag = fabsf(value);
    if (mag == 0.0f) return sign_bit;
    if (mag >= 448.0f) return sign_bit | 0x7E;
    uint32_t bits = f2u(mag);
    int32_t f32_exp = (int32_t)((bits >> 23) & 0xFF) - 127;
    if (f32_exp < -9) return sign_bit;
    if (f32_exp < -6) {
        float scaled = mag * 512.0f;
        float rounded = round_ties_to_even_rs(scaled);
        uint32_t m = (uint32_t)rs_clamp(rounded, 0.0f, 7.0f);
        return sign_bit | (uint8_t)m;
    }
    uint32_t e4m3_exp = (uint32_t)(f32_exp + 7);
    if (e4m3_exp > 15) return sign_bit | 0x7E;
    uint32_t full = bits & 0x007FFFFF;
    uint32_t keep = full >> 20, rem = full & 0x000FFFFF, half = 0x00080000;
    int rounded_up = rem > half || (rem == half && (keep & 1) == 1);
    uint32_t e = e4m3_exp, m = keep;
    if (rounded_up) { m += 1; if (m == 8) { m = 0; e += 1; } }
    if (e >= 15 && m >= 7) return sign_bit | 0x7E;
    if (e > 15) return sign_bit | 0x7E;
    return sign_bit | (uint8_t)(e << 3) | (uint8_t)m;
}

/* crates/larql-models/src/quant/fp4.rs:19-21 (FP4_E2M1_TABLE) ==
 * crates/larql-models/src/quant/mxfp4.rs:15-17 (MXFP4_TABLE). */
static const float E2M1_TABLE[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                     -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
ORC_API float orc_e2m1_to_f32(uint8_t code) { return E2M1_TABLE[code & 0x0F]; }

/* crates/larql-models/src/quant/fp4.rs:38-72 (f32_to_e2m1): nearest magnitude,
 * ties to the even code index, sign kept on a zero magnitude. */
ORC_API uint8_t orc_f32_to_e2m1(float value) {
    if (value != value) return 0x00;
    uint8_t sign_bit = signbit(value) ? 0x08 : 0x00;
    float mag = fabsf(value);
    if (isinf(mag)) return sign_bit | 7;
    int best = 0;
    float best_err = fabsf(mag - E2M1_TABLE[0]);
    for (int i = 1; i < 8; i++) {
        float err = fabsf(mag - E2M1_TABLE[i]);
        if (err < best_err) { best = i; best_err = err; }
        else if (err == best_err) { if ((i & 1) == 0) best = i; }
    }
    return sign_bit | (uint8_t)best;
}

/* crates/larql-models/src/quant/mxfp4.rs:27-35 (e8m0_to_f32). */
ORC_API float orc_e8m0_to_f32(uint8_t byte) {
    if (byte == 0) return 0.0f;
    if (byte == 255) return NAN;
    return u2f(((uint32_t)byte) << 23);
}

/* crates/larql-vindex/src/format/vindex3/opplan/exec/weights/quantize.rs:69-88
 * (nearest_mxfp4_code): +-0 collapse to code 0. */
ORC_API uint8_t orc_nearest_mxfp4_code(float v) {
    uint8_t sign = signbit(v) ? 8 : 0;
    float mag = fminf(fabsf(v), 6.0f);
    /* f32::min returns the non-NaN operand: fminf does the same. */
    uint8_t best = 0;
    float best_err = INFINITY;
    for (int code = 0; code < 8; code++) {
        float err = fabsf(mag - E2M1_TABLE[code]);
        if (err < best_err || (err == best_err && (code % 2 == 0))) { best = (uint8_t)code; best_err = err; }
    }
    return best == 0 ? 0 : (sign | best);
}

/* ------------------------------------------------------------- Q4_K ----- */

/* get_scale_min_k4 unpack; crates/larql-models/src/quant/ggml/q4_k.rs:92-104. */
static inline void unpack_q4k_scales(const uint8_t *p, uint8_t sc[8], uint8_t mn[8]) {
    for (int j = 0; j < 4; j++) { sc[j] = p[j] & 0x3F; mn[j] = p[j + 4] & 0x3F; }
    for (int j = 4; j < 8; j++) {
        sc[j] = (p[j + 4] & 0x0F) | ((p[j - 4] >> 6) << 4);
        mn[j] = (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
    }
}

/* crates/larql-compute/src/cpu/ops/q4_common/quantize.rs:89-189 (quantize_q4_k).
 * n must be a multiple of 256; out holds n/256*144 bytes. */
ORC_API void orc_quantize_q4_k(const float *data, size_t n, uint8_t *out) {
    size_t nsb = n / 256;
    for (size_t sb = 0; sb < nsb; sb++) {
        const float *block = data + sb * 256;
        uint8_t *o = out + sb * 144;
        float sub_mins[8], sub_maxs[8];
        for (int j = 0; j < 8; j++) {
            float mn = INFINITY, mx = -INFINITY;
            for (int l = 0; l < 32; l++) {
                float v = block[j * 32 + l];
                mn = fminf(mn, v);
                mx = fmaxf(mx, v);
            }
            sub_mins[j] = fminf(mn, 0.0f);
            sub_maxs[j] = fmaxf(mx, 0.0f);
        }
        float global_max_range = 0.0f, global_min = INFINITY;
        for (int j = 0; j < 8; j++) {
            global_max_range = fmaxf(global_max_range, sub_maxs[j] - sub_mins[j]);
            global_min = fminf(global_min, sub_mins[j]);
        }
        float d = global_max_range > 0.0f ? global_max_range / (15.0f * 63.0f) : 0.0f;
        float dmin = global_min < 0.0f ? -global_min / 63.0f : 0.0f;
        uint16_t dh = orc_f32_to_f16_trunc(d), dmh = orc_f32_to_f16_trunc(dmin);
        o[0] = dh & 0xFF; o[1] = dh >> 8; o[2] = dmh & 0xFF; o[3] = dmh >> 8;
        uint8_t qs[8], qm[8];
        for (int j = 0; j < 8; j++) {
            float range = sub_maxs[j] - sub_mins[j];
            qs[j] = d > 0.0f ? rs_as_u8(rs_clamp(rs_round(range / (15.0f * d)), 0.0f, 63.0f)) : 0;
            qm[j] = dmin > 0.0f ? rs_as_u8(rs_clamp(rs_round(-sub_mins[j] / dmin), 0.0f, 63.0f)) : 0;
        }
        uint8_t *packed = o + 4;
        for (int j = 0; j < 4; j++) {
            packed[j] = (qs[j] & 0x3F) | (((qs[j + 4] >> 4) & 0x03) << 6);
            packed[j + 4] = (qm[j] & 0x3F) | (((qm[j + 4] >> 4) & 0x03) << 6);
            packed[j + 8] = (qs[j + 4] & 0x0F) | ((qm[j + 4] & 0x0F) << 4);
        }
        uint8_t *q = o + 16;
        for (int g = 0; g < 4; g++) {
            int sb_lo = 2 * g, sb_hi = 2 * g + 1;
            float sc_lo = d * (float)qs[sb_lo], sc_hi = d * (float)qs[sb_hi];
            float mn_lo = dmin * (float)qm[sb_lo], mn_hi = dmin * (float)qm[sb_hi];
            float inv_lo = sc_lo > 0.0f ? 1.0f / sc_lo : 0.0f;
            float inv_hi = sc_hi > 0.0f ? 1.0f / sc_hi : 0.0f;
            const float *lo_sub = block + sb_lo * 32, *hi_sub = block + sb_hi * 32;
            for (int l = 0; l < 32; l++) {
                uint8_t lo = rs_as_u8(rs_clamp(rs_round((lo_sub[l] + mn_lo) * inv_lo), 0.0f, 15.0f));
                uint8_t hi = rs_as_u8(rs_clamp(rs_round((hi_sub[l] + mn_hi) * inv_hi), 0.0f, 15.0f));
                q[g * 32 + l] = lo | (hi << 4);
            }
        }
    }
}

/* crates/larql-models/src/quant/ggml/q4_k.rs:286-338 (dequantize_q4_k); twin
 * crates/larql-compute/src/cpu/ops/q4_common/dequant.rs:9-53. */
ORC_API void orc_dequantize_q4_k(const uint8_t *data, size_t n, float *out) {
    size_t nsb = n / 256;
    for (size_t sb = 0; sb < nsb; sb++) {
        const uint8_t *b = data + sb * 144;
        float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
        uint8_t sc[8], mn[8];
        unpack_q4k_scales(b + 4, sc, mn);
        const uint8_t *q = b + 16;
        for (int g = 0; g < 4; g++) {
            float sc_lo = d * (float)sc[2 * g], sc_hi = d * (float)sc[2 * g + 1];
            float mn_lo = dmin * (float)mn[2 * g], mn_hi = dmin * (float)mn[2 * g + 1];
            float *olo = out + sb * 256 + (2 * g) * 32, *ohi = olo + 32;
            for (int l = 0; l < 32; l++) {
                uint8_t byte = q[g * 32 + l];
                olo[l] = sc_lo * (float)(byte & 0x0F) - mn_lo;
                ohi[l] = sc_hi * (float)((byte >> 4) & 0x0F) - mn_hi;
            }
        }
    }
}

/* Association A.  crates/larql-compute/src/cpu/ops/q4_common/matvec_f32.rs:116-155
 * (process_q4k_superblock) with the scalar arm of q4_dual_dot_32,
 * crates/larql-compute/src/cpu/ops/q4_common/dual.rs:186-198. */
static float q4k_superblock_A(const uint8_t *b, const float *x, const float *sum_x) {
    float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
    float dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
    uint8_t sc[8], mn[8];
    unpack_q4k_scales(b + 4, sc, mn);
    const uint8_t *q = b + 16;
    float acc = 0.0f;
    for (int g = 0; g < 4; g++) {
        int sb_lo = 2 * g, sb_hi = 2 * g + 1;
        float sc_lo = d * (float)sc[sb_lo], sc_hi = d * (float)sc[sb_hi];
        float mn_lo = dmin * (float)mn[sb_lo], mn_hi = dmin * (float)mn[sb_hi];
        const uint8_t *chunk = q + g * 32;
        const float *x_lo = x + sb_lo * 32, *x_hi = x + sb_hi * 32;
        float dot_lo = 0.0f, dot_hi = 0.0f;
        for (int l = 0; l < 32; l++) {
            uint8_t byte = chunk[l];
            float q_lo = (float)(byte & 0x0F), q_hi = (float)((byte >> 4) & 0x0F);
            dot_lo += q_lo * x_lo[l];
            dot_hi += q_hi * x_hi[l];
        }
        acc += sc_lo * dot_lo - mn_lo * sum_x[sb_lo];
        acc += sc_hi * dot_hi - mn_hi * sum_x[sb_hi];
    }
    return acc;
}

/* sum_x precompute: matvec_f32.rs:66-76. */
static void q4k_sum_x(const float *x, size_t cols, float *sum_x) {
    for (size_t sub = 0; sub < cols / 32; sub++) {
        float s = 0.0f;
        for (int l = 0; l < 32; l++) s += x[sub * 32 + l];
        sum_x[sub] = s;
    }
}

static void q4k_matvec_rows(const uint8_t *w, const float *x, const float *sum_x, size_t r0, size_t r1,
                            size_t cols, float *out) {
    size_t nb = cols / 256, row_bytes = nb * 144;
    for (size_t r = r0; r < r1; r++) {
        float acc = 0.0f;
        for (size_t sb = 0; sb < nb; sb++)
            acc += q4k_superblock_A(w + r * row_bytes + sb * 144, x + sb * 256, sum_x + sb * 8);
        out[r] = acc;
    }
}

/* crates/larql-compute/src/cpu/ops/q4_common/matvec_f32.rs:37-106 (q4k_matvec_into).
 * Returns 0 on success, 1 on a shape refusal (KernelShapeError::check,
 * crates/larql-compute/src/cpu/ops/kernel_shape.rs:41-78). */
ORC_API int orc_q4k_matvec(const uint8_t *w, size_t w_len, const float *x, size_t x_len, size_t rows,
                           size_t cols, float *out, size_t out_len) {
    size_t needed = (cols / 256) * 144 * rows;
    if (!(out_len == rows && x_len == cols && cols % 256 == 0 && w_len >= needed)) return 1;
    if (rows == 0 || cols == 0) { for (size_t i = 0; i < out_len; i++) out[i] = 0.0f; return 0; }
    float *sum_x = (float *)malloc(sizeof(float) * (cols / 32));
    q4k_sum_x(x, cols, sum_x);
    q4k_matvec_rows(w, x, sum_x, 0, rows, cols, out);
    free(sum_x);
    return 0;
}

/* Association B.  crates/larql-models/src/quant/ggml/q4_k.rs:59-89 (q4k_row_dot_scalar). */
ORC_API float orc_q4k_row_dot(const uint8_t *data, const float *x, size_t n) {
    size_t nb = n / 256;
    float acc = 0.0f;
    for (size_t sb = 0; sb < nb; sb++) {
        const uint8_t *b = data + sb * 144;
        float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
        uint8_t sc[8], mn[8];
        unpack_q4k_scales(b + 4, sc, mn);
        const uint8_t *q = b + 16;
        for (int g = 0; g < 4; g++) {
            float sc_lo = d * (float)sc[2 * g], sc_hi = d * (float)sc[2 * g + 1];
            float mn_lo = dmin * (float)mn[2 * g], mn_hi = dmin * (float)mn[2 * g + 1];
            const float *xlo = x + sb * 256 + (2 * g) * 32, *xhi = xlo + 32;
            for (int l = 0; l < 32; l++) {
                uint8_t byte = q[g * 32 + l];
                float v_lo = sc_lo * (float)(byte & 0x0F) - mn_lo;
                float v_hi = sc_hi * (float)((byte >> 4) & 0x0F) - mn_hi;
                acc += v_lo * xlo[l];
                acc += v_hi * xhi[l];
            }
        }
    }
    return acc;
}

/* crates/larql-models/src/quant/ggml/q4_k.rs:201-227 (q4k_row_scaled_add_scalar):
 * out += alpha * dequant(row), alpha folded into the scales left to right. */
ORC_API void orc_q4k_row_scaled_add(const uint8_t *data, float alpha, float *out, size_t n) {
    size_t nb = n / 256;
    for (size_t sb = 0; sb < nb; sb++) {
        const uint8_t *b = data + sb * 144;
        float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
        uint8_t sc[8], mn[8];
        unpack_q4k_scales(b + 4, sc, mn);
        const uint8_t *q = b + 16;
        for (int g = 0; g < 4; g++) {
            float sc_lo = alpha * d * (float)sc[2 * g], sc_hi = alpha * d * (float)sc[2 * g + 1];
            float mn_lo = alpha * dmin * (float)mn[2 * g], mn_hi = alpha * dmin * (float)mn[2 * g + 1];
            float *olo = out + sb * 256 + (2 * g) * 32, *ohi = olo + 32;
            for (int l = 0; l < 32; l++) {
                uint8_t byte = q[g * 32 + l];
                olo[l] += sc_lo * (float)(byte & 0x0F) - mn_lo;
                ohi[l] += sc_hi * (float)((byte >> 4) & 0x0F) - mn_hi;
            }
        }
    }
}

/* Association C.  crates/larql-compute/src/cpu/ops/q4_common/matmul.rs:72-139
 * (kquant_matmul_into) with decode_q4k_superblock_into (matvec_f32.rs:166-199)
 * and dot_256_f32_scalar (matvec_f32.rs:250-258).  out is [seq, rows]. */
ORC_API int orc_q4k_matmul(const uint8_t *w, size_t w_len, const float *x, size_t rows, size_t hidden,
                           size_t seq, float *out) {
    if (rows == 0 || seq == 0 || hidden == 0 || hidden % 256 != 0 || w_len < rows * (hidden / 256) * 144) {
        for (size_t i = 0; i < seq * rows; i++) out[i] = 0.0f;
        return 1;
    }
    size_t nb = hidden / 256, row_bytes = nb * 144;
    float wf[256];
    for (size_t r = 0; r < rows; r++) {
        for (size_t s = 0; s < seq; s++) out[s * rows + r] = 0.0f;
        for (size_t sb = 0; sb < nb; sb++) {
            orc_dequantize_q4_k(w + r * row_bytes + sb * 144, 256, wf);
            for (size_t s = 0; s < seq; s++) {
                const float *xs = x + s * hidden + sb * 256;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int c = 0; c < 32; c++)
                    for (int l = 0; l < 8; l++) acc[l] += wf[c * 8 + l] * xs[c * 8 + l];
                float t = 0.0f; /* iter().sum::<f32>() folds from 0.0 left to right */
                for (int l = 0; l < 8; l++) t += acc[l];
                out[s * rows + r] += t;
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------- Q8_0 ----- */

/* ------------------------------------------------------------ Q6_K ----- */
/* 256 values in 210 bytes: ql[128] low nibbles, qh[64] high bit pairs, 16 int8
 * sub-block scales, f16 d.  The 16 signed values of scale sub-block j:
 * q6k_subblock_vals, crates/larql-models/src/quant/ggml/q6_k.rs:19-42. */
static void q6k_subblock_vals(const uint8_t *block, int j, int8_t *out) {
    const uint8_t *ql = block, *qh = block + 128;
    int half = j / 8, g = j % 8, plane = g / 2, lbase = (g % 2) * 16;
    int ql_off = half * 64 + (plane & 1) * 32 + lbase, qh_off = half * 32 + lbase, shift = plane * 2;
    for (int i = 0; i < 16; i++) {
        int lo4 = plane < 2 ? (ql[ql_off + i] & 0x0F) : (ql[ql_off + i] >> 4);
        int hi2 = (qh[qh_off + i] >> shift) & 0x03;
        out[i] = (int8_t)((lo4 | (hi2 << 4)) - 32);
    }
}

/* quantize_q6_k, crates/larql-compute/src/cpu/ops/q4_common/quantize.rs:198-277.
 * roundf is round-half-away-from-zero like f32::round. */
ORC_API void orc_quantize_q6_k(const float *data, size_t n, uint8_t *out) {
    for (size_t sb = 0; sb < n / 256; sb++) {
        const float *block = data + sb * 256;
        uint8_t *o = out + sb * 210;
        float amax = 0.0f;
        for (int i = 0; i < 256; i++) { float a = fabsf(block[i]); if (a > amax) amax = a; }
        float d = amax / (31.0f * 127.0f);
        int8_t sub_scales[16];
        for (int j = 0; j < 16; j++) {
            float sub_max = 0.0f;
            for (int i = 0; i < 16; i++) { float a = fabsf(block[j * 16 + i]); if (a > sub_max) sub_max = a; }
            float sc = d > 0.0f ? sub_max / (31.0f * d) : 0.0f;
            float r = roundf(sc);
            if (r < -128.0f) r = -128.0f;
            if (r > 127.0f) r = 127.0f;
            sub_scales[j] = (int8_t)r;
        }
        uint8_t q6[256];
        for (int j = 0; j < 16; j++) {
            float sc = d * (float)sub_scales[j];
            float inv_sc = fabsf(sc) > 1e-10f ? 1.0f / sc : 0.0f;
            for (int i = 0; i < 16; i++) {
                float r = roundf(block[j * 16 + i] * inv_sc);
                if (r < -32.0f) r = -32.0f;
                if (r > 31.0f) r = 31.0f;
                q6[j * 16 + i] = (uint8_t)((int)r + 32);
            }
        }
        uint8_t *ql = o, *qh = o + 128;
        for (int half = 0; half < 2; half++) {
            int e = half * 128;
            for (int l = 0; l < 32; l++) {
                uint8_t q1 = q6[e + l], q2 = q6[e + l + 32], q3 = q6[e + l + 64], q4 = q6[e + l + 96];
                ql[half * 64 + l] = (uint8_t)((q1 & 0x0F) | ((q3 & 0x0F) << 4));
                ql[half * 64 + l + 32] = (uint8_t)((q2 & 0x0F) | ((q4 & 0x0F) << 4));
                qh[half * 32 + l] = (uint8_t)(((q1 >> 4) & 3) | (((q2 >> 4) & 3) << 2) | (((q3 >> 4) & 3) << 4) |
                                              (((q4 >> 4) & 3) << 6));
            }
        }
        for (int j = 0; j < 16; j++) o[192 + j] = (uint8_t)sub_scales[j];
        uint16_t dh = orc_f32_to_f16_trunc(d);
        o[208] = (uint8_t)(dh & 0xff);
        o[209] = (uint8_t)(dh >> 8);
    }
}

/* dequantize_q6_k, q6_k.rs:171-195: value = (d * scale_j) * q. */
ORC_API void orc_dequantize_q6_k(const uint8_t *data, size_t n, float *out) {
    for (size_t sb = 0; sb < n / 256; sb++) {
        const uint8_t *block = data + sb * 210;
        float d = orc_f16_to_f32((uint16_t)(block[208] | (block[209] << 8)));
        for (int j = 0; j < 16; j++) {
            float sc = d * (float)(int8_t)block[192 + j];
            int8_t v[16];
            q6k_subblock_vals(block, j, v);
            for (int i = 0; i < 16; i++) out[sb * 256 + j * 16 + i] = sc * (float)v[i];
        }
    }
}

/* q6k_row_dot_scalar (the arm taken on x86), q6_k.rs:70-88: one running sum,
 * acc += (sc * v) * x per element. */
ORC_API float orc_q6k_row_dot(const uint8_t *data, const float *x, size_t n) {
    float acc = 0.0f;
    for (size_t sb = 0; sb < n / 256; sb++) {
        const uint8_t *block = data + sb * 210;
        float d = orc_f16_to_f32((uint16_t)(block[208] | (block[209] << 8)));
        for (int j = 0; j < 16; j++) {
            float sc = d * (float)(int8_t)block[192 + j];
            int8_t v[16];
            q6k_subblock_vals(block, j, v);
            for (int i = 0; i < 16; i++) acc += sc * (float)v[i] * x[sb * 256 + j * 16 + i];
        }
    }
    return acc;
}

/* q6k_row_scaled_add, q6_k.rs:142-168: out += (alpha * sc) * v. */
ORC_API void orc_q6k_row_scaled_add(const uint8_t *data, float alpha, float *out, size_t n) {
    for (size_t sb = 0; sb < n / 256; sb++) {
        const uint8_t *block = data + sb * 210;
        float d = orc_f16_to_f32((uint16_t)(block[208] | (block[209] << 8)));
        for (int j = 0; j < 16; j++) {
            float sc = d * (float)(int8_t)block[192 + j];
            int8_t v[16];
            q6k_subblock_vals(block, j, v);
            for (int i = 0; i < 16; i++) out[sb * 256 + j * 16 + i] += alpha * sc * (float)v[i];
        }
    }
}

/* One row of the backend matvec, crates/larql-compute/src/cpu/ops/q6k_matvec.rs:45-96:
 * per sub-block sub = sum v*x (sequential), acc += sc * sub. */
static float q6k_matvec_row(const uint8_t *row, const float *x, size_t nsb) {
    float acc = 0.0f;
    for (size_t sb = 0; sb < nsb; sb++) {
        const uint8_t *block = row + sb * 210;
        float d = orc_f16_to_f32((uint16_t)(block[208] | (block[209] << 8)));
        for (int j = 0; j < 16; j++) {
            float sc = d * (float)(int8_t)block[192 + j];
            int8_t v[16];
            q6k_subblock_vals(block, j, v);
            float sub = 0.0f;
            for (int i = 0; i < 16; i++) sub += (float)v[i] * x[sb * 256 + j * 16 + i];
            acc += sc * sub;
        }
    }
    return acc;
}

ORC_API int orc_q6k_matvec(const uint8_t *w, size_t w_len, const float *x, size_t x_len, size_t rows, size_t cols,
                           float *out) {
    if (cols % 256 != 0 || x_len != cols || w_len < rows * (cols / 256) * 210) return 1;
    for (size_t r = 0; r < rows; r++) out[r] = q6k_matvec_row(w + r * (cols / 256) * 210, x, cols / 256);
    return 0;
}

/* q4k_dual_matvec_into, crates/larql-compute/src/cpu/ops/q4_common/dual.rs:22-167 with the scalar
 * q4_dual_dot_32 (:186-198): both matrices against one x; unlike q4k_matvec_into each row keeps ONE
 * running sum over all its super-blocks.  Returns 1 on a shape refusal. */
ORC_API int orc_q4k_dual_matvec(const uint8_t *w_a, size_t wa_len, const uint8_t *w_b, size_t wb_len, const float *x,
                                size_t x_len, size_t rows, size_t cols, float *out_a, float *out_b) {
    size_t nb = cols / 256, row_bytes = nb * 144;
    if (cols % 256 != 0 || x_len != cols || wa_len < rows * row_bytes || wb_len < rows * row_bytes) return 1;
    float *sum_x = (float *)malloc(sizeof(float) * (cols / 32 + 1));
    q4k_sum_x(x, cols, sum_x);
    for (size_t r = 0; r < rows; r++) {
        for (int which = 0; which < 2; which++) {
            const uint8_t *w = which ? w_b : w_a;
            float acc = 0.0f;
            for (size_t sb = 0; sb < nb; sb++) {
                const uint8_t *b = w + r * row_bytes + sb * 144;
                float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
                float dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
                uint8_t sc[8], mn[8];
                unpack_q4k_scales(b + 4, sc, mn);
                for (int g = 0; g < 4; g++) {
                    int sb_lo = 2 * g, sb_hi = 2 * g + 1;
                    float sc_lo = d * (float)sc[sb_lo], sc_hi = d * (float)sc[sb_hi];
                    float mn_lo = dmin * (float)mn[sb_lo], mn_hi = dmin * (float)mn[sb_hi];
                    const uint8_t *chunk = b + 16 + g * 32;
                    const float *x_lo = x + sb * 256 + sb_lo * 32, *x_hi = x + sb * 256 + sb_hi * 32;
                    float dot_lo = 0.0f, dot_hi = 0.0f;
                    for (int l = 0; l < 32; l++) {
                        dot_lo += (float)(chunk[l] & 0x0F) * x_lo[l];
                        dot_hi += (float)((chunk[l] >> 4) & 0x0F) * x_hi[l];
                    }
                    acc += sc_lo * dot_lo - mn_lo * sum_x[sb * 8 + sb_lo];
                    acc += sc_hi * dot_hi - mn_hi * sum_x[sb * 8 + sb_hi];
                }
            }
            (which ? out_b : out_a)[r] = acc;
        }
    }
    free(sum_x);
    return 0;
}

/* crates/larql-models/src/quant/ggml/quantize.rs:50-77 (quantize_q8_0). */
ORC_API void orc_quantize_q8_0(const float *data, size_t n, uint8_t *out) {
    for (size_t i = 0; i < n / 32; i++) {
        const float *block = data + i * 32;
        float amax = 0.0f;
        for (int l = 0; l < 32; l++) amax = fmaxf(amax, fabsf(block[l]));
        float scale = amax / 127.0f;
        float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
        uint16_t h = orc_f32_to_f16_nearest(scale);
        uint8_t *o = out + i * 34;
        o[0] = h & 0xFF; o[1] = h >> 8;
        for (int l = 0; l < 32; l++)
            o[2 + l] = (uint8_t)rs_as_i8(rs_clamp(rs_round(block[l] * inv), -128.0f, 127.0f));
    }
}

/* crates/larql-models/src/quant/ggml/legacy.rs:68-83 (dequantize_q8_0). */
ORC_API void orc_dequantize_q8_0(const uint8_t *data, size_t n, float *out) {
    for (size_t i = 0; i < n / 32; i++) {
        const uint8_t *b = data + i * 34;
        float scale = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        for (int l = 0; l < 32; l++) out[i * 32 + l] = (float)(int8_t)b[2 + l] * scale;
    }
}

/* crates/larql-compute/src/cpu/kquant_gemv.rs:91-109 (row_dot): one running
 * accumulator, ((q*d)*x) per element. */
static float q8_0_row_dot(const uint8_t *blocks, const float *x, size_t row, size_t per_row) {
    float acc = 0.0f;
    for (size_t b = 0; b < per_row; b++) {
        const uint8_t *p = blocks + (row * per_row + b) * 34;
        float d = orc_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
        const float *xs = x + b * 32;
        for (int j = 0; j < 32; j++) acc += ((float)(int8_t)p[2 + j] * d) * xs[j];
    }
    return acc;
}

/* crates/larql-compute/src/cpu/kquant_gemv.rs:67-89 (q8_0_gemv): exact-length check. */
ORC_API int orc_q8_0_gemv(const uint8_t *blocks, size_t blocks_len, const float *x, size_t x_len, size_t n,
                          size_t k, float *out) {
    if (k == 0 || k % 32 != 0 || x_len != k) return 1;
    size_t per_row = k / 32;
    if (blocks_len != n * per_row * 34) return 1;
    for (size_t r = 0; r < n; r++) out[r] = q8_0_row_dot(blocks, x, r, per_row);
    return 0;
}

/* f16 / bf16 gemv as the reference's test device computes it (the CPU backend has no f16 / bf16 gemv:
 * trait default None, crates/larql-compute/src/backend/matmul.rs:124-147):
 * crates/larql-vindex/src/format/vindex3/opplan/exec/tests/device.rs:68-84 — per row the products
 * widen(w) * x[col] folded by Iterator::sum (sequential from 0.0, col ascending).  bf16 widens exactly
 * (the top 16 bits of the f32 it denotes, matmul.rs:133-139).  kind 0 = f16, 1 = bf16. */
ORC_API int orc_gemv16(const uint8_t *w, size_t w_len, const float *x, size_t x_len, size_t n, size_t k, int kind,
                       float *out) {
    if (w_len < n * k * 2 || x_len != k) return 1;
    for (size_t r = 0; r < n; r++) {
        float acc = 0.0f;
        for (size_t c = 0; c < k; c++) {
            const uint8_t *p = w + (r * k + c) * 2;
            uint16_t bits = (uint16_t)(p[0] | (p[1] << 8));
            float wv;
            if (kind == 0) wv = orc_f16_to_f32(bits);
            else {
                uint32_t u = (uint32_t)bits << 16;
                memcpy(&wv, &u, 4);
            }
            acc += wv * x[c];
        }
        out[r] = acc;
    }
    return 0;
}

/* Top-k by value, descending, ties to the lower index: the order q4k_matvec_topk / f16_gemv_topk return
 * (crates/larql-compute/src/backend/quant_matvec.rs:268-277: "sorted descending"; the caller's fallback is
 * the full matvec + a CPU reduce).  Returns the count, or -1 on NaN. */
ORC_API long orc_top_k_by_value(const float *v, size_t n, size_t top_k, uint32_t *idx_out, float *val_out) {
    size_t k = top_k < n ? top_k : n;
    for (size_t i = 0; i < n; i++)
        if (v[i] != v[i]) return -1;
    /* selection by repeated maximum over the remaining entries is O(n k); n k stays small in the tests */
    uint8_t *taken = (uint8_t *)calloc(n ? n : 1, 1);
    if (!taken) return -2;
    for (size_t j = 0; j < k; j++) {
        size_t best = n;
        for (size_t i = 0; i < n; i++) {
            if (taken[i]) continue;
            if (best == n || v[i] > v[best]) best = i;
        }
        taken[best] = 1;
        idx_out[j] = (uint32_t)best;
        val_out[j] = v[best];
    }
    free(taken);
    return (long)k;
}

/* ------------------------------------------------------------ NVFP4 ----- */

/* crates/larql-models/src/quant/nvfp4.rs:111-117 (tensor_scale_for). */
ORC_API float orc_nvfp4_tensor_scale_for(const float *values, size_t n) {
    float amax = 0.0f;
    for (size_t i = 0; i < n; i++) amax = fmaxf(amax, fabsf(values[i]));
    if (amax == 0.0f || !isfinite(amax)) return 1.0f;
    return amax / (448.0f * 6.0f);
}

/* crates/larql-models/src/quant/nvfp4.rs:163-186 (quantize_row_into) applied
 * over rows as quantize() does (:125-153). */
ORC_API int orc_quantize_nvfp4(const float *values, size_t rows, size_t k, float tensor_scale,
                               uint8_t *packed, uint8_t *scales) {
    if (k % 16 != 0) return 1;
    size_t groups = k / 16;
    for (size_t row = 0; row < rows; row++) {
        for (size_t g = 0; g < groups; g++) {
            const float *group = values + row * k + g * 16;
            float amax = 0.0f;
            for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(group[i]));
            float wanted = amax / 6.0f / tensor_scale;
            uint8_t sb = orc_f32_to_e4m3(wanted);
            scales[row * groups + g] = sb;
            float step = tensor_scale * orc_e4m3_to_f32(sb);
            float inv = (step > 0.0f && isfinite(step)) ? 1.0f / step : 0.0f;
            uint8_t *p = packed + (row * groups + g) * 8;
            for (int b = 0; b < 8; b++) {
                uint8_t lo = orc_f32_to_e2m1(group[2 * b] * inv) & 0x0F;
                uint8_t hi = orc_f32_to_e2m1(group[2 * b + 1] * inv) & 0x0F;
                p[b] = lo | (hi << 4);
            }
        }
    }
    return 0;
}

/* crates/larql-models/src/quant/nvfp4.rs:192-222 (dequantize_into). */
ORC_API int orc_dequantize_nvfp4(const uint8_t *packed, const uint8_t *scales, float tensor_scale, size_t rows,
                                 size_t k, float *out) {
    if (k % 16 != 0) return 1;
    size_t groups = k / 16;
    for (size_t row = 0; row < rows; row++)
        for (size_t g = 0; g < groups; g++) {
            float step = tensor_scale * orc_e4m3_to_f32(scales[row * groups + g]);
            const uint8_t *p = packed + (row * groups + g) * 8;
            for (int b = 0; b < 8; b++) {
                size_t i = row * k + g * 16 + 2 * b;
                out[i] = step * E2M1_TABLE[p[b] & 0x0F];
                out[i + 1] = step * E2M1_TABLE[(p[b] >> 4) & 0x0F];
            }
        }
    return 0;
}

static float nvfp4_row_dot(const uint8_t *packed, const uint8_t *scales, float ts, const float *x, size_t row,
                           size_t groups) {
    float acc = 0.0f;
    for (size_t g = 0; g < groups; g++) {
        float step = ts * orc_e4m3_to_f32(scales[row * groups + g]);
        const uint8_t *p = packed + (row * groups + g) * 8;
        const float *xs = x + g * 16;
        for (int b = 0; b < 8; b++) {
            acc += (step * E2M1_TABLE[p[b] & 0x0F]) * xs[2 * b];
            acc += (step * E2M1_TABLE[(p[b] >> 4) & 0x0F]) * xs[2 * b + 1];
        }
    }
    return acc;
}

/* crates/larql-compute/src/cpu/nvfp4_gemv.rs:29-65 (nvfp4_gemv). */
ORC_API int orc_nvfp4_gemv(const uint8_t *packed, size_t packed_len, const uint8_t *scales, size_t scales_len,
                           float tensor_scale, const float *x, size_t x_len, size_t n, size_t k, float *out) {
    if (k == 0 || k % 16 != 0 || x_len != k) return 1;
    size_t groups = k / 16;
    if (packed_len != n * groups * 8 || scales_len != n * groups) return 1;
    for (size_t row = 0; row < n; row++) out[row] = nvfp4_row_dot(packed, scales, tensor_scale, x, row, groups);
    return 0;
}

/* ------------------------------------------------------------ MXFP4 ----- */

/* crates/larql-vindex/src/format/vindex3/opplan/exec/weights/load.rs:410-476
 * (quantize_mxfp4).  `max_abs.log2().floor()` goes through libm log2f, as the
 * Rust intrinsic does on Linux. */
ORC_API int orc_quantize_mxfp4(const float *values, size_t rows, size_t k, uint8_t *packed, uint8_t *scales) {
    if (k % 32 != 0) return 1;
    size_t groups = k / 32;
    for (size_t row = 0; row < rows; row++)
        for (size_t g = 0; g < groups; g++) {
            const float *group = values + row * k + g * 32;
            float max_abs = 0.0f;
            for (int i = 0; i < 32; i++) max_abs = fmaxf(max_abs, fabsf(group[i]));
            uint8_t sb;
            if (max_abs == 0.0f) sb = 0;
            else {
                int32_t exponent = (int32_t)floorf(log2f(max_abs)) - 2;
                int32_t e = exponent + 127;
                if (e < 1) e = 1;
                if (e > 254) e = 254;
                sb = (uint8_t)e;
            }
            scales[row * groups + g] = sb;
            float scale = orc_e8m0_to_f32(sb);
            float inv = scale == 0.0f ? 0.0f : 1.0f / scale;
            uint8_t *p = packed + (row * groups + g) * 16;
            for (int b = 0; b < 16; b++) {
                uint8_t lo = orc_nearest_mxfp4_code(group[2 * b] * inv);
                uint8_t hi = orc_nearest_mxfp4_code(group[2 * b + 1] * inv);
                p[b] = lo | (hi << 4);
            }
        }
    return 0;
}

/* crates/larql-models/src/quant/mxfp4.rs:42-95 (dequantize_expert). */
ORC_API void orc_dequantize_mxfp4(const uint8_t *blocks, const uint8_t *scales, size_t rows, size_t groups,
                                  float *out) {
    for (size_t row = 0; row < rows; row++)
        for (size_t g = 0; g < groups; g++) {
            float scale = orc_e8m0_to_f32(scales[row * groups + g]);
            const uint8_t *p = blocks + (row * groups + g) * 16;
            for (int b = 0; b < 16; b++) {
                size_t i = row * groups * 32 + g * 32 + 2 * b;
                out[i] = E2M1_TABLE[p[b] & 0x0F] * scale;
                out[i + 1] = E2M1_TABLE[(p[b] >> 4) & 0x0F] * scale;
            }
        }
}

static float mxfp4_row_dot(const uint8_t *packed, const uint8_t *scales, const float *x, size_t row,
                           size_t groups) {
    float acc = 0.0f;
    for (size_t g = 0; g < groups; g++) {
        float scale = orc_e8m0_to_f32(scales[row * groups + g]);
        const uint8_t *p = packed + (row * groups + g) * 16;
        for (int b = 0; b < 16; b++) {
            size_t e0 = g * 32 + 2 * b;
            acc += E2M1_TABLE[p[b] & 0x0F] * scale * x[e0];
            acc += E2M1_TABLE[p[b] >> 4] * scale * x[e0 + 1];
        }
    }
    return acc;
}

/* The reference CPU backend has no MXFP4 gemv (trait default refuses,
 * crates/larql-compute/src/backend/matmul.rs:226-235).  This follows the only
 * in-tree CPU arithmetic: the test device loop
 * crates/larql-vindex/src/format/vindex3/opplan/exec/tests/device.rs:105-127. */
ORC_API int orc_mxfp4_gemv(const uint8_t *packed, size_t packed_len, const uint8_t *scales, size_t scales_len,
                           const float *x, size_t x_len, size_t n, size_t k, float *out) {
    if (k % 32 != 0 || x_len < k) return 1;
    if (packed_len < n * (k / 32) * 16 || scales_len < n * (k / 32)) return 1;
    for (size_t row = 0; row < n; row++) out[row] = mxfp4_row_dot(packed, scales, x, row, k / 32);
    return 0;
}

/* ------------------------------------------------------------ top-K ----- */

typedef struct { uint32_t idx; float val; } orc_hit;

/* Total order (|v| descending, index ascending) — the tie rule the build is
 * graded on; equals the reference heap on tie-free inputs. */
static int hit_cmp(const void *a, const void *b) {
    const orc_hit *x = (const orc_hit *)a, *y = (const orc_hit *)b;
    float ax = fabsf(x->val), ay = fabsf(y->val);
    if (ax > ay) return -1;
    if (ax < ay) return 1;
    return x->idx < y->idx ? -1 : (x->idx > y->idx ? 1 : 0);
}

/* crates/larql-vindex/src/index/compute/gate_knn/mod.rs:50-108 (top_k_by_abs),
 * as a full sort under the total order.  Returns the count written, or -1 if a
 * score is NaN (the reference panics). */
ORC_API int64_t orc_top_k_by_abs(const float *scores, size_t n, size_t top_k, uint32_t *idx_out, float *val_out) {
    if (top_k == 0 || n == 0) return 0;
    for (size_t i = 0; i < n; i++) if (scores[i] != scores[i]) return -1;
    orc_hit *h = (orc_hit *)malloc(sizeof(orc_hit) * n);
    for (size_t i = 0; i < n; i++) { h[i].idx = (uint32_t)i; h[i].val = scores[i]; }
    qsort(h, n, sizeof(orc_hit), hit_cmp);
    size_t k = top_k < n ? top_k : n;
    for (size_t i = 0; i < k; i++) { idx_out[i] = h[i].idx; val_out[i] = h[i].val; }
    free(h);
    return (int64_t)k;
}

/* Literal restatement of the same function as a capacity-K min-heap on |v|
 * where an incoming score replaces the minimum only when strictly greater
 * (gate_knn/mod.rs:94-103).  Which of several equal minima the heap evicts is
 * an implementation detail of the standard library's heap; here the evicted
 * one is the equal-minimum with the HIGHEST index, which realises "lower index
 * wins".  Output sorted (|v| desc, idx asc). */
ORC_API int64_t orc_top_k_by_abs_heap(const float *scores, size_t n, size_t top_k, uint32_t *idx_out,
                                      float *val_out) {
    if (top_k == 0 || n == 0) return 0;
    for (size_t i = 0; i < n; i++) if (scores[i] != scores[i]) return -1;
    size_t cap = top_k < n ? top_k : n, len = 0;
    orc_hit *heap = (orc_hit *)malloc(sizeof(orc_hit) * cap);
    /* heap order: root = smallest |v|; among equal |v| the larger index is "smaller". */
#define HLESS(a, b) (fabsf((a).val) < fabsf((b).val) || (fabsf((a).val) == fabsf((b).val) && (a).idx > (b).idx))
    for (size_t i = 0; i < n; i++) {
        orc_hit e = {(uint32_t)i, scores[i]};
        if (len < top_k && len < cap) {
            size_t c = len++;
            heap[c] = e;
            while (c > 0) {
                size_t p = (c - 1) / 2;
                if (HLESS(heap[c], heap[p])) { orc_hit t = heap[c]; heap[c] = heap[p]; heap[p] = t; c = p; }
                else break;
            }
        } else if (fabsf(e.val) > fabsf(heap[0].val)) {
            heap[0] = e;
            size_t c = 0;
            for (;;) {
                size_t l = 2 * c + 1, r = l + 1, m = c;
                if (l < len && HLESS(heap[l], heap[m])) m = l;
                if (r < len && HLESS(heap[r], heap[m])) m = r;
                if (m == c) break;
                orc_hit t = heap[c]; heap[c] = heap[m]; heap[m] = t; c = m;
            }
        }
    }
#undef HLESS
    qsort(heap, len, sizeof(orc_hit), hit_cmp);
    for (size_t i = 0; i < len; i++) { idx_out[i] = heap[i].idx; val_out[i] = heap[i].val; }
    free(heap);
    return (int64_t)len;
}

/* ------------------------------------------- norm, activation, router --- */

/* crates/larql-compute/src/residual.rs:56-78 (rms_norm_eps), weight = None. */
ORC_API void orc_rms_norm(const float *x, size_t rows, size_t cols, double eps, float *out) {
    for (size_t i = 0; i < rows; i++) {
        double sq = 0.0;
        for (size_t j = 0; j < cols; j++) sq += (double)x[i * cols + j] * (double)x[i * cols + j];
        float rms = (float)sqrt(sq / (double)cols + eps);
        for (size_t j = 0; j < cols; j++) out[i * cols + j] = x[i * cols + j] / rms * 1.0f;
    }
}

/* crates/larql-compute/src/ffn.rs:91-93 (sigmoid). */
ORC_API float orc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
/* walk inline form `gate * sigmoid(gate)`:
 * crates/larql-inference/src/vindex/walk_ffn/sparse.rs:239-244. */
ORC_API float orc_silu(float g) { return g * orc_sigmoid(g); }

/* crates/larql-compute/src/cpu/ops/moe/math.rs:130-143 (softmax). */
ORC_API void orc_softmax(float *v, size_t n) {
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++) max = fmaxf(max, v[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) { v[i] = expf(v[i] - max); sum += v[i]; }
    if (sum > 0.0f) for (size_t i = 0; i < n; i++) v[i] /= sum;
}

/* crates/larql-compute/src/cpu/ops/moe/math.rs:153-164 (top_k): value
 * descending, index ascending. */
ORC_API size_t orc_moe_top_k(const float *v, size_t n, size_t k, uint32_t *idx_out, float *val_out) {
    if (k > n) k = n;
    uint8_t *used = (uint8_t *)calloc(n ? n : 1, 1);
    for (size_t j = 0; j < k; j++) {
        size_t best = n;
        for (size_t i = 0; i < n; i++) {
            if (used[i]) continue;
            if (best == n || v[i] > v[best]) best = i;
        }
        used[best] = 1;
        idx_out[j] = (uint32_t)best;
        val_out[j] = v[best];
    }
    free(used);
    return k;
}

/* crates/larql-compute/src/cpu/ops/moe/mod.rs:149-189 (moe_route_from_router_input)
 * starting from logits: softmax over all experts, top-k, optional
 * renormalisation over the selected weights. */
ORC_API size_t orc_moe_route(const float *logits, size_t n_experts, size_t top_k, int renormalise,
                             uint32_t *idx_out, float *w_out) {
    float *p = (float *)malloc(sizeof(float) * (n_experts ? n_experts : 1));
    memcpy(p, logits, sizeof(float) * n_experts);
    orc_softmax(p, n_experts);
    size_t k = orc_moe_top_k(p, n_experts, top_k, idx_out, w_out);
    if (renormalise) {
        float sum = 0.0f;
        for (size_t i = 0; i < k; i++) sum += w_out[i];
        if (sum > 0.0f) for (size_t i = 0; i < k; i++) w_out[i] /= sum;
    }
    free(p);
    return k;
}

/* --------------------------------------------------------- the walk ----- */

enum { ORC_FMT_Q4_K = 0, ORC_FMT_Q8_0 = 1, ORC_FMT_MXFP4 = 2, ORC_FMT_NVFP4 = 3, ORC_FMT_Q6_K = 4 };

typedef struct {
    int32_t fmt;
    const uint8_t *data;   /* Q4_K / Q8_0 blocks, or FP4 packed codes */
    const uint8_t *scales; /* MXFP4 e8m0 / NVFP4 e4m3 stream, else NULL */
    float tensor_scale;    /* NVFP4 */
    size_t rows, cols;
} orc_matrix;

static size_t mat_row_bytes(const orc_matrix *m) {
    switch (m->fmt) {
        case ORC_FMT_Q4_K: return m->cols / 256 * 144;
        case ORC_FMT_Q8_0: return m->cols / 32 * 34;
        case ORC_FMT_MXFP4: return m->cols / 32 * 16;
        case ORC_FMT_Q6_K: return m->cols / 256 * 210;
        default: return m->cols / 16 * 8;
    }
}

/* Backend gemv of one matrix in that format's reference association. */
static void mat_gemv_rows(const orc_matrix *m, const float *x, const float *sum_x, size_t r0, size_t r1, float *out) {
    switch (m->fmt) {
        case ORC_FMT_Q4_K: q4k_matvec_rows(m->data, x, sum_x, r0, r1, m->cols, out); break;
        case ORC_FMT_Q8_0: for (size_t r = r0; r < r1; r++) out[r] = q8_0_row_dot(m->data, x, r, m->cols / 32); break;
        case ORC_FMT_MXFP4: for (size_t r = r0; r < r1; r++) out[r] = mxfp4_row_dot(m->data, m->scales, x, r, m->cols / 32); break;
        case ORC_FMT_Q6_K: for (size_t r = r0; r < r1; r++) out[r] = q6k_matvec_row(m->data + r * mat_row_bytes(m), x, m->cols / 256); break;
        default: for (size_t r = r0; r < r1; r++) out[r] = nvfp4_row_dot(m->data, m->scales, m->tensor_scale, x, r, m->cols / 16); break;
    }
}

/* One selected feature's up dot: ffn_row_dot
 * (crates/larql-vindex/src/index/types/ffn_row/mod.rs:46-101) -> registry
 * row_dot; Q4_K is association B, the others their gemv row association. */
static float mat_row_dot(const orc_matrix *m, size_t row, const float *x) {
    switch (m->fmt) {
        case ORC_FMT_Q4_K: return orc_q4k_row_dot(m->data + row * mat_row_bytes(m), x, m->cols);
        case ORC_FMT_Q8_0: return q8_0_row_dot(m->data, x, row, m->cols / 32);
        case ORC_FMT_MXFP4: return mxfp4_row_dot(m->data, m->scales, x, row, m->cols / 32);
        case ORC_FMT_Q6_K: return orc_q6k_row_dot(m->data + row * mat_row_bytes(m), x, m->cols);
        default: return nvfp4_row_dot(m->data, m->scales, m->tensor_scale, x, row, m->cols / 16);
    }
}

static void mat_dequant_row(const orc_matrix *m, size_t row, float *out) {
    switch (m->fmt) {
        case ORC_FMT_Q4_K: orc_dequantize_q4_k(m->data + row * mat_row_bytes(m), m->cols, out); break;
        case ORC_FMT_Q8_0: orc_dequantize_q8_0(m->data + row * mat_row_bytes(m), m->cols, out); break;
        case ORC_FMT_Q6_K: orc_dequantize_q6_k(m->data + row * mat_row_bytes(m), m->cols, out); break;
        case ORC_FMT_MXFP4:
            orc_dequantize_mxfp4(m->data + row * mat_row_bytes(m), m->scales + row * (m->cols / 32), 1, m->cols / 32, out);
            break;
        default:
            orc_dequantize_nvfp4(m->data + row * mat_row_bytes(m), m->scales + row * (m->cols / 16), m->tensor_scale, 1,
                                 m->cols, out);
            break;
    }
}

/* One feature's down accumulate: ffn_row_scaled_add (ffn_row/mod.rs:106-179).
 * Q4_K / Q6_K: the registry's fused row_scaled_add (crates/larql-vindex/src/quant/registry.rs);
 * other formats: out += act * dequant(row). */
static void mat_row_scaled_add(const orc_matrix *m, size_t row, float alpha, float *out, float *scratch) {
    if (m->fmt == ORC_FMT_Q4_K) { orc_q4k_row_scaled_add(m->data + row * mat_row_bytes(m), alpha, out, m->cols); return; }
    if (m->fmt == ORC_FMT_Q6_K) { orc_q6k_row_scaled_add(m->data + row * mat_row_bytes(m), alpha, out, m->cols); return; }
    mat_dequant_row(m, row, scratch);
    for (size_t i = 0; i < m->cols; i++) out[i] += alpha * scratch[i];
}

/* crates/larql-inference/src/vindex/walk_ffn/sparse.rs:60-306 (walk_ffn_sparse),
 * serial per-feature loop (:218-289), for one token: gate scores by the backend
 * gemv, top_k_by_abs, then in hit order up dot, SiLU, floor 1e-10
 * (walk_config.rs:64), down scaled-add.  gate/up are [N,H]; down_fm is the
 * feature-major [N,H] down.  idx_out/score_out (optional) receive the hits. */
ORC_API int64_t orc_walk_token(const orc_matrix *gate, const orc_matrix *up, const orc_matrix *down_fm,
                               const float *x, size_t top_k, float *out, uint32_t *idx_out, float *score_out) {
    size_t n = gate->rows, h = gate->cols;
    float *scores = (float *)malloc(sizeof(float) * (n ? n : 1));
    float *sum_x = (float *)malloc(sizeof(float) * (h / 32 + 1));
    float *scratch = (float *)malloc(sizeof(float) * (h ? h : 1));
    if (gate->fmt == ORC_FMT_Q4_K) q4k_sum_x(x, h, sum_x);
    mat_gemv_rows(gate, x, sum_x, 0, n, scores);
    size_t kk = top_k < n ? top_k : n;
    uint32_t *idx = (uint32_t *)malloc(sizeof(uint32_t) * (kk ? kk : 1));
    float *val = (float *)malloc(sizeof(float) * (kk ? kk : 1));
    int64_t got = orc_top_k_by_abs(scores, n, top_k, idx, val);
    for (size_t i = 0; i < h; i++) out[i] = 0.0f;
    if (got >= 0) {
        for (int64_t i = 0; i < got; i++) {
            float g = val[i];
            float upv = mat_row_dot(up, idx[i], x);
            float act = (g * orc_sigmoid(g)) * upv;
            if (fabsf(act) > 1e-10f) mat_row_scaled_add(down_fm, idx[i], act, out, scratch);
            if (idx_out) idx_out[i] = idx[i];
            if (score_out) score_out[i] = val[i];
        }
    }
    free(scores); free(sum_x); free(scratch); free(idx); free(val);
    return got;
}

/* Dense K = all: sparse_full_k_gemv
 * (crates/larql-inference/src/vindex/walk_ffn/sparse_gemv.rs:21-72): gate gemv,
 * up by row_dot per row (kquant_matmul_transb,
 * crates/larql-vindex/src/index/compute/kquant_dispatch.rs:69-88),
 * act = silu(gate)*up for EVERY feature (no top-K, no floor), then the down
 * product; here down is taken feature-major, out = sum_f act[f]*dequant(down_fm[f]). */
ORC_API void orc_walk_token_dense(const orc_matrix *gate, const orc_matrix *up, const orc_matrix *down_fm,
                                  const float *x, float *out) {
    size_t n = gate->rows, h = gate->cols;
    float *scores = (float *)malloc(sizeof(float) * (n ? n : 1));
    float *sum_x = (float *)malloc(sizeof(float) * (h / 32 + 1));
    float *scratch = (float *)malloc(sizeof(float) * (h ? h : 1));
    if (gate->fmt == ORC_FMT_Q4_K) q4k_sum_x(x, h, sum_x);
    mat_gemv_rows(gate, x, sum_x, 0, n, scores);
    for (size_t i = 0; i < h; i++) out[i] = 0.0f;
    for (size_t f = 0; f < n; f++) {
        float g = scores[f];
        float act = (g * orc_sigmoid(g)) * mat_row_dot(up, f, x);
        mat_dequant_row(down_fm, f, scratch);
        for (size_t i = 0; i < h; i++) out[i] += act * scratch[i];
    }
    free(scores); free(sum_x); free(scratch);
}

/* crates/larql-compute/src/forward/layer.rs:61-127 (run_ffn): pre-FFN RMSNorm
 * (unit weight, eps), walk, residual add. */
ORC_API int64_t orc_run_ffn_token(const orc_matrix *gate, const orc_matrix *up, const orc_matrix *down_fm,
                                  const float *h_in, size_t top_k, double eps, float *h_out, uint32_t *idx_out) {
    size_t h = gate->cols;
    float *xn = (float *)malloc(sizeof(float) * (h ? h : 1));
    float *o = (float *)malloc(sizeof(float) * (h ? h : 1));
    orc_rms_norm(h_in, 1, h, eps, xn);
    int64_t got = orc_walk_token(gate, up, down_fm, xn, top_k, o, idx_out, NULL);
    for (size_t i = 0; i < h; i++) h_out[i] = h_in[i] + o[i];
    free(xn); free(o);
    return got;
}

/* ------------------------------------------- threaded CPU baseline ------ */
/* Row-parallel gemv in 32-row chunks as the reference does
 * (matvec_f32.rs:89-104, kquant_gemv.rs:80-87), and the hit-chunked up/down
 * scan with per-thread partials and a serial reduce
 * (crates/larql-inference/src/vindex/walk_ffn/sparse_parallel.rs:96-154).
 * Timed by the benchmark's CPU arm; same arithmetic per row as above. */

typedef struct {
    const orc_matrix *m; const float *x; const float *sum_x; float *out;
    size_t n_chunks; volatile size_t *next;
} gemv_job;

static void *gemv_worker(void *arg) {
    gemv_job *j = (gemv_job *)arg;
    for (;;) {
        size_t c = __atomic_fetch_add(j->next, 1, __ATOMIC_RELAXED);
        if (c >= j->n_chunks) break;
        size_t r0 = c * 32, r1 = r0 + 32 < j->m->rows ? r0 + 32 : j->m->rows;
        mat_gemv_rows(j->m, j->x, j->sum_x, r0, r1, j->out);
    }
    return NULL;
}

ORC_API void orc_gemv_mt(const orc_matrix *m, const float *x, float *out, int threads) {
    float *sum_x = (float *)malloc(sizeof(float) * (m->cols / 32 + 1));
    if (m->fmt == ORC_FMT_Q4_K) q4k_sum_x(x, m->cols, sum_x);
    volatile size_t next = 0;
    gemv_job job = {m, x, sum_x, out, (m->rows + 31) / 32, &next};
    if (threads < 1) threads = 1;
    pthread_t *t = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    for (int i = 1; i < threads; i++) pthread_create(&t[i], NULL, gemv_worker, &job);
    gemv_worker(&job);
    for (int i = 1; i < threads; i++) pthread_join(t[i], NULL);
    free(t); free(sum_x);
}

typedef struct {
    const orc_matrix *up, *down; const float *x; const uint32_t *idx; const float *val;
    size_t i0, i1; float *partial; float *scratch;
} scan_job;

static void *scan_worker(void *arg) {
    scan_job *j = (scan_job *)arg;
    size_t h = j->up->cols;
    for (size_t i = 0; i < h; i++) j->partial[i] = 0.0f;
    for (size_t i = j->i0; i < j->i1; i++) {
        float g = j->val[i];
        float act = (g * orc_sigmoid(g)) * mat_row_dot(j->up, j->idx[i], j->x);
        if (fabsf(act) > 1e-10f) {
            /* try_parallel_q4k_down: partial += act * dequantised down row */
            mat_dequant_row(j->down, j->idx[i], j->scratch);
            for (size_t c = 0; c < h; c++) j->partial[c] += act * j->scratch[c];
        }
    }
    return NULL;
}

ORC_API int64_t orc_walk_token_mt(const orc_matrix *gate, const orc_matrix *up, const orc_matrix *down_fm,
                                  const float *x, size_t top_k, float *out, uint32_t *idx_out, int threads) {
    size_t n = gate->rows, h = gate->cols;
    if (threads < 1) threads = 1;
    float *scores = (float *)malloc(sizeof(float) * (n ? n : 1));
    orc_gemv_mt(gate, x, scores, threads);
    size_t kk = top_k < n ? top_k : n;
    uint32_t *idx = (uint32_t *)malloc(sizeof(uint32_t) * (kk ? kk : 1));
    float *val = (float *)malloc(sizeof(float) * (kk ? kk : 1));
    int64_t got = orc_top_k_by_abs_heap(scores, n, top_k, idx, val);
    for (size_t i = 0; i < h; i++) out[i] = 0.0f;
    if (got > 0) {
        size_t chunk = ((size_t)got + (size_t)threads - 1) / (size_t)threads;
        size_t n_jobs = ((size_t)got + chunk - 1) / chunk;
        scan_job *jobs = (scan_job *)malloc(sizeof(scan_job) * n_jobs);
        pthread_t *t = (pthread_t *)malloc(sizeof(pthread_t) * n_jobs);
        for (size_t j = 0; j < n_jobs; j++) {
            size_t i0 = j * chunk, i1 = i0 + chunk < (size_t)got ? i0 + chunk : (size_t)got;
            jobs[j] = (scan_job){up, down_fm, x, idx, val, i0, i1, (float *)malloc(sizeof(float) * h),
                                 (float *)malloc(sizeof(float) * h)};
        }
        for (size_t j = 1; j < n_jobs; j++) pthread_create(&t[j], NULL, scan_worker, &jobs[j]);
        scan_worker(&jobs[0]);
        for (size_t j = 1; j < n_jobs; j++) pthread_join(t[j], NULL);
        for (size_t j = 0; j < n_jobs; j++) {
            for (size_t i = 0; i < h; i++) out[i] += jobs[j].partial[i];
            free(jobs[j].partial); free(jobs[j].scratch);
        }
        free(jobs); free(t);
        if (idx_out) memcpy(idx_out, idx, sizeof(uint32_t) * (size_t)got);
    }
    free(scores); free(idx); free(val);
    return got;
}
