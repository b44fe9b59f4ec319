// Device-side scalar decoders shared by the kernels (exact, table-free where possible).
#pragma once
#include "common.cuh"

namespace lq {

// FP4 E2M1 code -> f32: {0,.5,1,1.5,2,3,4,6} with the sign in bit 3; -0.0 is kept
// (crates/larql-models/src/quant/fp4.rs:19-21).
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
    const uint32_t mag = code & 7u, e = mag >> 1, m = mag & 1u;
    // normal: (1 + m/2) * 2^(e-1); subnormal (e == 0): m * 0.5
    const uint32_t bits = e ? (((e + 126u) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
    return __uint_as_float(bits | ((code & 8u) << 28));
}

// E8M0 scale byte -> f32 (crates/larql-models/src/quant/mxfp4.rs:27-35).
__device__ __forceinline__ float e8m0_to_f32(uint32_t byte) {
    if (byte == 0u) return 0.0f;
    if (byte == 255u) return __uint_as_float(0x7FC00000u);
    return __uint_as_float(byte << 23);
}

// FP8 E4M3 byte -> f32 (crates/larql-models/src/quant/fp8.rs:33-56): bias 7, subnormals
// m * 2^-9, 0x7F / 0xFF are NaN, no infinities.
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
    const uint32_t sign = (byte & 0x80u) << 24, exp = (byte >> 3) & 0x0Fu, mant = byte & 7u;
    if (exp == 0x0Fu && mant == 7u) return __uint_as_float(0x7FC00000u);
    if (exp == 0u) return __uint_as_float(__float_as_uint((float)mant * 0.001953125f) | sign);
    return __uint_as_float(sign | ((exp + 120u) << 23) | (mant << 20));
}

// Q4_K 6-bit scale and min of sub-block j from the 12 packed bytes (get_scale_min_k4;
// crates/larql-models/src/quant/ggml/q4_k.rs:92-104).
__device__ __forceinline__ void q4k_scale_min(const uint8_t* p, int j, uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = p[j] & 0x3Fu;
        m = p[j + 4] & 0x3Fu;
    } else {
        sc = (p[j + 4] & 0x0Fu) | ((uint32_t)(p[j - 4] >> 6) << 4);
        m = (uint32_t)(p[j + 4] >> 4) | ((uint32_t)(p[j] >> 6) << 4);
    }
}

}  // namespace lq
