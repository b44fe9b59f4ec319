// Device-side Q4_K quantiser: the reference's quantize_q4_k
// (crates/larql-compute/src/cpu/ops/q4_common/quantize.rs:89-189) with its truncating,
// subnormal-keeping f32->f16 (…/q4_common/f16.rs:10-41), one thread per super-block.
// Every operation is the reference's, in its order, with no fused multiply-add, so the
// bytes equal the CPU encoder's.  Used to build synthetic layers directly in HBM.
#include "kernels.h"

namespace lq {

namespace {

__device__ __forceinline__ uint32_t f32_to_f16_trunc(float val) {
    const uint32_t bits = __float_as_uint(val);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const int exp = (int)((bits >> 23) & 0xFFu);
    const uint32_t mant = bits & 0x7FFFFFu;
    if (exp == 0) return sign;
    if (exp == 255) return sign | 0x7C00u | (mant >> 13);
    const int new_exp = exp - 127 + 15;
    if (new_exp >= 31) return sign | 0x7C00u;
    if (new_exp <= 0) {
        const int shift = 1 - new_exp;
        if (13 + shift >= 24) return sign;
        return sign | ((mant | 0x800000u) >> (13 + shift));
    }
    return sign | ((uint32_t)new_exp << 10) | (mant >> 13);
}

// round half away from zero, clamp, cast (f32::round().clamp(lo,hi) as u8)
__device__ __forceinline__ uint32_t round_clamp_u8(float v, float hi) {
    float r = roundf(v);
    if (!(r == r)) return 0u;
    r = fminf(fmaxf(r, 0.0f), hi);
    return (uint32_t)r;
}

__global__ void quantize_q4k_kernel(const float* __restrict__ data, size_t n_sb, uint8_t* __restrict__ out) {
    const size_t sb = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (sb >= n_sb) return;
    const float* block = data + sb * 256;
    uint8_t* o = out + sb * 144;
    float sub_min[8], sub_max[8];
    for (int j = 0; j < 8; ++j) {
        float mn = INFINITY, mx = -INFINITY;
        for (int l = 0; l < 32; ++l) {
            const float v = block[j * 32 + l];
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        sub_min[j] = fminf(mn, 0.0f);
        sub_max[j] = fmaxf(mx, 0.0f);
    }
    float gmr = 0.0f, gmin = INFINITY;
    for (int j = 0; j < 8; ++j) {
        gmr = fmaxf(gmr, __fsub_rn(sub_max[j], sub_min[j]));
        gmin = fminf(gmin, sub_min[j]);
    }
    const float d = gmr > 0.0f ? __fdiv_rn(gmr, 15.0f * 63.0f) : 0.0f;
    const float dmin = gmin < 0.0f ? __fdiv_rn(-gmin, 63.0f) : 0.0f;
    const uint32_t dh = f32_to_f16_trunc(d), dmh = f32_to_f16_trunc(dmin);
    uint32_t qs[8], qm[8];
    for (int j = 0; j < 8; ++j) {
        const float range = __fsub_rn(sub_max[j], sub_min[j]);
        qs[j] = d > 0.0f ? round_clamp_u8(__fdiv_rn(range, __fmul_rn(15.0f, d)), 63.0f) : 0u;
        qm[j] = dmin > 0.0f ? round_clamp_u8(__fdiv_rn(-sub_min[j], dmin), 63.0f) : 0u;
    }
    uint32_t w[36];  // 144 bytes, little-endian words
    w[0] = dh | (dmh << 16);
    uint8_t packed[12];
    for (int j = 0; j < 4; ++j) {
        packed[j] = (uint8_t)((qs[j] & 0x3F) | (((qs[j + 4] >> 4) & 0x03) << 6));
        packed[j + 4] = (uint8_t)((qm[j] & 0x3F) | (((qm[j + 4] >> 4) & 0x03) << 6));
        packed[j + 8] = (uint8_t)((qs[j + 4] & 0x0F) | ((qm[j + 4] & 0x0F) << 4));
    }
    for (int k = 0; k < 3; ++k)
        w[1 + k] = packed[4 * k] | (packed[4 * k + 1] << 8) | (packed[4 * k + 2] << 16) | ((uint32_t)packed[4 * k + 3] << 24);
    for (int g = 0; g < 4; ++g) {
        const float sc_lo = __fmul_rn(d, (float)qs[2 * g]), sc_hi = __fmul_rn(d, (float)qs[2 * g + 1]);
        const float mn_lo = __fmul_rn(dmin, (float)qm[2 * g]), mn_hi = __fmul_rn(dmin, (float)qm[2 * g + 1]);
        const float inv_lo = sc_lo > 0.0f ? __fdiv_rn(1.0f, sc_lo) : 0.0f;
        const float inv_hi = sc_hi > 0.0f ? __fdiv_rn(1.0f, sc_hi) : 0.0f;
        const float* lo_sub = block + (2 * g) * 32;
        const float* hi_sub = lo_sub + 32;
        for (int l4 = 0; l4 < 8; ++l4) {
            uint32_t word = 0;
            for (int b = 0; b < 4; ++b) {
                const int l = 4 * l4 + b;
                const uint32_t lo = round_clamp_u8(__fmul_rn(__fadd_rn(lo_sub[l], mn_lo), inv_lo), 15.0f);
                const uint32_t hi = round_clamp_u8(__fmul_rn(__fadd_rn(hi_sub[l], mn_hi), inv_hi), 15.0f);
                word |= (lo | (hi << 4)) << (8 * b);
            }
            w[4 + g * 8 + l4] = word;
        }
    }
    uint4* o4 = reinterpret_cast<uint4*>(o);  // 144-byte blocks from a 16-byte aligned base
    for (int k = 0; k < 9; ++k) o4[k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}

}  // namespace

cudaError_t launch_quantize_q4k(const float* data, size_t n_elems, uint8_t* out, cudaStream_t st) {
    const size_t n_sb = n_elems / 256;
    if (n_sb == 0) return cudaSuccess;
    quantize_q4k_kernel<<<(unsigned)((n_sb + 127) / 128), 128, 0, st>>>(data, n_sb, out);
    return cudaGetLastError();
}

}  // namespace lq
