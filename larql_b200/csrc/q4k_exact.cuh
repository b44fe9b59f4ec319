// One Q4_K row in the reference CPU backend's exact f32 order (Association A:
// process_q4k_superblock, crates/larql-compute/src/cpu/ops/q4_common/matvec_f32.rs:116-155,
// with the scalar q4_dual_dot_32, .../q4_common/dual.rs:186-198), computed by one warp.
#pragma once
#include "common.cuh"

namespace lq {

// xs: the activation in shared memory, 64-float chunks at a stride of 68 floats so that the
// eight lanes of a 128-bit load phase (chunks 64 floats apart) fall in different banks.
// IN_SMEM: the row was staged in shared memory (plain loads); otherwise it is read from global memory through
// the read-only path.
// The super-block partials of the passes first_pass, first_pass + pass_step, ... of a row (a pass is eight
// super-blocks, one per group of four lanes) into sb_part[]: super-blocks are independent of each other until the
// final sum, so several warps may share a row.
template <bool IN_SMEM = false>
__device__ __forceinline__ void exact_row_q4k_passes(const uint8_t* __restrict__ row, const float* __restrict__ xs, int nsb,
                                                     float* sb_part /* [nsb] */, int lane, int first_pass, int pass_step) {
    const int g = lane & 3;
    auto ld16 = [](const uint8_t* p) -> uint4 {
        return IN_SMEM ? *reinterpret_cast<const uint4*>(p) : __ldg(reinterpret_cast<const uint4*>(p));
    };
    // The loads of the next eight super-blocks are issued before the current eight are summed, so the
    // passes of a row overlap their memory latency (the arithmetic and its order are unchanged).
    uint4 n_hdr = make_uint4(0u, 0u, 0u, 0u), n_q0 = n_hdr, n_q1 = n_hdr;
    const int sb_step = 8 * pass_step;
    if (8 * first_pass + (lane >> 2) < nsb) {
        const uint8_t* cell = row + (size_t)(8 * first_pass + (lane >> 2)) * 144;
        n_hdr = ld16(cell);
        n_q0 = ld16(cell + 16 + g * 32);
        n_q1 = ld16(cell + 32 + g * 32);
    }
#pragma unroll 1
    for (int s0 = 8 * first_pass; s0 < nsb; s0 += sb_step) {
        const int s = s0 + (lane >> 2);
        const uint4 hdr = n_hdr, q0 = n_q0, q1 = n_q1;
        if (s + sb_step < nsb) {
            const uint8_t* cell = row + (size_t)(s + sb_step) * 144;
            n_hdr = ld16(cell);
            n_q0 = ld16(cell + 16 + g * 32);
            n_q1 = ld16(cell + 32 + g * 32);
        }
        float u_lo = 0.0f, u_hi = 0.0f;
        if (s < nsb) {
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const float* x_lo = xs + (s * 4 + g) * 68;
            const float* x_hi = x_lo + 32;
            float dot_lo = 0.0f, dot_hi = 0.0f, sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 xl = *reinterpret_cast<const float4*>(x_lo + 4 * j);
                const float4 xh = *reinterpret_cast<const float4*>(x_hi + 4 * j);
                const float xls[4] = {xl.x, xl.y, xl.z, xl.w}, xhs[4] = {xh.x, xh.y, xh.z, xh.w};
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint32_t byte = (qw[j] >> (8 * b)) & 0xffu;
                    dot_lo = __fadd_rn(dot_lo, __fmul_rn((float)(byte & 0x0fu), xls[b]));
                    dot_hi = __fadd_rn(dot_hi, __fmul_rn((float)(byte >> 4), xhs[b]));
                    sum_lo = __fadd_rn(sum_lo, xls[b]);
                    sum_hi = __fadd_rn(sum_hi, xhs[b]);
                }
            }
            const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
            uint32_t sc2, m2;
            q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
            const float sc_lo = __fmul_rn(d, (float)(sc2 & 0xff)), sc_hi = __fmul_rn(d, (float)(sc2 >> 8));
            const float mn_lo = __fmul_rn(dmin, (float)(m2 & 0xff)), mn_hi = __fmul_rn(dmin, (float)(m2 >> 8));
            u_lo = __fsub_rn(__fmul_rn(sc_lo, dot_lo), __fmul_rn(mn_lo, sum_lo));
            u_hi = __fsub_rn(__fmul_rn(sc_hi, dot_hi), __fmul_rn(mn_hi, sum_hi));
        }
        // Super-block partial: acc = 0; for g in 0..4 { acc += u_lo(g); acc += u_hi(g) }.
        const int base = lane & ~3;
        float acc = 0.0f;
#pragma unroll
        for (int gg = 0; gg < 4; ++gg) {
            const float a = __shfl_sync(0xffffffffu, u_lo, base + gg);
            const float b = __shfl_sync(0xffffffffu, u_hi, base + gg);
            acc = __fadd_rn(acc, a);
            acc = __fadd_rn(acc, b);
        }
        if (g == 0 && s < nsb) sb_part[s] = acc;
    }
}

// The whole row by one warp: all passes, then the partials summed in super-block order (valid on lane 0).
template <bool IN_SMEM = false>
__device__ __forceinline__ float exact_row_q4k(const uint8_t* __restrict__ row, const float* __restrict__ xs, int nsb,
                                               float* sb_part /* [nsb] per-warp scratch */, int lane) {
    exact_row_q4k_passes<IN_SMEM>(row, xs, nsb, sb_part, lane, 0, 1);
    __syncwarp();
    float total = 0.0f;
    if (lane == 0)
        for (int s = 0; s < nsb; ++s) total = __fadd_rn(total, sb_part[s]);
    __syncwarp();
    return total;  // valid on lane 0
}

}  // namespace lq
