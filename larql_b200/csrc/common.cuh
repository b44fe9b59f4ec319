// Shared device helpers for the walk kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lq {

// Device-side error codes written to the context's error word (first writer wins).
enum DevErr : int {
    DEV_OK = 0,
    DEV_ERR_TMA_TIMEOUT = 1,   // a bounded mbarrier wait ran out
    DEV_ERR_NAN_SCORE = 2,     // a gate score was NaN (the reference panics there)
    DEV_ERR_INTERNAL = 3,
};

__device__ __forceinline__ void set_err(int* err, int code) {
    if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier + TMA bulk copy (global -> this CTA's shared memory) -------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Both addresses 16-byte aligned, bytes a multiple of 16 (callers guarantee it).
__device__ __forceinline__ void tma_bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same with a suspend-time hint: the hardware may park the thread for up to `ns` nanoseconds
// (it is woken when the phase completes), so a waiting warp does not spend issue slots and
// shared-memory bandwidth on polling while its neighbours work.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^31 clocks (about a second) and reports it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0; it < (1u << 26); ++it) {
        if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
        if (clock64() - t0 > (1ll << 31)) break;
    }
    return false;
}

// ---- small numeric helpers --------------------------------------------------
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xffffu)));
}
// u8 x s8 and u8 x u8 four-way dot products with 32-bit accumulate.
__device__ __forceinline__ int dp4a_us(uint32_t a_u8, uint32_t b_s8, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_s8), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a_u8, uint32_t b_u8, int c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_u8), "r"(c));
    return static_cast<int>(d);
}
__device__ __forceinline__ int dp4a_ss(uint32_t a_s8, uint32_t b_s8, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8), "r"(b_s8), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a_s8, uint32_t b_u8, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8), "r"(b_u8), "r"(c));
    return d;
}

// Q4_K: the 6-bit (scale, min) pairs of sub-blocks 2g and 2g+1 from the 12 packed
// bytes (three little-endian words h1,h2,h3), two at a time (get_scale_min_k4).
// Returns sc_lo | sc_hi<<8 in sc2 and m_lo | m_hi<<8 in m2.
__device__ __forceinline__ void q4k_pair_scales(uint32_t h1, uint32_t h2, uint32_t h3, int g, uint32_t& sc2,
                                                uint32_t& m2) {
    const int sh = 16 * (g & 1);
    const bool low = g < 2;
    const uint32_t A16 = ((low ? h1 : h2) >> sh) & 0xffffu;  // scales16[g]
    const uint32_t B16 = ((low ? h2 : h3) >> sh) & 0xffffu;  // scales16[g+2]
    const uint32_t C16 = (h1 >> sh) & 0xffffu;               // scales16[g-2] when g >= 2
    sc2 = low ? (A16 & 0x3f3fu) : ((B16 & 0x0f0fu) | ((C16 & 0xc0c0u) >> 2));
    m2 = low ? (B16 & 0x3f3fu) : (((B16 >> 4) & 0x0f0fu) | ((A16 & 0xc0c0u) >> 2));
}

// Prepared activation for one token: the f32 vector plus a 16-bit fixed-point copy
// per 32-element block, split in a signed high byte plane and an unsigned low byte
// plane so integer dot products run as dp4a.
//   x ~= scale[blk] * (256 * a + b),  a in [-128,127], b in [0,255]
struct XPrep {
    const float* xn;        // [H] activation actually multiplied (after the optional RMSNorm)
    const uint32_t* xa;     // [H/4] high-byte plane, four consecutive elements per word
    const uint32_t* xb;     // [H/4] low-byte plane
    const float* scale;     // [H/32] fixed-point step per block
    const float* sum;       // [H/32] sum of the block's x
    const float* abs;       // [H/32] sum of the block's |x|
};

// Worst-case |x_hat - x| per element in units of the block's step (rint + two roundings).
#define LQ_XQ_ERR_STEPS 0.52f

}  // namespace lq
