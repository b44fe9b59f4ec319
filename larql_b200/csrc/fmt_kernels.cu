// Gate scan, exact re-score and gather for the block formats other than Q4_K:
// ggml Q8_0, MXFP4 and NVFP4.  Same pipeline as Q4_K (fast score + rigorous bound, exact
// reference-order re-score of the boundary band, SiLU-gated gather), simpler kernels.
//
// Reference arithmetic (one running f32 accumulator over the whole row, element order):
//   Q8_0  : acc += ((q as f32) * d) * x[j]            crates/larql-compute/src/cpu/kquant_gemv.rs:91-109
//   NVFP4 : acc += ((ts * e4m3(s)) * e2m1(c)) * x[j]   crates/larql-compute/src/cpu/nvfp4_gemv.rs:48-62
//   MXFP4 : acc += (e2m1(c) * 2^(e-127)) * x[j]        crates/larql-vindex/src/format/vindex3/opplan/exec/
//                                                       tests/device.rs:105-127 (the reference CPU
//                                                       backend has no MXFP4 gemv)
// The fast scan takes the same products in any order (Q8_0: integer dp4a dots against the
// fixed-point activation planes; FP4: f32 FMAs with the code table held across a warp's lanes
// and read by shuffle); the exact kernel runs one thread per row in the reference's order with
// separate multiply and add.
#include "../../include/larql_cuda.h"
#include "codecs.cuh"
#include "kernels.h"

namespace lq {

namespace {

constexpr int FK_THREADS = 256;
constexpr float FK_NOISE_FLOOR = 1e-10f;

__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 2 * e2m1 magnitude per code, sign in bit 3: {0,.5,1,1.5,2,3,4,6}
__device__ __forceinline__ float fp4_lut_lane(int lane) { return e2m1_to_f32((uint32_t)lane & 15u); }

// One warp: fast dot of row `row` with the prepared activation; also the row's bound on
// |fast - reference|: c1 sum |w x| (for the FP4 formats the sum itself, accumulated beside the dot; for
// Q8_0 an upper estimate plus the fixed-point error term).  c1 covers the roundings of the reference's
// one running sum over the row and of this evaluation; sum |w x| here is itself rounded, which the 1 %
// margin in c1 absorbs.
// xs_pad (optional, FP4 formats): the activation in shared memory, every 32-element block at a stride of 36
// floats.  A lane reads the 32 (or 16) activations of ITS block: from global memory that is 32 lines per warp load,
// from an unpadded copy a 32-way bank conflict; at a stride of 36 the eight lanes of a 128-bit load phase fall into
// different banks.
template <int FMT>
__device__ __forceinline__ float fast_row(const FmtMat& m, size_t row, const XPrep& xp, float c1, float& bound, int lane,
                                          float lut, const float* xs_pad = nullptr) {
    float acc = 0.0f, bnd = 0.0f;
    if (FMT == LQ_FMT_Q8_0) {
        const int nb = m.cols / 32;
        for (int blk = lane; blk < nb; blk += 32) {
            const uint16_t* p = reinterpret_cast<const uint16_t*>(m.data + ((size_t)row * nb + blk) * 34);
            const float d = f16_bits_to_f32(p[0]);
            int ia = 0, ib = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t w = (uint32_t)p[1 + 2 * j] | ((uint32_t)p[2 + 2 * j] << 16);
                ia = dp4a_ss(w, xp.xa[blk * 8 + j], ia);
                ib = dp4a_su(w, xp.xb[blk * 8 + j], ib);
            }
            const float step = xp.scale[blk];
            acc += d * (step * (float)(ia * 256 + ib));
            bnd += fabsf(d) * (c1 * 128.0f * xp.abs[blk] + 128.0f * 32.0f * LQ_XQ_ERR_STEPS * step);
        }
    } else if (FMT == LQ_FMT_MXFP4) {
        const int nb = m.cols / 32;
        for (int b0 = 0; b0 < nb; b0 += 32) {  // all lanes iterate together: the table read is a shuffle
            const int blk = b0 + lane;
            const bool on = blk < nb;
            uint4 q = make_uint4(0, 0, 0, 0);
            float scale = 0.0f;
            if (on) {
                q = *reinterpret_cast<const uint4*>(m.data + ((size_t)row * nb + blk) * 16);
                scale = e8m0_to_f32(m.scales[(size_t)row * nb + blk]);
            }
            const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
            float s = 0.0f, sa = 0.0f;  // sum w x and sum |w x| of the block (before the scale)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 x0 = make_float4(0, 0, 0, 0), x1 = x0;
                if (on) {
                    const float* xsrc = xs_pad ? xs_pad + blk * 36 + 8 * j : xp.xn + blk * 32 + 8 * j;
                    x0 = *reinterpret_cast<const float4*>(xsrc);
                    x1 = *reinterpret_cast<const float4*>(xsrc + 4);
                }
                const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float t = __shfl_sync(0xffffffffu, lut, (qw[j] >> (4 * e)) & 15u);
                    s = fmaf(t, xs[e], s);
                    sa = fmaf(fabsf(t), fabsf(xs[e]), sa);
                }
            }
            if (on) {
                acc += s * scale;
                bnd += c1 * fabsf(scale) * sa;
            }
        }
    } else {  // NVFP4: groups of 16
        const int ng = m.cols / 16;
        for (int g0 = 0; g0 < ng; g0 += 32) {
            const int g = g0 + lane;
            const bool on = g < ng;
            uint2 q = make_uint2(0, 0);
            float step = 0.0f;
            if (on) {
                q = *reinterpret_cast<const uint2*>(m.data + ((size_t)row * ng + g) * 8);
                step = m.ts * e4m3_to_f32(m.scales[(size_t)row * ng + g]);
            }
            const uint32_t qw[2] = {q.x, q.y};
            float s = 0.0f, sa = 0.0f;  // sum w x and sum |w x| of the group (before the scale)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float4 x0 = make_float4(0, 0, 0, 0), x1 = x0;
                if (on) {
                    const float* xsrc = xs_pad ? xs_pad + (g >> 1) * 36 + (g & 1) * 16 + 8 * j : xp.xn + g * 16 + 8 * j;
                    x0 = *reinterpret_cast<const float4*>(xsrc);
                    x1 = *reinterpret_cast<const float4*>(xsrc + 4);
                }
                const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float t = __shfl_sync(0xffffffffu, lut, (qw[j] >> (4 * e)) & 15u);
                    s = fmaf(t, xs[e], s);
                    sa = fmaf(fabsf(t), fabsf(xs[e]), sa);
                }
            }
            if (on) {
                acc += s * step;
                bnd += c1 * fabsf(step) * sa;
            }
        }
    }
    bound = warp_sum(bnd);
    return warp_sum(acc);
}

template <int FMT>
__global__ void __launch_bounds__(FK_THREADS) scan_fmt_kernel(FmtMat m, XPrep xp, float* __restrict__ scores,
                                                             uint32_t* __restrict__ hist,
                                                             uint32_t* __restrict__ bound_bits, float c1, int* err) {
    const int lane = threadIdx.x & 31;
    const int warp_g = (blockIdx.x * FK_THREADS + threadIdx.x) >> 5, n_warps = (gridDim.x * FK_THREADS) >> 5;
    const float lut = fp4_lut_lane(lane);
    float bmax = 0.0f;
    for (int row = warp_g; row < m.rows; row += n_warps) {
        float b;
        const float s = fast_row<FMT>(m, (size_t)row, xp, c1, b, lane, lut);
        if (lane == 0) {
            scores[row] = s;
            if (hist) {
                if (s != s) set_err(err, DEV_ERR_NAN_SCORE);
                atomicAdd(&hist[__float_as_uint(fabsf(s)) >> LQ_HIST_SHIFT], 1u);
                bmax = fmaxf(bmax, b);
            }
        }
    }
    if (hist && lane == 0 && bmax > 0.0f) atomicMax(bound_bits, __float_as_uint(bmax));
}

// One thread per listed row, the reference's element order, no fused multiply-add.
template <int FMT>
__device__ float exact_row_fmt(const FmtMat& m, size_t row, const float* __restrict__ x) {
    float acc = 0.0f;
    if (FMT == LQ_FMT_Q8_0) {
        const int nb = m.cols / 32;
        for (int b = 0; b < nb; ++b) {
            const uint8_t* p = m.data + (row * nb + b) * 34;
            const float d = f16_bits_to_f32((uint32_t)p[0] | ((uint32_t)p[1] << 8));
            for (int j = 0; j < 32; ++j)
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn((float)(int8_t)p[2 + j], d), x[b * 32 + j]));
        }
    } else if (FMT == LQ_FMT_MXFP4) {
        const int nb = m.cols / 32;
        for (int g = 0; g < nb; ++g) {
            const float scale = e8m0_to_f32(m.scales[row * nb + g]);
            const uint8_t* p = m.data + (row * nb + g) * 16;
            for (int b = 0; b < 16; ++b) {
                const uint32_t byte = p[b];
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(e2m1_to_f32(byte & 15u), scale), x[g * 32 + 2 * b]));
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(e2m1_to_f32(byte >> 4), scale), x[g * 32 + 2 * b + 1]));
            }
        }
    } else {
        const int ng = m.cols / 16;
        for (int g = 0; g < ng; ++g) {
            const float step = __fmul_rn(m.ts, e4m3_to_f32(m.scales[row * ng + g]));
            const uint8_t* p = m.data + (row * ng + g) * 8;
            for (int b = 0; b < 8; ++b) {
                const uint32_t byte = p[b];
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(step, e2m1_to_f32(byte & 15u)), x[g * 16 + 2 * b]));
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(step, e2m1_to_f32(byte >> 4)), x[g * 16 + 2 * b + 1]));
            }
        }
    }
    return acc;
}

template <int FMT>
__global__ void rescore_fmt_kernel(FmtMat m, const float* __restrict__ xn, const uint32_t* __restrict__ rows_idx,
                                   const int* __restrict__ n_rows_dev, int n_rows_host, float* __restrict__ out) {
    const int n = n_rows_dev ? min(*n_rows_dev, m.rows) : n_rows_host;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const size_t r = rows_idx ? rows_idx[i] : (size_t)i;
        out[i] = exact_row_fmt<FMT>(m, r, xn);
    }
}

// Exact-order scan: one thread per row walks the row in the reference's element order (one running
// f32 sum, separate multiplies and add), so the scores ARE the reference's scores and the top-K
// needs no bound, band or re-score.  The sum over a row cannot be split without changing its bits;
// rows are the parallelism (one row per thread, the activation broadcast from shared memory, each
// thread streaming its own row with 16-byte loads that the L1 turns into whole lines).
template <int FMT>
__device__ __forceinline__ void scan_exact_fmt_body(const FmtMat& m, const float* __restrict__ xn,
                                                    float* __restrict__ scores, int* err) {
    extern __shared__ __align__(16) float xs[];  // [cols], then the scale bytes of this CTA's rows (FP4 formats)
    for (int i = threadIdx.x; i < m.cols; i += blockDim.x) xs[i] = xn[i];
    // A row's scale bytes sit hidden / 32 (or / 16) bytes apart from the next row's: read per thread, every load
    // would touch 32 sectors for 32 bytes.  The rows of a CTA are consecutive, so their scales are one contiguous
    // run: copied once, coalesced.
    uint8_t* sc_s = reinterpret_cast<uint8_t*>(xs + m.cols);
    const int nsc = FMT == LQ_FMT_MXFP4 ? m.cols / 32 : (FMT == LQ_FMT_NVFP4 ? m.cols / 16 : 0);
    if (FMT != LQ_FMT_Q8_0) {
        const int r0 = blockIdx.x * blockDim.x;
        const int n_sc = max(0, min((int)blockDim.x, m.rows - r0)) * nsc;
        const uint8_t* src = m.scales + (size_t)r0 * nsc;
        for (int i = threadIdx.x; i < n_sc; i += blockDim.x) sc_s[i] = src[i];
    }
    __syncthreads();
    const int row_raw = blockIdx.x * blockDim.x + threadIdx.x;
    if (row_raw - (int)(threadIdx.x & 31) >= m.rows) return;  // (a whole warp past the end)
    const int row = min(row_raw, m.rows - 1);  // lanes past the end redo the last row: the FP4 table read is a shuffle
    const float lut = fp4_lut_lane(threadIdx.x & 31);
    float acc = 0.0f;
    if (FMT == LQ_FMT_Q8_0) {
        const int nb = m.cols / 32;
        const uint16_t* p = reinterpret_cast<const uint16_t*>(m.data + (size_t)row * nb * 34);
        for (int b = 0; b < nb; ++b, p += 17) {
            const float d = f16_bits_to_f32(p[0]);
            uint32_t q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = (uint32_t)p[1 + 2 * j] | ((uint32_t)p[2 + 2 * j] << 16);
            const float4* xv = reinterpret_cast<const float4*>(xs + b * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 x4 = xv[j];
                const float xe[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float qf = (float)(int)(int8_t)(q[j] >> (8 * e));
                    acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(qf, d), xe[e]));
                }
            }
        }
    } else {
        // FP4 formats: 32 weights (16 bytes of codes) at a time.  A thread streams its own row, so a load touches 32
        // different lines of the matrix; two blocks (one whole 32-byte sector) are fetched together, one pair ahead
        // of the pair being summed.
        const int nb = m.cols / 32;
        const uint4* p = reinterpret_cast<const uint4*>(m.data + (size_t)row * nb * 16);
        const uint8_t* sc = sc_s + (size_t)(row - blockIdx.x * blockDim.x) * nsc;
        auto block = [&](const uint4& w, int b) {
            float s0, s1;
            if (FMT == LQ_FMT_MXFP4) {
                s0 = s1 = e8m0_to_f32(sc[b]);
            } else {
                s0 = __fmul_rn(m.ts, e4m3_to_f32(sc[2 * b]));
                s1 = __fmul_rn(m.ts, e4m3_to_f32(sc[2 * b + 1]));
            }
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            const float4* xv = reinterpret_cast<const float4*>(xs + b * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 xa4 = xv[2 * j], xb4 = xv[2 * j + 1];
                const float xe[8] = {xa4.x, xa4.y, xa4.z, xa4.w, xb4.x, xb4.y, xb4.z, xb4.w};
                const float s = j < 2 ? s0 : s1;
#pragma unroll
                for (int e = 0; e < 8; ++e) {  // nibble e of the word: low nibble of a byte first
                    const float v = __shfl_sync(0xffffffffu, lut, (int)(ww[j] >> (4 * e)));
                    // MXFP4 multiplies value * scale, NVFP4 scale * value: the same product either way
                    acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(v, s), xe[e]));
                }
            }
        };
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        // (an NVFP4 code stream is only promised 8-byte alignment: two 8-byte loads then)
        const bool al16 = (reinterpret_cast<uintptr_t>(p) & 15) == 0;
        auto ld = [&](int b) -> uint4 {
            if (al16) return p[b];
            const uint2* q = reinterpret_cast<const uint2*>(p) + 2 * b;
            const uint2 lo = q[0], hi = q[1];
            return make_uint4(lo.x, lo.y, hi.x, hi.y);
        };
        uint4 n0 = ld(0), n1 = nb > 1 ? ld(1) : zero;
        for (int b = 0; b < nb; b += 2) {
            const uint4 w0 = n0, w1 = n1;
            if (b + 2 < nb) n0 = ld(b + 2);
            if (b + 3 < nb) n1 = ld(b + 3);
            block(w0, b);
            if (b + 1 < nb) block(w1, b + 1);
        }
    }
    if (row_raw < m.rows) {
        scores[row] = acc;
        if (acc != acc) set_err(err, DEV_ERR_NAN_SCORE);
    }
}

template <int FMT>
__global__ void __launch_bounds__(64) scan_exact_fmt_kernel(FmtMat m, const float* __restrict__ xn,
                                                           float* __restrict__ scores, int* err) {
    scan_exact_fmt_body<FMT>(m, xn, scores, err);
}

// The same scan for many (token, expert) pairs of a mixture-of-experts layer in one launch: pair blockIdx.y
// scans the gate matrix of ITS expert (table[pair_expert[y]]) against its token's activation; workspaces of
// the pairs lie a constant stride apart.
template <int FMT>
__global__ void __launch_bounds__(64) scan_exact_pairs_kernel(const FmtMat* __restrict__ table,
                                                             const uint32_t* __restrict__ pair_expert, TokenWs ws0,
                                                             size_t ws_stride, int* err) {
    const FmtMat m = table[pair_expert[blockIdx.y]];
    const TokenWs ws = ws_at(ws0, ws_stride * blockIdx.y);
    scan_exact_fmt_body<FMT>(m, ws.xn, ws.scores, err);
}

// Exact-order scan, staged: the same arithmetic as scan_exact_fmt_kernel, but a warp brings the next
// 256 elements of its 32 rows into shared memory with coalesced 16-byte loads (rows are a power-of-two
// stride apart, which makes per-thread streaming thrash the L1 sets) and every lane then walks its own
// row's chunk from shared memory.  Needs cols % 256 == 0 and 16-byte aligned streams.
template <int FMT>
struct StagedGeom {
    static constexpr int CHB = FMT == LQ_FMT_Q8_0 ? 272 : 128;                           // data bytes per row and chunk
    static constexpr int SCB = FMT == LQ_FMT_NVFP4 ? 16 : (FMT == LQ_FMT_MXFP4 ? 8 : 0);  // scale bytes
    static constexpr int ROWB = CHB + (FMT == LQ_FMT_Q8_0 ? 32 : 16);                    // padded: shifts the banks per row
    static constexpr int WARP_BYTES = 32 * ROWB + 32 * 32;
    static constexpr int NBUF = FMT == LQ_FMT_Q8_0 ? 2 : 3;  // chunk buffers per warp (two CTAs of four warps fit an SM)
};

// Two IEEE round-to-nearest f32 multiplies in one instruction (sm_100 packed f32x2): {a0 * b0, a1 * b1}.
__device__ __forceinline__ void fmul2_rn(float a0, float a1, float b0, float b1, float& r0, float& r1) {
    asm("{\n\t.reg .b64 ra, rb, rr;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rr, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rr;\n\t}"
        : "=f"(r0), "=f"(r1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// The 32 reference products (decoded weight times activation, each rounded as the reference
// rounds it) of one 32-element block of a staged row chunk.  For the FP4 formats the code -> value table
// sits in the lanes of the warp (lane i holds the value of code i & 15, `lut`): a weight is decoded by one
// shuffle whose source lane is the word shifted down to the nibble (a shuffle takes its source lane modulo
// 32, and lanes 16..31 repeat the table), so every lane of the warp must call this together.
// CHAIN: the running sum takes the previous block's products (`prev`) in between, in the reference's order, so the
// dependent adds and the independent products alternate in program order.
template <int FMT, bool CHAIN = false>
__device__ __forceinline__ void block_products(const uint8_t* mine, const uint8_t* sc, float ts, int b, const float* xc,
                                               float lut, float (&p)[32], const float* prev = nullptr, float* acc_io = nullptr) {
    float acc = CHAIN ? *acc_io : 0.0f;
    float xe[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float4 x4 = *reinterpret_cast<const float4*>(xc + b * 32 + 4 * j);
        xe[4 * j] = x4.x; xe[4 * j + 1] = x4.y; xe[4 * j + 2] = x4.z; xe[4 * j + 3] = x4.w;
    }
    if (FMT == LQ_FMT_Q8_0) {
        const uint16_t* q = reinterpret_cast<const uint16_t*>(mine + b * 34);
        const float d = f16_bits_to_f32(q[0]);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t w = q[1 + j];
            const float n0 = __fmul_rn(__fmul_rn((float)(int)(int8_t)(w & 0xff), d), xe[2 * j]);
            const float n1 = __fmul_rn(__fmul_rn((float)(int)(int8_t)(w >> 8), d), xe[2 * j + 1]);
            if (CHAIN) {
                acc = __fadd_rn(acc, prev[2 * j]);
                acc = __fadd_rn(acc, prev[2 * j + 1]);
            }
            p[2 * j] = n0;
            p[2 * j + 1] = n1;
        }
    } else {
        const uint4 w = *reinterpret_cast<const uint4*>(mine + b * 16);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        float s0, s1;
        if (FMT == LQ_FMT_MXFP4) {
            s0 = s1 = e8m0_to_f32(sc[b]);
        } else {
            s0 = __fmul_rn(ts, e4m3_to_f32(sc[2 * b]));
            s1 = __fmul_rn(ts, e4m3_to_f32(sc[2 * b + 1]));
        }
        // all 32 table reads first, back to back: a shuffle answers after some 25 cycles, and nothing below depends
        // on more than its own two
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __shfl_sync(0xffffffffu, lut, (int)(ww[e >> 3] >> (4 * (e & 7))));
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const float s = e < 16 ? s0 : s1;
            float w0, w1, n0, n1;
            fmul2_rn(v[e], v[e + 1], s, s, w0, w1);  // (multiplication commutes: the reference's scale * value or value * scale)
            fmul2_rn(w0, w1, xe[e], xe[e + 1], n0, n1);
            if (CHAIN) {
                acc = __fadd_rn(acc, prev[e]);
                acc = __fadd_rn(acc, prev[e + 1]);
            }
            p[e] = n0;
            p[e + 1] = n1;
        }
    }
    if (CHAIN) *acc_io = acc;
}

__device__ __forceinline__ void cp_async16_f(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async8_f(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(128) scan_exact_staged_kernel(FmtMat m, const float* __restrict__ xn,
                                                               float* __restrict__ scores, int* err) {
    using SG = StagedGeom<FMT>;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* xs = reinterpret_cast<float*>(smem_raw);  // [cols]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* wbase = smem_raw + (size_t)m.cols * 4 + (size_t)warp * SG::NBUF * SG::WARP_BYTES;
    for (int i = threadIdx.x; i < m.cols; i += blockDim.x) xs[i] = xn[i];
    __syncthreads();
    const int row0 = (blockIdx.x * 4 + warp) * 32;
    if (row0 >= m.rows) return;
    const int row = row0 + lane;
    const int n_chunks = m.cols / 256;
    const size_t data_stride = (size_t)n_chunks * SG::CHB;
    const size_t sc_stride = (size_t)n_chunks * SG::SCB;
    constexpr int PIECES = SG::CHB / 16;  // 16-byte pieces per row and chunk
    // coalesced asynchronous copy of chunk c of this warp's 32 rows into buffer (c mod NBUF); past the end: an empty group
    auto stage = [&](int c) {
        uint8_t* wbuf = wbase + (c % SG::NBUF) * SG::WARP_BYTES;
        for (int p = lane; c < n_chunks && p < 32 * PIECES; p += 32) {
            const int r = p / PIECES, piece = p % PIECES;
            const int rr = min(row0 + r, m.rows - 1);
            cp_async16_f(wbuf + r * SG::ROWB + piece * 16, m.data + (size_t)rr * data_stride + (size_t)c * SG::CHB + piece * 16);
        }
        if (SG::SCB && c < n_chunks) {
            const int rr = min(row0 + lane, m.rows - 1);
            uint8_t* sdst = wbuf + 32 * SG::ROWB + lane * 32;
            const uint8_t* ssrc = m.scales + (size_t)rr * sc_stride + (size_t)c * SG::SCB;
            if (SG::SCB == 16) cp_async16_f(sdst, ssrc);
            else cp_async8_f(sdst, ssrc);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc = 0.0f;
    const float lut = fp4_lut_lane(lane);
    // NBUF - 1 chunks are in flight while one is summed.  The products of a block are formed while the running sum
    // takes the previous block's (across chunk borders too), so the chain of dependent adds never waits for them.
#pragma unroll
    for (int c = 0; c < SG::NBUF; ++c) stage(c);
    if (SG::NBUF == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncwarp();
    if (FMT != LQ_FMT_Q8_0) {
        // FP4 formats: a three-stage software pipeline over the row's 32-element blocks, two blocks per trip so that
        // the stages' registers swap roles without copies.  In one step
        //   S(B + 2): the codes and scales of block B + 2 leave shared memory and its 32 table shuffles are issued,
        //   P(B + 1): the two rounded multiplies of block B + 1 (its shuffles were issued a step ago),
        //   A(B):     the running sum takes block B's products, in the reference's order.
        // Nothing in a step waits for a shuffle or a load issued in the same step, and the chain of dependent
        // adds always has a step's worth of independent work beside it.
        const int n_blocks = n_chunks * 8;
        float va[32], vb[32], pa[32], pb[32];
        float sa0 = 0.f, sa1 = 0.f, sb0 = 0.f, sb1 = 0.f;
        // S: block B (all lanes together: the table read is a shuffle)
        auto S = [&](int B, float (&v)[32], float& s0, float& s1) {
            const int c = B >> 3, b = B & 7;
            if (b == 0) {  // the first block of a chunk: the chunk has landed (the later ones may be in flight)
                asm volatile("cp.async.wait_group 2;" ::: "memory");
                __syncwarp();
            }
            const uint8_t* wbuf = wbase + (c % SG::NBUF) * SG::WARP_BYTES;
            const uint4 w = *reinterpret_cast<const uint4*>(wbuf + lane * SG::ROWB + b * 16);
            const uint8_t* sc = wbuf + 32 * SG::ROWB + lane * 32;
            if (FMT == LQ_FMT_MXFP4) {
                s0 = s1 = e8m0_to_f32(sc[b]);
            } else {
                s0 = __fmul_rn(m.ts, e4m3_to_f32(sc[2 * b]));
                s1 = __fmul_rn(m.ts, e4m3_to_f32(sc[2 * b + 1]));
            }
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __shfl_sync(0xffffffffu, lut, (int)(ww[e >> 3] >> (4 * (e & 7))));
            if (b == 7) {  // the chunk's buffer is free: chunk c + NBUF goes into it
                __syncwarp();
                stage(c + SG::NBUF);
            }
        };
        // P: products of block B from its table values; A: the sum takes `prev` in between
        auto PA = [&](int B, const float (&v)[32], float s0, float s1, float (&pout)[32], const float (&prev)[32],
                      bool do_p, bool do_a) {
            const float* xc = xs + B * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                float n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f;
                if (do_p) {
                    const float4 x4 = *reinterpret_cast<const float4*>(xc + e);
                    const float s = e < 16 ? s0 : s1;
                    float w0, w1, w2, w3;
                    fmul2_rn(v[e], v[e + 1], s, s, w0, w1);
                    fmul2_rn(v[e + 2], v[e + 3], s, s, w2, w3);
                    fmul2_rn(w0, w1, x4.x, x4.y, n0, n1);
                    fmul2_rn(w2, w3, x4.z, x4.w, n2, n3);
                }
                if (do_a) {
                    acc = __fadd_rn(acc, prev[e]);
                    acc = __fadd_rn(acc, prev[e + 1]);
                    acc = __fadd_rn(acc, prev[e + 2]);
                    acc = __fadd_rn(acc, prev[e + 3]);
                }
                pout[e] = n0; pout[e + 1] = n1; pout[e + 2] = n2; pout[e + 3] = n3;
            }
        };
        // prologue: S(0) -> va, S(1) -> vb, P(0) -> pa
        S(0, va, sa0, sa1);
        S(1, vb, sb0, sb1);
        PA(0, va, sa0, sa1, pa, pb, true, false);
#pragma unroll 1
        for (int B = 0; B < n_blocks; B += 2) {
            // step B (even): S(B + 2) -> va, P(B + 1) from vb -> pb, A(B) from pa
            if (B + 2 < n_blocks) S(B + 2, va, sa0, sa1);
            PA(B + 1, vb, sb0, sb1, pb, pa, true, true);
            // step B + 1 (odd): S(B + 3) -> vb, P(B + 2) from va -> pa, A(B + 1) from pb
            if (B + 3 < n_blocks) S(B + 3, vb, sb0, sb1);
            PA(B + 2, va, sa0, sa1, pa, pb, B + 2 < n_blocks, true);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (row < m.rows) {
            scores[row] = acc;
            if (acc != acc) set_err(err, DEV_ERR_NAN_SCORE);
        }
        return;
    }
    float p[32], pn[32];
    block_products<FMT>(wbase + lane * SG::ROWB, wbase + 32 * SG::ROWB + lane * 32, m.ts, 0, xs, lut, p);
    for (int c = 0; c < n_chunks; ++c) {
        const uint8_t* wbuf = wbase + (c % SG::NBUF) * SG::WARP_BYTES;
        const uint8_t* mine = wbuf + lane * SG::ROWB;
        const uint8_t* sc = wbuf + 32 * SG::ROWB + lane * 32;
        const float* xc = xs + c * 256;
#pragma unroll 1
        for (int b = 1; b < 8; ++b) {
            block_products<FMT, true>(mine, sc, m.ts, b, xc, lut, pn, p, &acc);
#pragma unroll
            for (int e = 0; e < 32; ++e) p[e] = pn[e];
        }
        // this chunk's buffer is free (its last block sits in p): chunk c + NBUF goes into it
        __syncwarp();
        stage(c + SG::NBUF);
        if (c + 1 < n_chunks) {
            // chunk c + 1 has landed (the later ones may be in flight)
            if (SG::NBUF == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else asm volatile("cp.async.wait_group 1;" ::: "memory");
            __syncwarp();
            const uint8_t* nbuf = wbase + ((c + 1) % SG::NBUF) * SG::WARP_BYTES;
            block_products<FMT, true>(nbuf + lane * SG::ROWB, nbuf + 32 * SG::ROWB + lane * 32, m.ts, 0, xc + 256, lut, pn, p, &acc);
#pragma unroll
            for (int e = 0; e < 32; ++e) p[e] = pn[e];
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) acc = __fadd_rn(acc, p[e]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (row < m.rows) {
        scores[row] = acc;
        if (acc != acc) set_err(err, DEV_ERR_NAN_SCORE);
    }
}

// Coarse histogram of |score| keys (the classification's input) for scores that did not come from
// a scan kernel that builds it on the fly.
__global__ void hist_abs_kernel(const float* __restrict__ scores, int n, uint32_t* __restrict__ hist) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) atomicAdd(&hist[__float_as_uint(fabsf(scores[i])) >> LQ_HIST_SHIFT], 1u);
}

// Gather: each CTA takes a contiguous slice of the hit list, 64 hits at a time.  First the up dots
// of the chunk, one warp per hit (fast form), and the activations; then, hit by hit, every thread
// adds act * down[row] for its own 32-column block(s) - one vector load of the block, the 32 values
// decoded exactly as the reference's dequantiser does - into register accumulators.  Per-CTA
// partials; `finish` adds them in fixed order.
template <int FMT>
__device__ __forceinline__ void decode_block32(const FmtMat& m, size_t row, int blk, float (&v)[32]) {
    const int nblk = m.cols / 32;
    if (FMT == LQ_FMT_Q8_0) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(m.data + (row * nblk + blk) * 34);
        const float d = f16_bits_to_f32(p[0]);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t q = p[1 + j];
            v[2 * j] = __fmul_rn((float)(int)(int8_t)(q & 0xff), d);
            v[2 * j + 1] = __fmul_rn((float)(int)(int8_t)(q >> 8), d);
        }
    } else if (FMT == LQ_FMT_MXFP4) {
        const uint4 w = *reinterpret_cast<const uint4*>(m.data + (row * nblk + blk) * 16);
        const float scale = e8m0_to_f32(m.scales[row * nblk + blk]);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __fmul_rn(e2m1_to_f32((ww[e >> 3] >> (4 * (e & 7))) & 15u), scale);
    } else {
        const uint4 w = *reinterpret_cast<const uint4*>(m.data + (row * nblk + blk) * 16);
        const uint32_t sc2 = *reinterpret_cast<const uint16_t*>(m.scales + (row * nblk + blk) * 2);
        const float s0 = __fmul_rn(m.ts, e4m3_to_f32(sc2 & 0xff)), s1 = __fmul_rn(m.ts, e4m3_to_f32(sc2 >> 8));
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 32; ++e)
            v[e] = __fmul_rn(e < 16 ? s0 : s1, e2m1_to_f32((ww[e >> 3] >> (4 * (e & 7))) & 15u));
    }
}

// Packed f32x2 helpers (sm_100): two IEEE round-to-nearest operations per instruction on register pairs.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// One 32-weight block of an FP4 row as stored: 16 bytes of codes and its scale byte(s).
template <int FMT>
__device__ __forceinline__ void load_raw32(const FmtMat& m, size_t row, int blk, uint4& w, uint32_t& sc) {
    const size_t nblk = (size_t)(m.cols / 32);
    w = *reinterpret_cast<const uint4*>(m.data + (row * nblk + blk) * 16);
    if (FMT == LQ_FMT_MXFP4) sc = m.scales[row * nblk + blk];
    else sc = *reinterpret_cast<const uint16_t*>(m.scales + (row * nblk + blk) * 2);
}
// acc += act * dequantised block, the weights decoded as the reference's dequantiser does (scale * value,
// rounded once); the code -> value table sits in the lanes of the warp (`lut`), so every lane calls this together.
template <int FMT>
__device__ __forceinline__ void axpy_raw32(const uint4& w, uint32_t sc, float ts, float act, float lut,
                                           unsigned long long (&acc2)[16]) {
    float s0, s1;
    if (FMT == LQ_FMT_MXFP4) {
        s0 = s1 = e8m0_to_f32(sc);
    } else {
        s0 = __fmul_rn(ts, e4m3_to_f32(sc & 0xff));
        s1 = __fmul_rn(ts, e4m3_to_f32(sc >> 8));
    }
    const unsigned long long s0p = pack2(s0, s0), s1p = pack2(s1, s1), ap = pack2(act, act);
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        const float v0 = __shfl_sync(0xffffffffu, lut, (int)(ww[e >> 3] >> (4 * (e & 7))));
        const float v1 = __shfl_sync(0xffffffffu, lut, (int)(ww[e >> 3] >> (4 * (e & 7) + 4)));
        acc2[e >> 1] = fma2(ap, mul2(pack2(v0, v1), e < 16 ? s0p : s1p), acc2[e >> 1]);
    }
}

template <int FMT, int BPT, int NT = FK_THREADS>
__device__ __forceinline__ void gather_fmt_body(const FmtMat& up, const FmtMat& down, const XPrep& xp,
                                                const uint32_t* __restrict__ hit_idx,
                                                const float* __restrict__ hit_score,
                                                const int* __restrict__ n_hits_dev, int n_hits_host,
                                                float* __restrict__ partials) {
    __shared__ float act_s[64];
    __shared__ uint32_t row_s[64];
    extern __shared__ __align__(16) float xs_pad[];  // FP4 formats: [H / 32][36], see fast_row
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = up.cols, nblk = H / 32;
    const float lut = fp4_lut_lane(lane);
    if (FMT != LQ_FMT_Q8_0) {
        for (int i = tid; i < H / 4; i += NT) {
            const float4 v = *reinterpret_cast<const float4*>(xp.xn + 4 * i);
            *reinterpret_cast<float4*>(xs_pad + ((4 * i) >> 5) * 36 + ((4 * i) & 31)) = v;
        }
        __syncthreads();
    }
    constexpr bool FP4 = FMT != LQ_FMT_Q8_0;
    float acc[FP4 ? 1 : BPT][32];            // Q8_0
    unsigned long long acc2[FP4 ? BPT : 1][16];  // FP4 formats: packed pairs
#pragma unroll
    for (int b = 0; b < (FP4 ? 1 : BPT); ++b)
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[b][e] = 0.0f;
#pragma unroll
    for (int b = 0; b < (FP4 ? BPT : 1); ++b)
#pragma unroll
        for (int e = 0; e < 16; ++e) acc2[b][e] = 0ull;
    const int n_hits = n_hits_dev ? *n_hits_dev : n_hits_host;
    const int per = (n_hits + gridDim.x - 1) / gridDim.x;
    const int h0 = min(n_hits, (int)blockIdx.x * per), h1 = min(n_hits, h0 + per);
    for (int c0 = h0; c0 < h1; c0 += 64) {
        const int nh = min(64, h1 - c0);
        for (int i = warp; i < nh; i += NT / 32) {
            const uint32_t row = hit_idx[c0 + i];
            float b;
            const float u = fast_row<FMT>(up, row, xp, 0.0f, b, lane, lut, FMT != LQ_FMT_Q8_0 ? xs_pad : nullptr);
            if (lane == 0) {
                const float gs = hit_score[c0 + i];
                const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
                const float act = (gs * sig) * u;
                act_s[i] = fabsf(act) > FK_NOISE_FLOOR ? act : 0.0f;
                row_s[i] = row;
            }
        }
        __syncthreads();
        if (FP4) {
            // The raw blocks of the next DEPTH hits are in flight while one hit is decoded and added: a hit's row is
            // known only from the list, so nothing else hides the latency of its first touch.
            constexpr int DEPTH = 4;
            uint4 wq[DEPTH][BPT];
            uint32_t sq[DEPTH][BPT];
            auto fetch = [&](int i, uint4 (&wv)[BPT], uint32_t (&sv)[BPT]) {
#pragma unroll
                for (int b = 0; b < BPT; ++b) {
                    const int blk = tid + b * NT;
                    wv[b] = make_uint4(0u, 0u, 0u, 0u);
                    sv[b] = 0u;
                    if (i < nh && blk < nblk) load_raw32<FMT>(down, (size_t)row_s[i], blk, wv[b], sv[b]);
                }
            };
#pragma unroll
            for (int u = 0; u < DEPTH; ++u) fetch(u, wq[u], sq[u]);
            for (int i0 = 0; i0 < nh; i0 += DEPTH) {
#pragma unroll
                for (int u = 0; u < DEPTH; ++u) {
                    const int i = i0 + u;
                    uint4 wc[BPT];
                    uint32_t sc[BPT];
#pragma unroll
                    for (int b = 0; b < BPT; ++b) {
                        wc[b] = wq[u][b];
                        sc[b] = sq[u][b];
                    }
                    fetch(i + DEPTH, wq[u], sq[u]);
                    const float act = i < nh ? act_s[i] : 0.0f;
                    if (act != 0.0f) {  // (the same for every thread of the CTA)
#pragma unroll
                        for (int b = 0; b < BPT; ++b) axpy_raw32<FMT>(wc[b], sc[b], down.ts, act, lut, acc2[b]);
                    }
                }
            }
        } else {
            for (int i = 0; i < nh; ++i) {
                const float act = act_s[i];
                if (act == 0.0f) continue;
                const size_t row = row_s[i];
#pragma unroll
                for (int b = 0; b < BPT; ++b) {
                    const int blk = tid + b * NT;
                    if (blk < nblk) {
                        float v[32];
                        decode_block32<FMT>(down, row, blk, v);
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[b][e] = fmaf(act, v[e], acc[b][e]);
                    }
                }
            }
        }
        __syncthreads();
    }
    float* dst = partials + (size_t)blockIdx.x * H;
#pragma unroll
    for (int b = 0; b < BPT; ++b) {
        const int blk = tid + b * NT;
        if (blk < nblk) {
            if (FP4) {
#pragma unroll
                for (int e = 0; e < 16; e += 2)
                    *reinterpret_cast<ulonglong2*>(dst + blk * 32 + 2 * e) = make_ulonglong2(acc2[b][e], acc2[b][e + 1]);
            } else {
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                    *reinterpret_cast<float4*>(dst + blk * 32 + e) = make_float4(acc[b][e], acc[b][e + 1], acc[b][e + 2], acc[b][e + 3]);
            }
        }
    }
}

template <int FMT, int BPT>
__global__ void __launch_bounds__(FK_THREADS) gather_fmt_kernel(FmtMat up, FmtMat down, XPrep xp,
                                                               const uint32_t* __restrict__ hit_idx,
                                                               const float* __restrict__ hit_score,
                                                               const int* __restrict__ n_hits_dev, int n_hits_host,
                                                               float* __restrict__ partials) {
    gather_fmt_body<FMT, BPT>(up, down, xp, hit_idx, hit_score, n_hits_dev, n_hits_host, partials);
}

// Gather for many (token, expert) pairs in one launch: pair blockIdx.y takes its expert's up / down matrices,
// its own hit list and activation, and writes gridDim.x partial outputs at partials[y][blockIdx.x][H].
// NT: threads per CTA; narrow activations (at most 128 blocks of 32 columns) take 128, so that fewer threads idle in
// the down rows' pass and more CTAs share an SM.
template <int FMT, int BPT, int NT>
__global__ void __launch_bounds__(NT) gather_fmt_pairs_kernel(const FmtMat* __restrict__ up_table,
                                                                     const FmtMat* __restrict__ down_table,
                                                                     const uint32_t* __restrict__ pair_expert,
                                                                     TokenWs ws0, size_t ws_stride,
                                                                     float* __restrict__ partials) {
    const uint32_t e = pair_expert[blockIdx.y];
    const FmtMat up = up_table[e], down = down_table[e];
    const TokenWs ws = ws_at(ws0, ws_stride * blockIdx.y);
    const XPrep xp{ws.xn, ws.xa, ws.xb, ws.bscale, ws.bsum, ws.babs};
    gather_fmt_body<FMT, BPT, NT>(up, down, xp, ws.hit_idx, ws.hit_score, &ws.sel->n_sel, 0,
                                  partials + (size_t)blockIdx.y * gridDim.x * up.cols);
}

}  // namespace

#define FMT_DISPATCH(fmt, CALL)                         \
    switch (fmt) {                                      \
        case LQ_FMT_Q8_0: { CALL(LQ_FMT_Q8_0); } break;  \
        case LQ_FMT_MXFP4: { CALL(LQ_FMT_MXFP4); } break; \
        case LQ_FMT_NVFP4: { CALL(LQ_FMT_NVFP4); } break; \
        default: return cudaErrorInvalidValue;          \
    }

cudaError_t launch_scan_fmt(const FmtMat& m, const XPrep& xp, float* scores, uint32_t* hist, uint32_t* bound_bits,
                            float c1, int* err, int sm_count, cudaStream_t st) {
    if (m.rows == 0) return cudaSuccess;
    int grid = (m.rows + 7) / 8;
    if (grid > sm_count * 8) grid = sm_count * 8;
#define CALL(F) scan_fmt_kernel<F><<<grid, FK_THREADS, 0, st>>>(m, xp, scores, hist, bound_bits, c1, err)
    FMT_DISPATCH(m.fmt, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_hist_abs(const float* scores, int n, uint32_t* hist, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    hist_abs_kernel<<<(n + 255) / 256, 256, 0, st>>>(scores, n, hist);
    return cudaGetLastError();
}

cudaError_t launch_scan_exact_fmt(const FmtMat& m, const float* xn, float* scores, int* err, cudaStream_t st) {
    if (m.rows == 0) return cudaSuccess;
    const bool aligned = (((uintptr_t)m.data | (uintptr_t)(m.scales ? m.scales : m.data)) & 15) == 0;
    if (m.cols % 256 == 0 && aligned) {
        const int sgrid = (m.rows + 127) / 128;
#define SCALL(F)                                                                                                   \
    {                                                                                                              \
        const size_t sm = (size_t)m.cols * 4 + 4 * (size_t)StagedGeom<F>::NBUF * StagedGeom<F>::WARP_BYTES;                              \
        cudaError_t e = set_max_dyn_smem((const void*)scan_exact_staged_kernel<F>, 200 * 1024);                    \
        if (e != cudaSuccess) return e;                                                                            \
        scan_exact_staged_kernel<F><<<sgrid, 128, sm, st>>>(m, xn, scores, err);                                   \
    }
        FMT_DISPATCH(m.fmt, SCALL)
#undef SCALL
        return cudaGetLastError();
    }
    const int grid = (m.rows + 63) / 64;
    const size_t smem = (size_t)m.cols * sizeof(float) + 64 * (size_t)(m.cols / 16);
#define CALL(F)                                                                                                     \
    {                                                                                                               \
        cudaError_t e = set_max_dyn_smem((const void*)scan_exact_fmt_kernel<F>, 140 * 1024);                         \
        if (e != cudaSuccess) return e;                                                                             \
        scan_exact_fmt_kernel<F><<<grid, 64, smem, st>>>(m, xn, scores, err);                                        \
    }
    FMT_DISPATCH(m.fmt, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_rescore_fmt(const FmtMat& m, const float* xn, const uint32_t* rows_idx, const int* n_rows_dev,
                               int n_rows_host, float* out, int sm_count, cudaStream_t st) {
    int grid = n_rows_dev ? sm_count * 4 : (n_rows_host + 63) / 64;
    if (grid < 1) grid = 1;
    if (grid > sm_count * 16) grid = sm_count * 16;
#define CALL(F) rescore_fmt_kernel<F><<<grid, 64, 0, st>>>(m, xn, rows_idx, n_rows_dev, n_rows_host, out)
    FMT_DISPATCH(m.fmt, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_gather_fmt(const FmtMat& up, const FmtMat& down, const XPrep& xp, const uint32_t* hit_idx,
                              const float* hit_score, const int* n_hits_dev, int n_hits_host, float* partials,
                              int grid, cudaStream_t st) {
    if (up.fmt != down.fmt || up.cols != down.cols || up.cols % 32 != 0 || up.cols > 16384) return cudaErrorInvalidValue;
    const int bpt = (up.cols / 32 + FK_THREADS - 1) / FK_THREADS;  // 32-column blocks per thread: 1 or 2
    const size_t xsm = up.fmt == LQ_FMT_Q8_0 ? 0 : (size_t)(up.cols / 32) * 36 * sizeof(float);  // padded activation
#define CALL(F)                                                                                                \
    {                                                                                                          \
        if (bpt <= 1)                                                                                          \
        {                                                                                                      \
            cudaError_t e = set_max_dyn_smem((const void*)gather_fmt_kernel<F, 1>, 80 * 1024);                  \
            if (e != cudaSuccess) return e;                                                                     \
            gather_fmt_kernel<F, 1><<<grid, FK_THREADS, xsm, st>>>(up, down, xp, hit_idx, hit_score, n_hits_dev, \
                                                                  n_hits_host, partials);                      \
        } else {                                                                                               \
            cudaError_t e = set_max_dyn_smem((const void*)gather_fmt_kernel<F, 2>, 80 * 1024);                  \
            if (e != cudaSuccess) return e;                                                                     \
            gather_fmt_kernel<F, 2><<<grid, FK_THREADS, xsm, st>>>(up, down, xp, hit_idx, hit_score, n_hits_dev, \
                                                                  n_hits_host, partials);                      \
        }                                                                                                      \
    }
    FMT_DISPATCH(up.fmt, CALL)
#undef CALL
    return cudaGetLastError();
}

// Pair-batched launches (mixture of experts): all matrices of one table share format and shape.
cudaError_t launch_scan_exact_pairs(int fmt, const FmtMat* table, const uint32_t* pair_expert, int n_pairs, int rows,
                                    int cols, TokenWs ws0, size_t ws_stride, int* err, cudaStream_t st) {
    if (n_pairs <= 0 || rows <= 0) return cudaSuccess;
    const dim3 grid((rows + 63) / 64, n_pairs);
    const size_t smem = (size_t)cols * sizeof(float) + 64 * (size_t)(cols / 16);
#define CALL(F)                                                                                             \
    {                                                                                                       \
        cudaError_t e = set_max_dyn_smem((const void*)scan_exact_pairs_kernel<F>, 140 * 1024);              \
        if (e != cudaSuccess) return e;                                                                     \
        scan_exact_pairs_kernel<F><<<grid, 64, smem, st>>>(table, pair_expert, ws0, ws_stride, err);        \
    }
    FMT_DISPATCH(fmt, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_gather_fmt_pairs(int fmt, const FmtMat* up_table, const FmtMat* down_table,
                                    const uint32_t* pair_expert, int n_pairs, int cols, TokenWs ws0, size_t ws_stride,
                                    float* partials, int grid_x, cudaStream_t st) {
    if (n_pairs <= 0) return cudaSuccess;
    if (cols % 32 != 0 || cols > 16384) return cudaErrorInvalidValue;
    const int nblk = cols / 32;
    const dim3 grid(grid_x, n_pairs);
    const size_t xsm = fmt == LQ_FMT_Q8_0 ? 0 : (size_t)nblk * 36 * sizeof(float);  // padded activation
#define LAUNCH(F, BPT, NT)                                                                                             \
    {                                                                                                                  \
        cudaError_t e = set_max_dyn_smem((const void*)gather_fmt_pairs_kernel<F, BPT, NT>, 80 * 1024);                  \
        if (e != cudaSuccess) return e;                                                                                \
        gather_fmt_pairs_kernel<F, BPT, NT><<<grid, NT, xsm, st>>>(up_table, down_table, pair_expert, ws0, ws_stride,   \
                                                                  partials);                                          \
    }
#define CALL(F)                                                                                                        \
    {                                                                                                                  \
        if (nblk <= 128) LAUNCH(F, 1, 128)                                                                             \
        else if (nblk <= FK_THREADS) LAUNCH(F, 1, FK_THREADS)                                                          \
        else LAUNCH(F, 2, FK_THREADS)                                                                                  \
    }
    FMT_DISPATCH(fmt, CALL)
#undef CALL
#undef LAUNCH
    return cudaGetLastError();
}

}  // namespace lq
