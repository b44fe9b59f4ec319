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

// One warp: fast dot of row `row` with the prepared activation; also the bound term
// sum |w||x| (upper estimate) scaled by c1, plus the fixed-point error term for Q8_0.
template <int FMT>
__device__ __forceinline__ float fast_row(const FmtMat& m, size_t row, const XPrep& xp, float c1, float& bound, int lane,
                                          float lut) {
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
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 x0 = make_float4(0, 0, 0, 0), x1 = x0;
                if (on) {
                    x0 = *reinterpret_cast<const float4*>(xp.xn + blk * 32 + 8 * j);
                    x1 = *reinterpret_cast<const float4*>(xp.xn + blk * 32 + 8 * j + 4);
                }
                const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float t = __shfl_sync(0xffffffffu, lut, (qw[j] >> (4 * e)) & 15u);
                    s = fmaf(t, xs[e], s);
                }
            }
            if (on) {
                acc += s * scale;
                bnd += c1 * 6.0f * fabsf(scale) * xp.abs[blk];
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
            float s = 0.0f, ax = 0.0f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float4 x0 = make_float4(0, 0, 0, 0), x1 = x0;
                if (on) {
                    x0 = *reinterpret_cast<const float4*>(xp.xn + g * 16 + 8 * j);
                    x1 = *reinterpret_cast<const float4*>(xp.xn + g * 16 + 8 * j + 4);
                }
                const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float t = __shfl_sync(0xffffffffu, lut, (qw[j] >> (4 * e)) & 15u);
                    s = fmaf(t, xs[e], s);
                    ax += fabsf(xs[e]);
                }
            }
            if (on) {
                acc += s * step;
                bnd += c1 * 6.0f * fabsf(step) * ax;
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

// Element h of row `row`, decoded exactly as the reference's dequantiser does.
template <int FMT>
__device__ __forceinline__ float decode_elem(const FmtMat& m, size_t row, int h) {
    if (FMT == LQ_FMT_Q8_0) {
        const uint8_t* p = m.data + (row * (m.cols / 32) + h / 32) * 34;
        return __fmul_rn((float)(int8_t)p[2 + (h & 31)], f16_bits_to_f32((uint32_t)p[0] | ((uint32_t)p[1] << 8)));
    } else if (FMT == LQ_FMT_MXFP4) {
        const size_t g = row * (m.cols / 32) + h / 32;
        const uint32_t byte = m.data[g * 16 + (h & 31) / 2];
        return __fmul_rn(e2m1_to_f32((h & 1) ? (byte >> 4) : (byte & 15u)), e8m0_to_f32(m.scales[g]));
    } else {
        const size_t g = row * (m.cols / 16) + h / 16;
        const uint32_t byte = m.data[g * 8 + (h & 15) / 2];
        return __fmul_rn(__fmul_rn(m.ts, e4m3_to_f32(m.scales[g])), e2m1_to_f32((h & 1) ? (byte >> 4) : (byte & 15u)));
    }
}

// Gather: each CTA takes a contiguous slice of the hit list; per hit the CTA's warps share the
// up dot (fast form), then every thread adds act * down[row][h] into its columns of out[H]
// kept in shared memory.  Partials per CTA; `finish` adds them in fixed order.
template <int FMT>
__global__ void __launch_bounds__(FK_THREADS) gather_fmt_kernel(FmtMat up, FmtMat down, XPrep xp,
                                                               const uint32_t* __restrict__ hit_idx,
                                                               const float* __restrict__ hit_score,
                                                               const int* __restrict__ n_hits_dev, int n_hits_host,
                                                               float* __restrict__ partials) {
    extern __shared__ __align__(16) float out_s[];  // [H]
    __shared__ float s_part[FK_THREADS / 32];
    __shared__ float s_act;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = up.cols;
    const float lut = fp4_lut_lane(lane);
    for (int h = tid; h < H; h += FK_THREADS) out_s[h] = 0.0f;
    const int n_hits = n_hits_dev ? *n_hits_dev : n_hits_host;
    const int per = (n_hits + gridDim.x - 1) / gridDim.x;
    const int h0 = min(n_hits, (int)blockIdx.x * per), h1 = min(n_hits, h0 + per);
    __syncthreads();
    for (int i = h0; i < h1; ++i) {
        const size_t row = hit_idx[i];
        // up dot: warp w takes the row's blocks w*32+lane, +256, ... by viewing the row as 8 sub-rows
        // is format specific; simpler and still parallel: warp 0..7 each compute the whole dot of a
        // different hit would need 8 hits in flight.  Here one warp does the dot, the rest wait.
        if (warp == 0) {
            float b;
            const float u = fast_row<FMT>(up, row, xp, 0.0f, b, lane, lut);
            if (lane == 0) {
                const float gs = hit_score[i];
                const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
                const float act = (gs * sig) * u;
                s_act = fabsf(act) > FK_NOISE_FLOOR ? act : 0.0f;
            }
        }
        __syncthreads();
        const float act = s_act;
        if (act != 0.0f)
            for (int h = tid; h < H; h += FK_THREADS) out_s[h] = fmaf(act, decode_elem<FMT>(down, row, h), out_s[h]);
        __syncthreads();
    }
    (void)s_part;
    float* dst = partials + (size_t)blockIdx.x * H;
    for (int h = tid; h < H; h += FK_THREADS) dst[h] = out_s[h];
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
    if (up.fmt != down.fmt || up.cols != down.cols) return cudaErrorInvalidValue;
    const size_t smem = (size_t)up.cols * sizeof(float);
#define CALL(F)                                                                                                  \
    {                                                                                                            \
        static bool attr = false;                                                                                \
        if (!attr) {                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(gather_fmt_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 64 * 1024);                                                     \
            if (e != cudaSuccess) return e;                                                                      \
            attr = true;                                                                                         \
        }                                                                                                        \
        gather_fmt_kernel<F><<<grid, FK_THREADS, smem, st>>>(up, down, xp, hit_idx, hit_score, n_hits_dev,       \
                                                            n_hits_host, partials);                             \
    }
    FMT_DISPATCH(up.fmt, CALL)
#undef CALL
    return cudaGetLastError();
}

}  // namespace lq
