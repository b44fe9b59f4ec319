// Q6_K rows and the mixed K-quant walk, and the fused gate+up Q4_K matvec.
//
// Real Q4_K vindexes keep gate and up as Q4_K and down as Q6_K (the Ollama convention,
// crates/larql-compute/PERFORMANCE.md:3-4); the walk takes each matrix's row functions from a
// per-format table (crates/larql-vindex/src/quant/registry.rs).  Here:
//   q6k_matvec_kernel      the backend's Q6_K matvec in its own f32 order
//                          (crates/larql-compute/src/cpu/ops/q6k_matvec.rs:45-96): per 16-element
//                          sub-block sub = sum v*x in element order, then acc += (d*scale) * sub over
//                          the row's sub-blocks in order.  The gate scan and the dense product of a
//                          Q6_K matrix.
//   q6k_dequant_kernel     dequantize_q6_k (crates/larql-models/src/quant/ggml/q6_k.rs:171-195)
//   gather_kquant_kernel   up dot, SiLU, down scaled-add over the selected rows with up and down each
//                          Q4_K or Q6_K (q4k_row_dot / q6k_row_dot, q4k_row_scaled_add /
//                          q6k_row_scaled_add; the walk's outputs are held to 1e-3, so the dots here
//                          are plain FMA sums)
//   q4k_dual_matvec_kernel q4k_dual_matvec_into (crates/larql-compute/src/cpu/ops/q4_common/dual.rs:22-167)
//                          in its own order: ONE running sum per row over all (super-block, pair)
//                          terms, where q4k_matvec_into sums each super-block first.
// A Q6_K super-block is 210 bytes, so rows are only 2-byte aligned: everything is read as 16-bit words.
#include "../../include/larql_cuda.h"
#include "codecs.cuh"
#include "kernels.h"

namespace lq {

namespace {

constexpr int KQ_THREADS = 256;
constexpr float KQ_NOISE_FLOOR = 1e-10f;  // ACTIVATION_NOISE_FLOOR, walk_config.rs:64

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }

// The 16 signed values of scale sub-block j of a Q6_K super-block (q6k_subblock_vals, q6_k.rs:19-42):
// 16 consecutive ql bytes (one nibble plane) and 16 consecutive qh bytes (one bit pair each).
__device__ __forceinline__ void q6k_sub_vals(const uint8_t* block, int j, int (&v)[16]) {
    const int half = j >> 3, g = j & 7, plane = g >> 1, lbase = (g & 1) * 16;
    const uint8_t* ql = block + half * 64 + (plane & 1) * 32 + lbase;
    const uint8_t* qh = block + 128 + half * 32 + lbase;
    const int shift = plane * 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t l2 = ld_u16(ql + 2 * i), h2 = ld_u16(qh + 2 * i);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const uint32_t lb = (l2 >> (8 * b)) & 0xffu, hb = (h2 >> (8 * b)) & 0xffu;
            const uint32_t lo4 = plane < 2 ? (lb & 0x0fu) : (lb >> 4);
            v[2 * i + b] = (int)(lo4 | (((hb >> shift) & 3u) << 4)) - 32;
        }
    }
}
__device__ __forceinline__ float q6k_sub_scale(const uint8_t* block, int j) {
    // d * (scale as i8 as f32), the product every reference routine forms first
    const uint32_t s2 = ld_u16(block + 192 + (j & ~1));
    const float d = f16_bits_to_f32(ld_u16(block + 208));
    return __fmul_rn(d, (float)(int)(int8_t)((s2 >> (8 * (j & 1))) & 0xffu));
}

// One warp per row.  Lanes 0-15 take the 16 sub-blocks of one super-block and lanes 16-31 those of the
// next; the chain acc += sc * sub then runs in (super-block, sub-block) order over the lanes' terms.
__global__ void __launch_bounds__(KQ_THREADS) q6k_matvec_kernel(const uint8_t* __restrict__ w, const float* __restrict__ x,
                                                                const uint32_t* __restrict__ rows_idx,
                                                                const int* __restrict__ n_rows_dev, int n_rows, int cols,
                                                                float* __restrict__ out, int* err) {
    extern __shared__ __align__(16) float xs[];  // [cols]
    for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, nsb = cols / 256;
    const size_t row_bytes = (size_t)nsb * 210;
    const int n = n_rows_dev ? *n_rows_dev : n_rows;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n; r += warps) {
        const uint8_t* row = w + (rows_idx ? (size_t)rows_idx[r] : (size_t)r) * row_bytes;
        float acc = 0.0f;
        for (int s0 = 0; s0 < nsb; s0 += 2) {
            const int sb = s0 + (lane >> 4), j = lane & 15;
            float term = 0.0f;
            if (sb < nsb) {
                const uint8_t* block = row + (size_t)sb * 210;
                int v[16];
                q6k_sub_vals(block, j, v);
                const float* xv = xs + sb * 256 + j * 16;
                float sub = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; ++i) sub = __fadd_rn(sub, __fmul_rn((float)v[i], xv[i]));
                term = __fmul_rn(q6k_sub_scale(block, j), sub);
            }
            const int n_terms = min(32, (nsb - s0) * 16);
            for (int i = 0; i < n_terms; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, term, i));
        }
        if (lane == 0) {
            out[r] = acc;
            if (acc != acc && err) set_err(err, DEV_ERR_NAN_SCORE);
        }
    }
}

__global__ void q6k_dequant_kernel(const uint8_t* __restrict__ data, size_t n_sub, float* __restrict__ out) {
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_sub; t += (size_t)gridDim.x * blockDim.x) {
        const uint8_t* block = data + (t >> 4) * 210;
        const int j = (int)(t & 15);
        int v[16];
        q6k_sub_vals(block, j, v);
        const float sc = q6k_sub_scale(block, j);
#pragma unroll
        for (int i = 0; i < 16; ++i) out[t * 16 + i] = __fmul_rn(sc, (float)v[i]);
    }
}

// 32 consecutive elements (block `blk` of a row) of a Q4_K or Q6_K row, decoded as the reference's
// dequantiser does: Q4_K d*sc*q - dmin*m, Q6_K (d*scale)*q.
template <int FMT>
__device__ __forceinline__ void kq_decode32(const uint8_t* row, int blk, float (&v)[32]) {
    if (FMT == LQ_FMT_Q4_K) {
        const uint8_t* cell = row + (size_t)(blk >> 3) * 144;
        const int b = blk & 7, g = b >> 1;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(cell));
        const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(cell + 16 + g * 32));
        const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(cell + 32 + g * 32));
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t sc2, m2;
        q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
        const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
        const float sc = d * (float)((b & 1) ? (sc2 >> 8) : (sc2 & 0xff));
        const float mn = dmin * (float)((b & 1) ? (m2 >> 8) : (m2 & 0xff));
#pragma unroll
        for (int e = 0; e < 32; ++e) {
            const uint32_t byte = (qw[e >> 2] >> (8 * (e & 3))) & 0xffu;
            v[e] = sc * (float)((b & 1) ? (byte >> 4) : (byte & 0x0fu)) - mn;
        }
    } else {
        const uint8_t* block = row + (size_t)(blk >> 3) * 210;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int j = (blk & 7) * 2 + h;
            int q[16];
            q6k_sub_vals(block, j, q);
            const float sc = q6k_sub_scale(block, j);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[16 * h + i] = sc * (float)q[i];
        }
    }
}

__host__ __device__ inline size_t kq_row_bytes(int fmt, int cols) {
    return (size_t)(cols / 256) * (fmt == LQ_FMT_Q4_K ? 144 : 210);
}

// Gather over the selected rows: each CTA takes a contiguous slice of the hit list, 64 hits at a time;
// up dots one warp per hit, then every thread adds act * down[row] for its own 32-column block(s).
template <int UPF, int DOWNF, int BPT>
__global__ void __launch_bounds__(KQ_THREADS) gather_kquant_kernel(const uint8_t* __restrict__ up,
                                                                   const uint8_t* __restrict__ down,
                                                                   const float* __restrict__ xn, int cols,
                                                                   const uint32_t* __restrict__ hit_idx,
                                                                   const float* __restrict__ hit_score,
                                                                   const int* __restrict__ n_hits_dev, int n_hits_host,
                                                                   float* __restrict__ partials) {
    extern __shared__ __align__(16) float xs[];  // [cols]
    __shared__ float act_s[64];
    __shared__ uint32_t row_s[64];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nblk = cols / 32;
    for (int i = tid; i < cols; i += KQ_THREADS) xs[i] = xn[i];
    float acc[BPT][32];
#pragma unroll
    for (int b = 0; b < BPT; ++b)
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[b][e] = 0.0f;
    const int n_hits = n_hits_dev ? *n_hits_dev : n_hits_host;
    const int per = (n_hits + gridDim.x - 1) / gridDim.x;
    const int h0 = min(n_hits, (int)blockIdx.x * per), h1 = min(n_hits, h0 + per);
    const size_t up_rb = kq_row_bytes(UPF, cols), down_rb = kq_row_bytes(DOWNF, cols);
    __syncthreads();
    for (int c0 = h0; c0 < h1; c0 += 64) {
        const int nh = min(64, h1 - c0);
        for (int i = warp; i < nh; i += KQ_THREADS / 32) {
            const uint32_t row = hit_idx[c0 + i];
            const uint8_t* rp = up + (size_t)row * up_rb;
            float u = 0.0f;
            for (int blk = lane; blk < nblk; blk += 32) {
                float v[32];
                kq_decode32<UPF>(rp, blk, v);
                const float* xv = xs + blk * 32;
#pragma unroll
                for (int e = 0; e < 32; ++e) u = fmaf(v[e], xv[e], u);
            }
            for (int o = 16; o > 0; o >>= 1) u += __shfl_xor_sync(0xffffffffu, u, o);
            if (lane == 0) {
                const float gs = hit_score[c0 + i];
                const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
                const float act = (gs * sig) * u;
                act_s[i] = fabsf(act) > KQ_NOISE_FLOOR ? act : 0.0f;
                row_s[i] = row;
            }
        }
        __syncthreads();
        for (int i = 0; i < nh; ++i) {
            const float act = act_s[i];
            if (act == 0.0f) continue;
            const uint8_t* rp = down + (size_t)row_s[i] * down_rb;
#pragma unroll
            for (int b = 0; b < BPT; ++b) {
                const int blk = tid + b * KQ_THREADS;
                if (blk < nblk) {
                    float v[32];
                    kq_decode32<DOWNF>(rp, blk, v);
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[b][e] = fmaf(act, v[e], acc[b][e]);
                }
            }
        }
        __syncthreads();
    }
    float* dst = partials + (size_t)blockIdx.x * cols;
#pragma unroll
    for (int b = 0; b < BPT; ++b) {
        const int blk = tid + b * KQ_THREADS;
        if (blk < nblk) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
                *reinterpret_cast<float4*>(dst + blk * 32 + e) = make_float4(acc[b][e], acc[b][e + 1], acc[b][e + 2], acc[b][e + 3]);
        }
    }
}

// Both matrices against one activation, one warp per row.  Lane (s, g) = (lane / 4, lane % 4) takes pair
// g of super-block s0 + s; a pass covers eight super-blocks, and the row's single running sum then takes
// the 64 terms of the pass in the reference's order: super-block, pair, low block then high block.
__global__ void __launch_bounds__(KQ_THREADS) q4k_dual_matvec_kernel(const uint8_t* __restrict__ wa,
                                                                     const uint8_t* __restrict__ wb,
                                                                     const float* __restrict__ x, int rows, int cols,
                                                                     float* __restrict__ out_a, float* __restrict__ out_b) {
    extern __shared__ __align__(16) float xs[];  // [cols]
    for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, g = lane & 3, nsb = cols / 256;
    const size_t row_bytes = (size_t)nsb * 144;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        float acc[2] = {0.0f, 0.0f};
        for (int s0 = 0; s0 < nsb; s0 += 8) {
            const int s = s0 + (lane >> 2);
            float lo[2] = {0.0f, 0.0f}, hi[2] = {0.0f, 0.0f};
            if (s < nsb) {
                const float* x_lo = xs + s * 256 + g * 64;
                const float* x_hi = x_lo + 32;
                float sum_lo = 0.0f, sum_hi = 0.0f;  // sum_x of the two blocks (dual.rs:62-70), element order
#pragma unroll
                for (int l = 0; l < 32; ++l) {
                    sum_lo = __fadd_rn(sum_lo, x_lo[l]);
                    sum_hi = __fadd_rn(sum_hi, x_hi[l]);
                }
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    const uint8_t* cell = (m ? wb : wa) + (size_t)r * row_bytes + (size_t)s * 144;
                    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(cell));
                    const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(cell + 16 + g * 32));
                    const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(cell + 32 + g * 32));
                    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    float dot_lo = 0.0f, dot_hi = 0.0f;
#pragma unroll
                    for (int l = 0; l < 32; ++l) {
                        const uint32_t byte = (qw[l >> 2] >> (8 * (l & 3))) & 0xffu;
                        dot_lo = __fadd_rn(dot_lo, __fmul_rn((float)(byte & 0x0fu), x_lo[l]));
                        dot_hi = __fadd_rn(dot_hi, __fmul_rn((float)(byte >> 4), x_hi[l]));
                    }
                    const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
                    uint32_t sc2, m2;
                    q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
                    const float sc_lo = __fmul_rn(d, (float)(sc2 & 0xff)), sc_hi = __fmul_rn(d, (float)(sc2 >> 8));
                    const float mn_lo = __fmul_rn(dmin, (float)(m2 & 0xff)), mn_hi = __fmul_rn(dmin, (float)(m2 >> 8));
                    lo[m] = __fsub_rn(__fmul_rn(sc_lo, dot_lo), __fmul_rn(mn_lo, sum_lo));
                    hi[m] = __fsub_rn(__fmul_rn(sc_hi, dot_hi), __fmul_rn(mn_hi, sum_hi));
                }
            }
            const int n_terms = min(32, (nsb - s0) * 4);
            for (int i = 0; i < n_terms; ++i) {
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    acc[m] = __fadd_rn(acc[m], __shfl_sync(0xffffffffu, lo[m], i));
                    acc[m] = __fadd_rn(acc[m], __shfl_sync(0xffffffffu, hi[m], i));
                }
            }
        }
        if (lane == 0) {
            out_a[r] = acc[0];
            out_b[r] = acc[1];
        }
    }
}

}  // namespace

cudaError_t launch_q6k_matvec(const uint8_t* w, const float* x, const uint32_t* rows_idx, const int* n_rows_dev,
                              int n_rows, int cols, float* out, int* err, int sm_count, cudaStream_t st) {
    if (cols <= 0 || cols % 256 != 0 || cols > 16384) return cudaErrorInvalidValue;
    if (n_rows <= 0 && !n_rows_dev) return cudaSuccess;
    cudaError_t e = set_max_dyn_smem((const void*)q6k_matvec_kernel, 64 * 1024);
    if (e != cudaSuccess) return e;
    int grid = n_rows_dev ? sm_count * 4 : (n_rows + 7) / 8;
    if (grid > sm_count * 8) grid = sm_count * 8;
    if (grid < 1) grid = 1;
    q6k_matvec_kernel<<<grid, KQ_THREADS, (size_t)cols * 4, st>>>(w, x, rows_idx, n_rows_dev, n_rows, cols, out, err);
    return cudaGetLastError();
}

cudaError_t launch_q6k_dequant(const uint8_t* data, size_t n_elems, float* out, cudaStream_t st) {
    if (n_elems == 0) return cudaSuccess;
    const size_t n_sub = n_elems / 16;
    const int grid = (int)std::min<size_t>((n_sub + 255) / 256, 65535);
    q6k_dequant_kernel<<<grid, 256, 0, st>>>(data, n_sub, out);
    return cudaGetLastError();
}

cudaError_t launch_gather_kquant(int up_fmt, const uint8_t* up, int down_fmt, const uint8_t* down, const float* xn,
                                 int cols, const uint32_t* hit_idx, const float* hit_score, const int* n_hits_dev,
                                 int n_hits_host, float* partials, int grid, cudaStream_t st) {
    if (cols % 256 != 0 || cols > 16384) return cudaErrorInvalidValue;
    const int bpt = (cols / 32 + KQ_THREADS - 1) / KQ_THREADS;  // 32-column blocks per thread: 1 or 2
    const size_t smem = (size_t)cols * 4;
#define KQ_LAUNCH(UF, DF)                                                                                          \
    {                                                                                                              \
        cudaError_t e;                                                                                             \
        if (bpt <= 1) {                                                                                            \
            e = set_max_dyn_smem((const void*)gather_kquant_kernel<UF, DF, 1>, 64 * 1024);                         \
            if (e != cudaSuccess) return e;                                                                        \
            gather_kquant_kernel<UF, DF, 1><<<grid, KQ_THREADS, smem, st>>>(up, down, xn, cols, hit_idx, hit_score, \
                                                                           n_hits_dev, n_hits_host, partials);     \
        } else {                                                                                                   \
            e = set_max_dyn_smem((const void*)gather_kquant_kernel<UF, DF, 2>, 64 * 1024);                         \
            if (e != cudaSuccess) return e;                                                                        \
            gather_kquant_kernel<UF, DF, 2><<<grid, KQ_THREADS, smem, st>>>(up, down, xn, cols, hit_idx, hit_score, \
                                                                           n_hits_dev, n_hits_host, partials);     \
        }                                                                                                          \
    }
    if (up_fmt == LQ_FMT_Q4_K && down_fmt == LQ_FMT_Q6_K) KQ_LAUNCH(LQ_FMT_Q4_K, LQ_FMT_Q6_K)
    else if (up_fmt == LQ_FMT_Q6_K && down_fmt == LQ_FMT_Q6_K) KQ_LAUNCH(LQ_FMT_Q6_K, LQ_FMT_Q6_K)
    else if (up_fmt == LQ_FMT_Q6_K && down_fmt == LQ_FMT_Q4_K) KQ_LAUNCH(LQ_FMT_Q6_K, LQ_FMT_Q4_K)
    else if (up_fmt == LQ_FMT_Q4_K && down_fmt == LQ_FMT_Q4_K) KQ_LAUNCH(LQ_FMT_Q4_K, LQ_FMT_Q4_K)
    else return cudaErrorInvalidValue;
#undef KQ_LAUNCH
    return cudaGetLastError();
}

cudaError_t launch_q4k_dual_matvec(const uint8_t* wa, const uint8_t* wb, const float* x, int rows, int cols,
                                   float* out_a, float* out_b, int sm_count, cudaStream_t st) {
    if (cols <= 0 || cols % 256 != 0 || cols > 16384) return cudaErrorInvalidValue;
    if (rows <= 0) return cudaSuccess;
    cudaError_t e = set_max_dyn_smem((const void*)q4k_dual_matvec_kernel, 64 * 1024);
    if (e != cudaSuccess) return e;
    int grid = (rows + 7) / 8;
    if (grid > sm_count * 6) grid = sm_count * 6;
    q4k_dual_matvec_kernel<<<grid, KQ_THREADS, (size_t)cols * 4, st>>>(wa, wb, x, rows, cols, out_a, out_b);
    return cudaGetLastError();
}

}  // namespace lq
