// Q4_K sparse gather-accumulate for one token: for every selected feature f
//   up   = dot(up_row[f], x)                     (fast integer form, like the scan)
//   act  = (g * sigmoid(g)) * up                 g = gate score of f
//   out += act * dequant(down_row[f])            skipped when |act| <= 1e-10
// which is the per-feature loop of walk_ffn_sparse
// (crates/larql-inference/src/vindex/walk_ffn/sparse.rs:218-289) with the reference's
// row primitives q4k_row_dot / q4k_row_scaled_add
// (crates/larql-models/src/quant/ggml/q4_k.rs:59-89,201-227).  The reference itself
// sums features in a thread-count-dependent order at K >= 512
// (…/walk_ffn/sparse_parallel.rs:96-154), so outputs are compared by relative L2.
//
// Each CTA takes a contiguous slice of the hit list, fetches the up and the
// feature-major down row of each feature with one TMA bulk copy per row into a
// double-buffered shared-memory staging area, and keeps its part of out[H] in
// registers (64 columns per thread).  Per-CTA partials go to global memory in a fixed
// layout; `finish` adds them in a fixed order, so results are run-to-run identical.
#include "kernels.h"

namespace lq {

namespace {

constexpr int GATHER_THREADS = 256;
constexpr int GATHER_BUF_TARGET = 72 * 1024;
constexpr float ACTIVATION_NOISE_FLOOR = 1e-10f;  // walk_config.rs:64

struct GatherGeom {
    int nsb, G, P, F;  // F = features per staging buffer
    int row_bytes;
    int buf_bytes;     // F * 2 * row_bytes
    int smem_bytes;
};

__host__ inline bool gather_geom(int hidden, GatherGeom& g) {
    if (hidden <= 0 || hidden % 256 != 0) return false;
    g.nsb = hidden / 256;
    g.G = 4 * g.nsb;
    if (g.G > GATHER_THREADS) return false;
    g.P = GATHER_THREADS / g.G;
    g.row_bytes = g.nsb * 144;
    int f = GATHER_BUF_TARGET / (2 * g.row_bytes);
    f = f / g.P * g.P;
    if (f < g.P) f = g.P;
    if (f > 64) f = 64 / g.P * g.P;
    g.F = f;
    g.buf_bytes = g.F * 2 * g.row_bytes;
    // barriers(128) + part[F][G] + act[F] + 2 buffers; the out[H] merge reuses buffer 0
    int fixed = 128 + g.F * g.G * 4 + 64 * 4;
    fixed = (fixed + 127) / 128 * 128;
    int bufs = 2 * g.buf_bytes;
    if (bufs < hidden * 4) bufs = hidden * 4;
    g.smem_bytes = fixed + bufs;
    return g.smem_bytes <= 220 * 1024;
}

__global__ void __launch_bounds__(GATHER_THREADS, 1)
gather_q4k_kernel(const uint8_t* __restrict__ Wup, const uint8_t* __restrict__ Wdown, GatherGeom gm, XPrep xp,
                  const uint32_t* __restrict__ hit_idx, const float* __restrict__ hit_score,
                  const int* __restrict__ n_hits_dev, int n_hits_host, float* __restrict__ partials, int* err,
                  TokStride ts) {
    extern __shared__ __align__(128) uint8_t smem[];
    {
        const size_t off = ts.ws * blockIdx.y;
        xp = xp_at(xp, off);
        hit_idx = tok_off(hit_idx, off);
        hit_score = tok_off(hit_score, off);
        n_hits_dev = tok_off(n_hits_dev, off);
        partials += ts.part * blockIdx.y;
    }
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // [2]
    float* part = reinterpret_cast<float*>(smem + 128);  // [F][G]
    float* act_s = part + gm.F * gm.G;                   // [F] (<= 64)
    uint8_t* buf0 = smem + ((128 + gm.F * gm.G * 4 + 64 * 4 + 127) / 128 * 128);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gm.G, P = gm.P, F = gm.F;
    const int c = tid % G, prow = tid / G;
    const bool active = prow < P;
    const int s = c >> 2, g = c & 3;
    const int hidden = gm.nsb * 256;

    const int n_hits = n_hits_dev ? *n_hits_dev : n_hits_host;
    const int per = (n_hits + gridDim.x - 1) / gridDim.x;
    const int h0 = min(n_hits, (int)blockIdx.x * per), h1 = min(n_hits, h0 + per);
    const int n_sub = (h1 - h0 + F - 1) / F;

    uint32_t xa_lo[8], xb_lo[8], xa_hi[8], xb_hi[8];
    const int blk_lo = s * 8 + 2 * g, blk_hi = blk_lo + 1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        xa_lo[j] = xp.xa[blk_lo * 8 + j];
        xb_lo[j] = xp.xb[blk_lo * 8 + j];
        xa_hi[j] = xp.xa[blk_hi * 8 + j];
        xb_hi[j] = xp.xb[blk_hi * 8 + j];
    }
    const float st_lo = xp.scale[blk_lo], st_hi = xp.scale[blk_hi];
    const float su_lo = xp.sum[blk_lo], su_hi = xp.sum[blk_hi];

    float acc_lo[32], acc_hi[32];
#pragma unroll
    for (int l = 0; l < 32; ++l) acc_lo[l] = acc_hi[l] = 0.0f;
    float corr_lo = 0.0f, corr_hi = 0.0f;  // sum of (128*a*d*sc + a*dmin*m) to subtract at the end

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        fence_mbar_init();
    }
    __syncthreads();

    // Warp 0 issues a staging buffer's copies: lane f fetches the row number of feature f
    // (one coalesced load) and launches that feature's two row copies.
    auto issue = [&](int sub) {
        const int f0 = h0 + sub * F, nf = min(F, h1 - f0);
        uint8_t* b = buf0 + (size_t)(sub & 1) * gm.buf_bytes;
        if (lane == 0) mbar_expect_tx(&full[sub & 1], (uint32_t)(nf * 2 * gm.row_bytes));
        __syncwarp();
        for (int f = lane; f < nf; f += 32) {
            const size_t row = hit_idx[f0 + f];
            tma_bulk_g2s(b + (size_t)(2 * f) * gm.row_bytes, Wup + row * gm.row_bytes, gm.row_bytes, &full[sub & 1]);
            tma_bulk_g2s(b + (size_t)(2 * f + 1) * gm.row_bytes, Wdown + row * gm.row_bytes, gm.row_bytes,
                         &full[sub & 1]);
        }
    };
    if (warp == 0) {
        if (n_sub > 0) issue(0);
        if (n_sub > 1) issue(1);
    }

    bool timed_out = false;
    for (int sub = 0; sub < n_sub; ++sub) {
        const int f0 = h0 + sub * F, nf = min(F, h1 - f0);
        const uint8_t* b = buf0 + (size_t)(sub & 1) * gm.buf_bytes;
        if (!timed_out && !mbar_wait(&full[sub & 1], (uint32_t)((sub >> 1) & 1))) timed_out = true;

        // Phase A: up dots, one cell per thread.
        if (active) {
            for (int f = prow; f < nf; f += P) {
                const uint8_t* cell = b + (size_t)(2 * f) * gm.row_bytes + s * 144;
                const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
                const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
                const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
                const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                int ia_lo = 0, ib_lo = 0, ia_hi = 0, ib_hi = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t lo = qw[j] & 0x0F0F0F0Fu, hi = qw[j] & 0xF0F0F0F0u;
                    ia_lo = dp4a_us(lo, xa_lo[j], ia_lo);
                    ib_lo = dp4a_uu(lo, xb_lo[j], ib_lo);
                    ia_hi = dp4a_us(hi, xa_hi[j], ia_hi);
                    ib_hi = dp4a_uu(hi, xb_hi[j], ib_hi);
                }
                const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
                uint32_t sc2, m2;
                q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
                const float dot_lo = st_lo * (float)(ia_lo * 256 + ib_lo);
                const float dot_hi = st_hi * (float)((ia_hi * 256 + ib_hi) >> 4);
                part[f * G + c] = d * ((float)(sc2 & 0xff) * dot_lo + (float)(sc2 >> 8) * dot_hi) -
                                  dmin * ((float)(m2 & 0xff) * su_lo + (float)(m2 >> 8) * su_hi);
            }
        }
        __syncthreads();
        for (int f = warp; f < nf; f += GATHER_THREADS / 32) {
            float a = 0.0f;
            for (int i = lane; i < G; i += 32) a += part[f * G + i];
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0) {
                const float gs = hit_score[f0 + f];
                const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
                const float act = (gs * sig) * a;
                act_s[f] = fabsf(act) > ACTIVATION_NOISE_FLOOR ? act : 0.0f;
            }
        }
        __syncthreads();

        // Phase B: down rows, out += act * (d*sc*q - dmin*m), q taken as 128*(f-1) with
        // f = 1 + q/128 built by a byte permute (no int->float conversion).
        if (active) {
            for (int f = prow; f < nf; f += P) {
                const float act = act_s[f];
                if (act == 0.0f) continue;
                const uint8_t* cell = b + (size_t)(2 * f + 1) * gm.row_bytes + s * 144;
                const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
                const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
                const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
                const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
                uint32_t sc2, m2;
                q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
                const float ad = act * d, am = act * dmin;
                const float A_lo = ad * (float)(sc2 & 0xff) * 128.0f, A_hi = ad * (float)(sc2 >> 8) * 128.0f;
                corr_lo += A_lo + am * (float)(m2 & 0xff);
                corr_hi += A_hi + am * (float)(m2 >> 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t lo = (qw[j] & 0x0F0F0F0Fu) | 0x80808080u;
                    const uint32_t hi = ((qw[j] >> 4) & 0x0F0F0F0Fu) | 0x80808080u;
#pragma unroll
                    for (int bb = 0; bb < 4; ++bb) {
                        const float fl = __uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7044u | (bb << 8)));
                        const float fh = __uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7044u | (bb << 8)));
                        acc_lo[4 * j + bb] = fmaf(A_lo, fl, acc_lo[4 * j + bb]);
                        acc_hi[4 * j + bb] = fmaf(A_hi, fh, acc_hi[4 * j + bb]);
                    }
                }
            }
        }
        __syncthreads();
        if (warp == 0 && sub + 2 < n_sub) issue(sub + 2);
    }
    if (__syncthreads_or(timed_out ? 1 : 0)) {
        set_err(err, DEV_ERR_TMA_TIMEOUT);
        if (tid == 0)
            for (int sub = max(0, n_sub - 2); sub < n_sub; ++sub)
                (void)mbar_wait(&full[sub & 1], (uint32_t)((sub >> 1) & 1));
        __syncthreads();
    }

    // Merge the P row-teams' accumulators in team order and write this CTA's partial.
    float* out_s = reinterpret_cast<float*>(buf0);
    for (int p = 0; p < P; ++p) {
        if (active && prow == p) {
            // 64-float chunks at a stride of 65 floats: neighbouring lanes' chunks start one
            // bank apart, so the unrolled element loop is conflict-free
            float* o_lo = out_s + c * 65;
            float* o_hi = o_lo + 32;
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                const float vl = acc_lo[l] - corr_lo, vh = acc_hi[l] - corr_hi;
                if (p == 0) {
                    o_lo[l] = vl;
                    o_hi[l] = vh;
                } else {
                    o_lo[l] += vl;
                    o_hi[l] += vh;
                }
            }
        }
        __syncthreads();
    }
    float* dst = partials + (size_t)blockIdx.x * hidden;
    for (int i = tid; i < hidden; i += GATHER_THREADS) dst[i] = out_s[(i >> 6) * 65 + (i & 63)];
}

// out[h] = residual[h] + sum_p partials[p][h], p ascending inside each of 8 interleaved
// groups and the 8 group sums added in group order: fixed, so run-to-run identical.
__global__ void __launch_bounds__(256) finish_kernel(const float* __restrict__ partials, int n_partials, int hidden,
                                                    const float* __restrict__ residual, float* __restrict__ out,
                                                    TokStride ts) {
    __shared__ float red[8][32];
    partials += ts.part * blockIdx.y;
    if (residual) residual += ts.io * blockIdx.y;
    out += ts.io * blockIdx.y;
    const int col = blockIdx.x * 32 + threadIdx.x, y = threadIdx.y;
    float a = 0.0f;
    if (col < hidden) {
#pragma unroll 4
        for (int p = y; p < n_partials; p += 8) a += partials[(size_t)p * hidden + col];
    }
    red[y][threadIdx.x] = a;
    __syncthreads();
    if (y == 0 && col < hidden) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x];
        out[col] = residual ? residual[col] + t : t;
    }
}

}  // namespace

int gather_q4k_grid(int sm_count) { return sm_count; }

cudaError_t launch_gather_q4k(const Q4kMat& up, const Q4kMat& down, const XPrep& xp, const uint32_t* hit_idx,
                              const float* hit_score, const int* n_hits_dev, int n_hits_host, float* partials,
                              int grid, int* err, cudaStream_t st, int batch, TokStride ts) {
    GatherGeom g;
    if (up.cols != down.cols || !gather_geom(up.cols, g)) return cudaErrorInvalidValue;
    cudaError_t e = set_max_dyn_smem((const void*)gather_q4k_kernel, 220 * 1024);
    if (e != cudaSuccess) return e;
    gather_q4k_kernel<<<dim3(grid, batch), GATHER_THREADS, g.smem_bytes, st>>>(up.w, down.w, g, xp, hit_idx, hit_score,
                                                                              n_hits_dev, n_hits_host, partials, err, ts);
    return cudaGetLastError();
}

cudaError_t launch_finish(const float* partials, int n_partials, int hidden, const float* residual, float* out,
                          cudaStream_t st, int batch, TokStride ts) {
    finish_kernel<<<dim3((hidden + 31) / 32, batch), dim3(32, 8), 0, st>>>(partials, n_partials, hidden, residual, out, ts);
    return cudaGetLastError();
}

}  // namespace lq
