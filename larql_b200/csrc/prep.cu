// Activation preparation: optional RMSNorm, then a 16-bit fixed-point copy of the
// vector per 32-element block (two byte planes for dp4a) with per-block step, sum
// and absolute sum.  One CTA per token.
//
// RMSNorm follows the reference's rms_norm_eps with unit weight
// (crates/larql-compute/src/residual.rs:56-78): f64 sum of squares,
// rms = (float)sqrt(sq/H + eps), out = x / rms * 1.0.  The f64 sum is taken as a
// fixed-shape tree, so it can differ from the sequential sum in the last f64 bit;
// after the cast to f32 the result is the reference's except with probability
// around 1e-8.
#include "kernels.h"

namespace lq {

namespace {

constexpr int PREP_THREADS = 1024;

__global__ void __launch_bounds__(PREP_THREADS) prep_kernel(const float* __restrict__ x_in, int hidden,
                                                           int apply_norm, double eps, float* xn, uint32_t* xa,
                                                           uint32_t* xb, float* bscale, float* bsum, float* babs,
                                                           size_t stride_f, int* err) {
    const int tok = blockIdx.x;
    const float* x = x_in + (size_t)tok * hidden;
    // Every per-token array advances by the same stride (in 4-byte words) per token.
    float* o_xn = xn + tok * stride_f;
    uint32_t* o_xa = xa + tok * stride_f;
    uint32_t* o_xb = xb + tok * stride_f;
    float* o_sc = bscale + tok * stride_f;
    float* o_su = bsum + tok * stride_f;
    float* o_ab = babs + tok * stride_f;

    __shared__ double red[PREP_THREADS / 32];
    __shared__ float s_rms;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    float rms = 1.0f;
    if (apply_norm) {
        double sq = 0.0;
        for (int i = tid; i < hidden; i += PREP_THREADS) {
            const double v = (double)x[i];
            sq += v * v;
        }
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) red[warp] = sq;
        __syncthreads();
        if (warp == 0) {
            double t = red[lane];
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0) s_rms = (float)sqrt(t / (double)hidden + eps);
        }
        __syncthreads();
        rms = s_rms;
    }

    // One warp per 32-element block, lane = element.
    const int n_blocks = hidden / 32;
    for (int blk = warp; blk < n_blocks; blk += PREP_THREADS / 32) {
        const int i = blk * 32 + lane;
        float v = x[i];
        if (apply_norm) v = __fmul_rn(__fdiv_rn(v, rms), 1.0f);
        o_xn[i] = v;
        if (!isfinite(v)) set_err(err, DEV_ERR_NAN_SCORE);  // the reference's top-K panics on NaN scores
        float amax = fabsf(v), sum = v, asum = fabsf(v);
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            asum += __shfl_xor_sync(0xffffffffu, asum, o);
        }
        const float step = amax / 32767.0f;
        const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
        int q = __float2int_rn(v * inv);
        q = max(-32767, min(32767, q));
        const uint32_t a = (uint32_t)((q >> 8) & 0xff), b = (uint32_t)(q & 0xff);
        uint32_t wa = a << (8 * (lane & 3)), wb = b << (8 * (lane & 3));
        wa |= __shfl_xor_sync(0xffffffffu, wa, 1);
        wb |= __shfl_xor_sync(0xffffffffu, wb, 1);
        wa |= __shfl_xor_sync(0xffffffffu, wa, 2);
        wb |= __shfl_xor_sync(0xffffffffu, wb, 2);
        if ((lane & 3) == 0) {
            o_xa[blk * 8 + (lane >> 2)] = wa;
            o_xb[blk * 8 + (lane >> 2)] = wb;
        }
        if (lane == 0) {
            o_sc[blk] = step;
            o_su[blk] = sum;
            o_ab[blk] = asum;
        }
    }
}

}  // namespace

void launch_prep(const float* x_in, int batch, int hidden, int apply_norm, double eps, float* xn, uint32_t* xa,
                 uint32_t* xb, float* bscale, float* bsum, float* babs, size_t token_stride_f, int* err,
                 cudaStream_t st) {
    if (batch <= 0 || hidden <= 0) return;
    prep_kernel<<<batch, PREP_THREADS, 0, st>>>(x_in, hidden, apply_norm, eps, xn, xa, xb, bscale, bsum, babs,
                                                token_stride_f, err);
}

}  // namespace lq
