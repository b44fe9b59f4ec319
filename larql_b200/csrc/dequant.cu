// Block decoders on the device: the reference's dequantisers, element for element, in
// its exact association (no fused multiply-add), for the bit-exact weight check.
//   Q4_K : (d*sc)*q - (dmin*m)        crates/larql-models/src/quant/ggml/q4_k.rs:286-338
//   Q8_0 : (q as f32) * d              crates/larql-models/src/quant/ggml/legacy.rs:68-83
//   MXFP4: TABLE[code] * 2^(e-127)     crates/larql-models/src/quant/mxfp4.rs:42-95
//   NVFP4: (ts * e4m3(s)) * e2m1(code) crates/larql-models/src/quant/nvfp4.rs:192-222
#include "../../include/larql_cuda.h"
#include "codecs.cuh"
#include "kernels.h"

namespace lq {

namespace {

__global__ void dequant_kernel(int fmt, const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                               float ts, long long rows, long long cols, float* __restrict__ out) {
    const long long n = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i % cols;
        float v;
        if (fmt == LQ_FMT_Q4_K) {
            const uint8_t* b = data + (r * (cols / 256) + c / 256) * 144;
            const int e = (int)(c % 256), j = e / 32, l = e % 32;
            const uint32_t dm = *reinterpret_cast<const uint32_t*>(b);
            const float d = f16_bits_to_f32(dm), dmin = f16_bits_to_f32(dm >> 16);
            uint32_t sc, m;
            q4k_scale_min(b + 4, j, sc, m);
            const uint32_t byte = b[16 + (j / 2) * 32 + l];
            const uint32_t q = (j & 1) ? (byte >> 4) : (byte & 0x0f);
            v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
        } else if (fmt == LQ_FMT_Q8_0) {
            const uint8_t* b = data + (r * (cols / 32) + c / 32) * 34;
            const float d = f16_bits_to_f32((uint32_t)b[0] | ((uint32_t)b[1] << 8));
            v = __fmul_rn((float)(int8_t)b[2 + c % 32], d);
        } else if (fmt == LQ_FMT_MXFP4) {
            const long long g = r * (cols / 32) + c / 32;
            const uint32_t byte = data[g * 16 + (c % 32) / 2];
            const uint32_t code = (c & 1) ? (byte >> 4) : (byte & 0x0f);
            v = __fmul_rn(e2m1_to_f32(code), e8m0_to_f32(scales[g]));
        } else {
            const long long g = r * (cols / 16) + c / 16;
            const uint32_t byte = data[g * 8 + (c % 16) / 2];
            const uint32_t code = (c & 1) ? (byte >> 4) : (byte & 0x0f);
            const float step = __fmul_rn(ts, e4m3_to_f32(scales[g]));
            v = __fmul_rn(step, e2m1_to_f32(code));
        }
        out[i] = v;
    }
}

}  // namespace

cudaError_t launch_dequantize(const lq_matrix& m, float* out, cudaStream_t st) {
    const long long n = (long long)m.rows * m.cols;
    if (n == 0) return cudaSuccess;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    dequant_kernel<<<(int)blocks, 256, 0, st>>>(m.fmt, (const uint8_t*)m.data, (const uint8_t*)m.scales,
                                                m.tensor_scale, m.rows, m.cols, out);
    return cudaGetLastError();
}

}  // namespace lq
