// Dense gemv over f16 / bf16 weight matrices (the device seam of VINDEX3 execution:
// MatMul::f16_gemv / bf16_gemv and their _multi forms, crates/larql-compute/src/backend/matmul.rs:124-205,
// as DevicePlanBackend calls them, crates/larql-vindex/src/format/vindex3/opplan/exec/device.rs:256-341).
//
//   out[n] = sum_k widen(W[n, k]) * x[k]
//
// exact order: one running f32 sum per row, k ascending, product rounded before the add — the loop of the
// reference's test device (…/opplan/exec/tests/device.rs:68-84); the CPU backend itself has no f16 / bf16
// gemv.  A warp stages 64 columns of its 32 rows with coalesced loads, then every lane walks its own row.
// fast order: one warp per row, lanes stride the columns, tree reduction.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"

namespace lq {

namespace {

__device__ __forceinline__ float widen16(unsigned short bits, int kind) {
    return kind == 0 ? __half2float(__ushort_as_half(bits)) : __uint_as_float((uint32_t)bits << 16);
}

constexpr int G16_CHUNK = 64;  // columns staged per step

__global__ void __launch_bounds__(128) gemv16_exact_kernel(const unsigned short* __restrict__ w, const float* __restrict__ x,
                                                           int n, int k, int kind, float* __restrict__ out) {
    extern __shared__ __align__(16) float xs[];                   // [k]
    __shared__ unsigned short stage[4][32][G16_CHUNK + 2];       // +2: rows land in different banks
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < k; i += 128) xs[i] = x[i];
    __syncthreads();
    const int row0 = (blockIdx.x * 4 + warp) * 32;
    if (row0 >= n) return;
    const int rows = min(32, n - row0);
    float acc = 0.0f;
    for (int c0 = 0; c0 < k; c0 += G16_CHUNK) {
        const int cols = min(G16_CHUNK, k - c0);
        for (int r = 0; r < rows; ++r) {
            const unsigned short* src = w + (size_t)(row0 + r) * k + c0;
            for (int c = lane; c < cols; c += 32) stage[warp][r][c] = src[c];
        }
        __syncwarp();
        if (lane < rows)
            for (int c = 0; c < cols; ++c) acc = __fadd_rn(acc, __fmul_rn(widen16(stage[warp][lane][c], kind), xs[c0 + c]));
        __syncwarp();
    }
    if (lane < rows) out[row0 + lane] = acc;
}

__global__ void __launch_bounds__(256) gemv16_fast_kernel(const unsigned short* __restrict__ w, const float* __restrict__ x,
                                                          int n, int k, int kind, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= n) return;
    const unsigned short* src = w + (size_t)row * k;
    float acc = 0.0f;
    for (int c = lane; c < k; c += 32) acc = fmaf(widen16(src[c], kind), x[c], acc);
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[row] = acc;
}

}  // namespace

cudaError_t launch_gemv16(const void* w, const float* x, int n, int k, int kind, int exact, float* out, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    if (exact) {
        const size_t smem = (size_t)k * sizeof(float);
        cudaError_t e = set_max_dyn_smem((const void*)gemv16_exact_kernel, 128 * 1024);
        if (e != cudaSuccess) return e;
        gemv16_exact_kernel<<<(n + 127) / 128, 128, smem, st>>>((const unsigned short*)w, x, n, k, kind, out);
    } else {
        gemv16_fast_kernel<<<(n + 7) / 8, 256, 0, st>>>((const unsigned short*)w, x, n, k, kind, out);
    }
    return cudaGetLastError();
}

}  // namespace lq
