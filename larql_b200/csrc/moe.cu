// MoE router: softmax over all experts (max-subtracted), top-k by (value descending, index
// ascending), optional renormalisation over the selected weights — moe_route_from_router_input
// (crates/larql-compute/src/cpu/ops/moe/mod.rs:149-189) with softmax and top_k from
// crates/larql-compute/src/cpu/ops/moe/math.rs:130-164.  One thread per token: the expert count
// is small (tens) and the order of the f32 sum is the reference's sequential one.
#include "kernels.h"

namespace lq {

namespace {

constexpr int MOE_MAX_EXPERTS = 256;

__global__ void moe_route_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int top_k,
                                 int renormalise, uint32_t* __restrict__ idx_out, float* __restrict__ w_out) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tokens) return;
    const float* v = logits + (size_t)t * n_experts;
    float p[MOE_MAX_EXPERTS];
    float mx = -INFINITY;
    for (int i = 0; i < n_experts; ++i) mx = fmaxf(mx, v[i]);
    float sum = 0.0f;
    for (int i = 0; i < n_experts; ++i) {
        p[i] = expf(__fsub_rn(v[i], mx));
        sum = __fadd_rn(sum, p[i]);
    }
    if (sum > 0.0f)
        for (int i = 0; i < n_experts; ++i) p[i] = __fdiv_rn(p[i], sum);
    const int k = min(top_k, n_experts);
    unsigned long long used[MOE_MAX_EXPERTS / 64] = {0, 0, 0, 0};
    float wsum = 0.0f;
    for (int j = 0; j < k; ++j) {
        int best = -1;
        for (int i = 0; i < n_experts; ++i) {
            if (used[i >> 6] >> (i & 63) & 1ull) continue;
            if (best < 0 || p[i] > p[best]) best = i;
        }
        used[best >> 6] |= 1ull << (best & 63);
        idx_out[(size_t)t * k + j] = (uint32_t)best;
        w_out[(size_t)t * k + j] = p[best];
        wsum = __fadd_rn(wsum, p[best]);
    }
    if (renormalise && wsum > 0.0f)
        for (int j = 0; j < k; ++j) w_out[(size_t)t * k + j] = __fdiv_rn(w_out[(size_t)t * k + j], wsum);
}

__global__ void moe_replicate_kernel(const float* __restrict__ x, int per_token, int hidden, float* __restrict__ out) {
    const float* src = x + (size_t)(blockIdx.y / per_token) * hidden;
    float* dst = out + (size_t)blockIdx.y * hidden;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// One thread per output column of a token: the experts' outputs (each the fixed-order sum of its partial blocks)
// weighted by the routing weights, in slot order (crates/larql-compute/src/cpu/ops/moe/forward.rs:24-140 adds the
// selected experts' outputs, scaled by their weights, in selection order).
__global__ void moe_combine_kernel(const float* __restrict__ partials, const float* __restrict__ w, int per_token,
                                   int n_partials, int hidden, float* __restrict__ out) {
    const int t = blockIdx.y, col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= hidden) return;
    float acc = 0.0f;
    for (int j = 0; j < per_token; ++j) {
        const float* p = partials + ((size_t)(t * per_token + j) * n_partials) * hidden + col;
        float s = 0.0f;
        for (int c = 0; c < n_partials; ++c) s += p[(size_t)c * hidden];
        acc = fmaf(w[t * per_token + j], s, acc);
    }
    out[(size_t)t * hidden + col] = acc;
}

}  // namespace

cudaError_t launch_moe_replicate(const float* x, int n_tokens, int per_token, int hidden, float* rows_out, cudaStream_t st) {
    if (n_tokens <= 0 || per_token <= 0) return cudaSuccess;
    moe_replicate_kernel<<<dim3((hidden + 1023) / 1024, n_tokens * per_token), 256, 0, st>>>(x, per_token, hidden, rows_out);
    return cudaGetLastError();
}

cudaError_t launch_moe_combine(const float* partials, const float* w, int n_tokens, int per_token, int n_partials,
                               int hidden, float* out, cudaStream_t st) {
    if (n_tokens <= 0) return cudaSuccess;
    moe_combine_kernel<<<dim3((hidden + 255) / 256, n_tokens), 256, 0, st>>>(partials, w, per_token, n_partials, hidden, out);
    return cudaGetLastError();
}

cudaError_t launch_moe_route(const float* logits, int n_tokens, int n_experts, int top_k, int renormalise,
                             uint32_t* idx_out, float* w_out, cudaStream_t st) {
    if (n_experts > MOE_MAX_EXPERTS || n_experts <= 0) return cudaErrorInvalidValue;
    if (n_tokens <= 0) return cudaSuccess;
    moe_route_kernel<<<(n_tokens + 63) / 64, 64, 0, st>>>(logits, n_tokens, n_experts, top_k, renormalise, idx_out,
                                                         w_out);
    return cudaGetLastError();
}

}  // namespace lq
