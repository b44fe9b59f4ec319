// Internal launch interface between the C-ABI layer and the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

namespace lq {

// Per-token selection record written by the select kernels.
struct SelHeader {
    int n_in;      // rows certainly in the top-K (fast |score| above the band)
    int n_band;    // rows whose membership needs the exact reference score
    int n_sel;     // final number of hits (min(K, N))
    int need;      // K - n_in: how many band rows make it
    float tau;     // K-th largest fast |score|
    float bound;   // B = max row error bound; band is |s| in [tau-2B, tau+2B]
    int done_ctr;  // rescore CTAs finished (last one runs the final pick)
    uint32_t bound_bits;  // running max of the scan's row error bounds (f32 bits; consumed by classify)
};

// Per-token workspace views (device pointers).
struct TokenWs {
    float* xn;
    uint32_t* xa;
    uint32_t* xb;
    float* bscale;
    float* bsum;
    float* babs;
    float* scores;      // [N] fast gate scores
    uint32_t* hist;     // [LQ_HIST_BINS] histogram of fast |score| keys >> LQ_HIST_SHIFT (zero between uses)
    SelHeader* sel;
    uint32_t* hit_idx;  // [N] final hits: certain rows (ascending), then picked band rows (ascending)
    float* hit_score;   // [N] gate score per hit (exact for band rows)
    uint32_t* band_idx; // [N]
    float* band_exact;  // [N] exact reference-order score per band row
};

// Batched launches: the kernels below take the views of token 0 and advance every per-token
// pointer by a constant byte stride per token (blockIdx.y).
struct TokStride {
    size_t ws;    // bytes between two tokens' workspaces (TokenWs / XPrep members)
    size_t io;    // floats between two tokens' residual / output rows
    size_t part;  // floats between two tokens' partial-output blocks
};
#ifdef __CUDACC__
template <class T>
__host__ __device__ __forceinline__ T* tok_off(T* p, size_t bytes) {
    return p ? reinterpret_cast<T*>(reinterpret_cast<uintptr_t>(p) + bytes) : p;
}
__host__ __device__ __forceinline__ TokenWs ws_at(TokenWs w, size_t b) {
    w.xn = tok_off(w.xn, b); w.xa = tok_off(w.xa, b); w.xb = tok_off(w.xb, b);
    w.bscale = tok_off(w.bscale, b); w.bsum = tok_off(w.bsum, b); w.babs = tok_off(w.babs, b);
    w.scores = tok_off(w.scores, b); w.hist = tok_off(w.hist, b); w.sel = tok_off(w.sel, b);
    w.hit_idx = tok_off(w.hit_idx, b); w.hit_score = tok_off(w.hit_score, b);
    w.band_idx = tok_off(w.band_idx, b); w.band_exact = tok_off(w.band_exact, b);
    return w;
}
__device__ __forceinline__ XPrep xp_at(XPrep x, size_t b) {
    x.xn = tok_off(x.xn, b); x.xa = tok_off(x.xa, b); x.xb = tok_off(x.xb, b);
    x.scale = tok_off(x.scale, b); x.sum = tok_off(x.sum, b); x.abs = tok_off(x.abs, b);
    return x;
}
#endif

// Coarse histogram of |score| bit patterns: 8 exponent + 6 mantissa bits.
#define LQ_HIST_SHIFT 17
#define LQ_HIST_BINS 16384

struct Q4kMat {
    const uint8_t* w;  // [rows][cols/256*144]
    int rows;
    int cols;
};

// A block-format matrix other than Q4_K (device pointers).
struct FmtMat {
    int fmt;               // LQ_FMT_Q8_0 / LQ_FMT_MXFP4 / LQ_FMT_NVFP4
    const uint8_t* data;   // blocks or packed codes
    const uint8_t* scales; // MXFP4 e8m0 / NVFP4 e4m3 stream
    float ts;              // NVFP4 tensor scale
    int rows, cols;
};

// launch_util.cu: cudaFuncAttributeMaxDynamicSharedMemorySize, set once per (device, kernel)
cudaError_t set_max_dyn_smem(const void* func, int bytes);

// fmt_kernels.cu
cudaError_t launch_scan_fmt(const FmtMat& m, const XPrep& xp, float* scores, uint32_t* hist, uint32_t* bound_bits,
                            float c1, int* err, int sm_count, cudaStream_t st);
cudaError_t launch_hist_abs(const float* scores, int n, uint32_t* hist, cudaStream_t st);
// Scores in the reference's exact element order (one thread per row).
cudaError_t launch_scan_exact_fmt(const FmtMat& m, const float* xn, float* scores, int* err, cudaStream_t st);
cudaError_t launch_rescore_fmt(const FmtMat& m, const float* xn, const uint32_t* rows_idx, const int* n_rows_dev,
                               int n_rows_host, float* out, int sm_count, cudaStream_t st);
cudaError_t launch_gather_fmt(const FmtMat& up, const FmtMat& down, const XPrep& xp, const uint32_t* hit_idx,
                              const float* hit_score, const int* n_hits_dev, int n_hits_host, float* partials,
                              int grid, cudaStream_t st);
// Pair-batched launches for a mixture-of-experts layer: pair y = (token, one of its experts) uses workspace y
// (a constant stride apart) and the matrices of expert pair_expert[y] from a device table.
cudaError_t launch_scan_exact_pairs(int fmt, const FmtMat* table, const uint32_t* pair_expert, int n_pairs, int rows,
                                    int cols, TokenWs ws0, size_t ws_stride, int* err, cudaStream_t st);
cudaError_t launch_gather_fmt_pairs(int fmt, const FmtMat* up_table, const FmtMat* down_table,
                                    const uint32_t* pair_expert, int n_pairs, int cols, TokenWs ws0, size_t ws_stride,
                                    float* partials, int grid_x, cudaStream_t st);
// moe.cu: softmax over all experts, top-k by (value desc, index asc), optional renormalisation
cudaError_t launch_moe_route(const float* logits, int n_tokens, int n_experts, int top_k, int renormalise,
                             uint32_t* idx_out, float* w_out, cudaStream_t st);
// rows_out[p] = x[p / per_token] for p < n_tokens * per_token (every pair gets its token's activation)
cudaError_t launch_moe_replicate(const float* x, int n_tokens, int per_token, int hidden, float* rows_out, cudaStream_t st);
// out[t] = sum_j w[t][j] * (sum_c partials[t * per_token + j][c]), c and j ascending: fixed order
cudaError_t launch_moe_combine(const float* partials, const float* w, int n_tokens, int per_token, int n_partials,
                               int hidden, float* out, cudaStream_t st);

// prep.cu
void launch_prep(const float* x_in, int batch, int hidden, int apply_norm, double eps, float* xn, uint32_t* xa,
                 uint32_t* xb, float* bscale, float* bsum, float* babs, size_t token_stride_f, int* err,
                 cudaStream_t st);

// scan_q4k.cu
int scan_q4k_smem_bytes(int hidden);
// Fast scores of every row for one token.  When hist != nullptr the kernel also adds every
// row's |score| key to the coarse histogram and folds the largest row error bound into
// *bound_bits (atomic max on the f32 bit pattern).
cudaError_t launch_scan_q4k(const Q4kMat& m, const XPrep& xp, float* scores, uint32_t* hist, uint32_t* bound_bits,
                            float c1, int* err, int sm_count, cudaStream_t st);
// Exact reference-order (sum_x form) scores for the rows listed in rows_idx[0..*n_rows), or for
// all rows when rows_idx == nullptr.  When sel != nullptr the last CTA to finish runs the final pick.
cudaError_t launch_rescore_q4k(const Q4kMat& m, const float* xn, const uint32_t* rows_idx, const int* n_rows_dev,
                               int n_rows_host, float* out, TokenWs ws, int top_k, int run_final, int* err,
                               int sm_count, cudaStream_t st, int batch = 1, size_t ws_stride = 0);
// scan_q4k_mma.cu: fast scores of every row for `batch` tokens at once on the tensor cores
// (integer dots of the 4-bit weights against the tokens' fixed-point planes), with the histogram
// and the bound of every token as launch_scan_q4k leaves them.
// scan_q4k_tc.cu: the same contract on tcgen05 (kind::i8, accumulators in tensor memory); batch <= 32 per launch
size_t scan_q4k_tc_scratch_bytes(int cols);
cudaError_t launch_scan_q4k_tc(const Q4kMat& m, TokenWs ws0, size_t ws_stride, int batch, int want_hist, float c1,
                               uint8_t* scratch, int* err, cudaStream_t st);
cudaError_t launch_scan_q4k_mma(const Q4kMat& m, TokenWs ws0, size_t ws_stride, int batch, int want_hist, float c1,
                                int* err, int sm_count, cudaStream_t st);

// select.cu
cudaError_t launch_select(const float* scores, int n, int top_k, TokenWs ws, int* err, cudaStream_t st, int batch = 1,
                          size_t ws_stride = 0);
// Band classification from the scan's coarse histogram (walk path).
cudaError_t launch_classify(const float* scores, int n, int top_k, TokenWs ws, int* err, cudaStream_t st,
                            int batch = 1, size_t ws_stride = 0);
// The same classification by several CTAs per token (launch_classify takes this route for many rows);
// band_scores: band_exact takes the band rows' scores (they are exact already).
cudaError_t launch_classify_mc(const float* scores, int n, int top_k, TokenWs ws, cudaStream_t st, int batch,
                               size_t ws_stride, int band_scores);
// Stand-alone exact top-K by |score| (ties -> lower index), sorted (|v| desc, idx asc).
cudaError_t launch_topk_abs_sorted(const float* scores, int n, int top_k, uint32_t* idx_out, float* val_out,
                                   int* count_out, void* scratch, int* err, cudaStream_t st);

// Top-K by value (descending, ties to the lower index), sorted; top_k <= 16384.
cudaError_t launch_topk_value_sorted(const float* scores, int n, int top_k, uint32_t* idx_out, float* val_out, int* err,
                                     cudaStream_t st);
// dense16.cu: gemv over f16 (kind 0) / bf16 (kind 1) weights [n, k]; exact = the reference loop's order
cudaError_t launch_gemv16(const void* w, const float* x, int n, int k, int kind, int exact, float* out, cudaStream_t st);

// kquant_rows.cu: Q6_K rows, the walk's gather with up / down each Q4_K or Q6_K, the fused gate+up matvec
cudaError_t launch_q6k_matvec(const uint8_t* w, const float* x, const uint32_t* rows_idx, const int* n_rows_dev,
                              int n_rows, int cols, float* out, int* err, int sm_count, cudaStream_t st);
cudaError_t launch_q6k_dequant(const uint8_t* data, size_t n_elems, float* out, cudaStream_t st);
cudaError_t launch_gather_kquant(int up_fmt, const uint8_t* up, int down_fmt, const uint8_t* down, const float* xn,
                                 int cols, const uint32_t* hit_idx, const float* hit_score, const int* n_hits_dev,
                                 int n_hits_host, float* partials, int grid, cudaStream_t st);
cudaError_t launch_q4k_dual_matvec(const uint8_t* wa, const uint8_t* wb, const float* x, int rows, int cols,
                                   float* out_a, float* out_b, int sm_count, cudaStream_t st);

// gather_q4k.cu
int gather_q4k_grid(int sm_count);
cudaError_t launch_gather_q4k(const Q4kMat& up, const Q4kMat& down, const XPrep& xp, const uint32_t* hit_idx,
                              const float* hit_score, const int* n_hits_dev, int max_hits, float* partials,
                              int grid, int* err, cudaStream_t st, int batch = 1, TokStride ts = TokStride{0, 0, 0});
// out[h] = (residual ? residual[h] : 0) + sum_c partials[c][h]   (fixed order)
cudaError_t launch_finish(const float* partials, int n_partials, int hidden, const float* residual, float* out,
                          cudaStream_t st, int batch = 1, TokStride ts = TokStride{0, 0, 0});

// walk_fused_q4k.cu — the fused persistent walk (one token, all layers, one cooperative launch)
bool fused_q4k_supported(int hidden, int n_rows, int top_k, int sm_count);
size_t fused_q4k_ws_bytes(int hidden, int n_rows, int sm_count);
int fused_q4k_stamp_count();
size_t fused_q4k_ws_dirty_bytes();
}  // namespace lq
