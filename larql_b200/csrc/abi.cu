// C ABI of the backend: context, weight residency cache, workspace, and the entry
// points declared in include/larql_cuda.h.  Host-side policy only; all arithmetic is
// in the kernels.  There is deliberately no CPU path here: a missing device is an
// error, an unsupported case is a refusal status.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>  // types and prototypes only: the library itself is loaded on demand (lq_comm_init)

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/larql_cuda.h"
#include "kernels.h"

using namespace lq;

namespace lq {
cudaError_t launch_final_pick(TokenWs ws, int* err, cudaStream_t st, int batch = 1, size_t ws_stride = 0);
cudaError_t launch_topk_abs_sorted(const float* scores, int n, int top_k, TokenWs ws, uint32_t* idx_out,
                                   float* val_out, int* count_out, unsigned long long* sort_buf, int* err,
                                   cudaStream_t st);
cudaError_t launch_dequantize(const lq_matrix& m, float* out, cudaStream_t st);
cudaError_t launch_quantize_q4k(const float* data, size_t n_elems, uint8_t* out, cudaStream_t st);
cudaError_t launch_shard_bound_max(const uint32_t* slots, int world, uint32_t* bound_bits, cudaStream_t st);
cudaError_t launch_shard_pack(TokenWs ws, uint32_t row_offset, int cap, int32_t* pack, int* err, cudaStream_t st);
cudaError_t launch_shard_pick(const int32_t* packs, int world, int rank, int cap, int top_k, uint32_t row_offset,
                              TokenWs ws, int* err, cudaStream_t st);
cudaError_t launch_walk_fused_q4k(const void* layers_dev, const uint8_t* const* single, int n_layers, int n_rows,
                                  int hidden, int top_k, uint32_t flags, float c1, const float* h_in, float* h_out,
                                  uint8_t* ws, uint32_t* hit_out, uint32_t* count_out, lq_walk_stats* stats_dev,
                                  int* err, int sm_count, cudaStream_t st);
size_t fused_q4k_xarea_bytes(int hidden, int n_rows_global, int world);
bool fused_q4k_sharded_supported(int hidden, int n_rows_local, int n_rows_global, int top_k, int world, int sm_count);
cudaError_t launch_walk_fused_q4k_sharded(const void* layers_dev, int n_layers, int n_rows_local, int n_rows_global,
                                          int hidden, int top_k, uint32_t flags, float c1, const float* h_in,
                                          float* h_out, uint8_t* ws, uint32_t* hit_out, uint32_t* count_out,
                                          lq_walk_stats* stats_dev, int* err, int sm_count, int world, int rank,
                                          uint8_t* const* areas, const int* row_offsets, uint32_t xepoch0,
                                          cudaStream_t st);
}  // namespace lq

struct lq_stack {
    std::vector<lq_matrix> gates, ups, downs;
    size_t batch = 0, top_k = 0;
    uint32_t flags = 0;
    int hidden = 0;
    float *h_in = nullptr, *h_out = nullptr, *h_buf[2] = {nullptr, nullptr};
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    void* layers_dev = nullptr;  // fused path: n_layers x {gate, up, down}
    bool fused = false;
    // feature-sharded stack (one rank's row range of every layer)
    bool sharded = false;
    size_t row_offset = 0, cap = 0;
    uint32_t* hist_buf = nullptr;   // [LQ_HIST_WORDS]
    int32_t* pack = nullptr;        // [2 + 2 cap]
    int32_t* packs = nullptr;       // [world][2 + 2 cap]
    float* out_partial = nullptr;   // [hidden]
    // sharded stack on the fused persistent kernel: the ranks exchange through each other's memory
    bool xfused = false;
    size_t n_global = 0;
    uint8_t* xarea = nullptr;             // this rank's exchange area
    std::vector<uint8_t*> areas;          // every rank's area as mapped here (areas[rank] == xarea)
    std::vector<int> row_offs;            // first global row of every rank
    uint32_t xepoch = 0;                  // layers walked so far on these areas (epoch of the exchange lines)
    uint32_t* xhits = nullptr;            // [top_k] rows of the last layer's selection + [1] their count
    uint32_t* sync_word = nullptr;        // one word for the launch rendezvous
};

struct lq_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    std::string last_error;
    std::string info;
    int* d_err = nullptr;
    uint64_t launches = 0;

    struct Region {
        const uint8_t* host;
        size_t len;
        uint8_t* dev;
    };
    std::vector<Region> regions;
    bool sealed = false;

    // workspace (grown on demand, never during graph capture)
    size_t ws_batch = 0, ws_hidden = 0, ws_feat = 0;
    uint8_t* ws_raw = nullptr;
    std::vector<TokenWs> tok;
    float* partials = nullptr;
    int gather_grid = 0;
    size_t batch_min = 2;  // smallest batch that takes the batched (tensor-core scan) path
    unsigned long long* sort_buf = nullptr;
    size_t sort_cap = 0;
    // staging for the host-pointer API
    uint8_t* stage = nullptr;
    size_t stage_cap = 0;
    lq_walk_stats stats = {};
    // fused persistent walk: control block + partials + residual ping-pong (zero-initialised)
    uint8_t* fws = nullptr;
    size_t fws_cap = 0;
    lq_walk_stats* stats_dev = nullptr;
    bool use_fused = true;
    bool last_fused = false;
    // batched gate scan: tcgen05 (default) or the mma.sync kernel (LARQL_B200_BATCH_SCAN=mma)
    bool use_tc_scan = true;
    uint8_t* tc_scratch = nullptr;
    size_t tc_scratch_cap = 0;
    // multi-GPU: one NCCL communicator per context (lq_comm_init)
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    const lq_stack* last_xstack = nullptr;  // sharded fused stack that ran last (its selection: lq_dev_shard_hits)
};

namespace {

// Every entry point runs with its context's device current (a host may hold contexts on several
// GPUs in one process and call them from any thread) and puts the caller's device back afterwards.
struct DevGuard {
    int prev = -1;
    explicit DevGuard(const lq_ctx* c) {
        if (!c) return;
        int cur = -1;
        if (cudaGetDevice(&cur) == cudaSuccess && cur != c->device && cudaSetDevice(c->device) == cudaSuccess) prev = cur;
    }
    ~DevGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
    DevGuard(const DevGuard&) = delete;
    DevGuard& operator=(const DevGuard&) = delete;
};

// NCCL is loaded when the first communicator is made, so the library has no link-time dependency on it
// (a single-GPU host needs none).
struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api.lib ? &api : nullptr;
    tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return nullptr;
#define LQ_SYM(field, name)                                             \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name)); \
    if (!api.field) return nullptr;
    LQ_SYM(GetUniqueId, "ncclGetUniqueId")
    LQ_SYM(CommInitRank, "ncclCommInitRank")
    LQ_SYM(CommDestroy, "ncclCommDestroy")
    LQ_SYM(AllReduce, "ncclAllReduce")
    LQ_SYM(AllGather, "ncclAllGather")
    LQ_SYM(GetErrorString, "ncclGetErrorString")
#undef LQ_SYM
    api.lib = h;
    return &api;
}

__global__ void add_vec_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

int fail(lq_ctx* c, int code, const std::string& msg) {
    if (c) c->last_error = msg;
    return code;
}
int cuda_fail(lq_ctx* c, cudaError_t e, const char* what) {
    return fail(c, LQ_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
#define CK(call)                                             \
    do {                                                     \
        cudaError_t e__ = (call);                            \
        if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #call); \
    } while (0)

size_t a256(size_t v) { return (v + 255) / 256 * 256; }

size_t row_bytes_of(int fmt, int64_t cols) {
    switch (fmt) {
        case LQ_FMT_Q4_K: return (size_t)(cols / 256) * 144;
        case LQ_FMT_Q8_0: return (size_t)(cols / 32) * 34;
        case LQ_FMT_MXFP4: return (size_t)(cols / 32) * 16;
        case LQ_FMT_NVFP4: return (size_t)(cols / 16) * 8;
        case LQ_FMT_Q6_K: return (size_t)(cols / 256) * 210;
    }
    return 0;
}

// Shape rule per format; mirrors KernelShapeError::check (>= for Q4_K) and the exact-length
// checks of q8_0_gemv / nvfp4_gemv.
int check_matrix(lq_ctx* ctx, const lq_matrix* m, const char* name) {
    if (!m || m->rows < 0 || m->cols < 0) return fail(ctx, LQ_ERR_ARGUMENT, std::string(name) + ": null/negative");
    const int64_t r = m->rows, k = m->cols;
    switch (m->fmt & 0xff) {
        case LQ_FMT_Q4_K:
            if (k % 256 != 0 || m->data_len < (size_t)r * row_bytes_of(LQ_FMT_Q4_K, k))
                return fail(ctx, LQ_REFUSED_SHAPE, std::string(name) + ": Q4_K geometry");
            break;
        case LQ_FMT_Q6_K:
            if (k % 256 != 0 || m->data_len < (size_t)r * row_bytes_of(LQ_FMT_Q6_K, k))
                return fail(ctx, LQ_REFUSED_SHAPE, std::string(name) + ": Q6_K geometry");
            break;
        case LQ_FMT_Q8_0:
            if (k == 0 || k % 32 != 0 || m->data_len != (size_t)r * row_bytes_of(LQ_FMT_Q8_0, k))
                return fail(ctx, LQ_REFUSED_SHAPE, std::string(name) + ": Q8_0 geometry");
            break;
        case LQ_FMT_MXFP4:
            if (k % 32 != 0 || m->data_len < (size_t)r * row_bytes_of(LQ_FMT_MXFP4, k) ||
                m->scales_len < (size_t)r * (size_t)(k / 32) || !m->scales)
                return fail(ctx, LQ_REFUSED_SHAPE, std::string(name) + ": MXFP4 geometry");
            break;
        case LQ_FMT_NVFP4:
            if (k == 0 || k % 16 != 0 || m->data_len != (size_t)r * row_bytes_of(LQ_FMT_NVFP4, k) ||
                m->scales_len != (size_t)r * (size_t)(k / 16) || !m->scales)
                return fail(ctx, LQ_REFUSED_SHAPE, std::string(name) + ": NVFP4 geometry");
            break;
        default: return fail(ctx, LQ_REFUSED_UNSUPPORTED, std::string(name) + ": unknown format");
    }
    if (r > 0 && k > 0 && !m->data) return fail(ctx, LQ_ERR_ARGUMENT, std::string(name) + ": null data");
    return LQ_OK;
}

// CTAs per token of the batched gather, and the partial-output blocks a batch needs.
int batch_gather_grid(const lq_ctx* ctx, size_t nb) {
    // one CTA per SM in total (the gather kernel fills an SM): a single wave, no tail
    if (nb <= 1) return ctx->gather_grid;
    return std::max(1, ctx->sm_count / (int)nb);
}
size_t partial_blocks(const lq_ctx* ctx, size_t batch) {
    const size_t chunk = std::min<size_t>(batch, 64);
    // (the block-format gather of one token runs fmt_gather_grid() CTAs: several per SM keep more rows in flight)
    return std::max<size_t>((size_t)3 * ctx->gather_grid, chunk * (size_t)batch_gather_grid(ctx, chunk));
}

int ensure_ws(lq_ctx* ctx, size_t batch, size_t hidden, size_t feat) {
    if (batch <= ctx->ws_batch && hidden <= ctx->ws_hidden && feat <= ctx->ws_feat) return LQ_OK;
    cudaStreamCaptureStatus cs;
    CK(cudaStreamIsCapturing(ctx->stream, &cs));
    if (cs != cudaStreamCaptureStatusNone) return fail(ctx, LQ_ERR_ARGUMENT, "workspace growth during capture");
    CK(cudaStreamSynchronize(ctx->stream));
    batch = std::max(batch, ctx->ws_batch);
    hidden = std::max(hidden, ctx->ws_hidden);
    feat = std::max(feat, ctx->ws_feat);
    if (ctx->ws_raw) CK(cudaFree(ctx->ws_raw));
    ctx->ws_raw = nullptr;
    const size_t H = (hidden + 255) / 256 * 256, N = (feat + 31) / 32 * 32;
    const size_t per_tok = a256(H * 4) + 2 * a256(H) + 3 * a256(H / 32 * 4) + a256(N * 4) + a256(LQ_HIST_BINS * 4) + 256 +
                           4 * a256(N * 4);
    ctx->gather_grid = ctx->sm_count;
    const size_t part_bytes = a256(partial_blocks(ctx, batch) * H * 4);
    const size_t total = batch * per_tok + part_bytes;
    CK(cudaMalloc(&ctx->ws_raw, total));
    CK(cudaMemsetAsync(ctx->ws_raw, 0, total, ctx->stream));
    uint8_t* p = ctx->ws_raw;
    auto take = [&](size_t bytes) {
        uint8_t* r = p;
        p += a256(bytes);
        return r;
    };
    ctx->tok.assign(batch, TokenWs{});
    for (size_t t = 0; t < batch; ++t) {
        TokenWs& w = ctx->tok[t];
        w.xn = (float*)take(H * 4);
        w.xa = (uint32_t*)take(H);
        w.xb = (uint32_t*)take(H);
        w.bscale = (float*)take(H / 32 * 4);
        w.bsum = (float*)take(H / 32 * 4);
        w.babs = (float*)take(H / 32 * 4);
        w.scores = (float*)take(N * 4);
        w.hist = (uint32_t*)take(LQ_HIST_BINS * 4);
        w.sel = (SelHeader*)take(256);
        w.hit_idx = (uint32_t*)take(N * 4);
        w.hit_score = (float*)take(N * 4);
        w.band_idx = (uint32_t*)take(N * 4);
        w.band_exact = (float*)take(N * 4);
    }
    ctx->partials = (float*)take(partial_blocks(ctx, batch) * H * 4);
    ctx->ws_batch = batch;
    ctx->ws_hidden = hidden;
    ctx->ws_feat = feat;
    return LQ_OK;
}

int ensure_fused(lq_ctx* ctx, size_t hidden, size_t feat) {
    const size_t need = fused_q4k_ws_bytes((int)hidden, (int)feat, ctx->sm_count);
    if (need <= ctx->fws_cap) return LQ_OK;
    cudaStreamCaptureStatus cs;
    CK(cudaStreamIsCapturing(ctx->stream, &cs));
    if (cs != cudaStreamCaptureStatusNone) return fail(ctx, LQ_ERR_ARGUMENT, "workspace growth during capture");
    CK(cudaStreamSynchronize(ctx->stream));
    if (ctx->fws) CK(cudaFree(ctx->fws));
    ctx->fws = nullptr;
    ctx->fws_cap = 0;
    CK(cudaMalloc(&ctx->fws, need));
    CK(cudaMemsetAsync(ctx->fws, 0, need, ctx->stream));
    ctx->fws_cap = need;

    if (!ctx->stats_dev) {
        CK(cudaMalloc(&ctx->stats_dev, 8192));  // lq_walk_stats, then (at +64) the clock stamps
        CK(cudaMemsetAsync(ctx->stats_dev, 0, 8192, ctx->stream));
    }
    return LQ_OK;
}

bool fused_ok(lq_ctx* ctx, const lq_matrix& gate, const lq_matrix& up, const lq_matrix& down, size_t k) {
    if (!ctx->use_fused) return false;
    if (gate.fmt != LQ_FMT_Q4_K || up.fmt != LQ_FMT_Q4_K || down.fmt != LQ_FMT_Q4_K) return false;
    if ((((uintptr_t)gate.data | (uintptr_t)up.data | (uintptr_t)down.data) & 15) != 0) return false;
    return fused_q4k_supported((int)gate.cols, (int)gate.rows, (int)k, ctx->sm_count);
}

int ensure_stage(lq_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->stage_cap) return LQ_OK;
    CK(cudaStreamSynchronize(ctx->stream));
    if (ctx->stage) CK(cudaFree(ctx->stage));
    ctx->stage = nullptr;
    ctx->stage_cap = 0;
    CK(cudaMalloc(&ctx->stage, a256(bytes)));
    ctx->stage_cap = a256(bytes);
    return LQ_OK;
}

int ensure_sort(lq_ctx* ctx, size_t n) {
    size_t pad = 1;
    while (pad < n) pad <<= 1;
    if (pad <= ctx->sort_cap) return LQ_OK;
    CK(cudaStreamSynchronize(ctx->stream));
    if (ctx->sort_buf) CK(cudaFree(ctx->sort_buf));
    ctx->sort_buf = nullptr;
    CK(cudaMalloc(&ctx->sort_buf, pad * 8));
    ctx->sort_cap = pad;
    return LQ_OK;
}

// Device copy of a host weight range: inside a registered region, else cached on first use
// by (address, length) — the reference GPU backend's buffer-cache rule.
int resolve(lq_ctx* ctx, const void* host, size_t len, const uint8_t** dev) {
    *dev = nullptr;
    if (len == 0) return LQ_OK;
    const uint8_t* h = (const uint8_t*)host;
    // A range at an offset inside a registered region that is not a multiple of 16 bytes would hand the
    // kernels a misaligned device pointer (they use 16-byte vector loads and bulk copies): such a
    // range gets a private, aligned copy, cached by (address, length) like any other range.
    bool inside_unaligned = false;
    for (auto& r : ctx->regions)
        if (h >= r.host && h + len <= r.host + r.len) {
            const uint8_t* cand = r.dev + (h - r.host);
            if (((uintptr_t)cand & 15) == 0) {
                *dev = cand;
                return LQ_OK;
            }
            inside_unaligned = true;
        }
    if (ctx->sealed && !inside_unaligned) return fail(ctx, LQ_ERR_ARGUMENT, "weight range outside the sealed regions");
    uint8_t* d = nullptr;
    CK(cudaMalloc(&d, a256(len) + 256));  // slack: bulk copies may round a ragged tail up to 16 B
    cudaError_t e = cudaMemcpyAsync(d, host, len, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(d);
        return cuda_fail(ctx, e, "weight upload");
    }
    ctx->regions.push_back({h, len, d});
    *dev = d;
    return LQ_OK;
}

int resolve_matrix(lq_ctx* ctx, const lq_matrix* m, lq_matrix* out) {
    *out = *m;
    out->fmt = m->fmt & 0xff;
    if (m->fmt & LQ_MAT_DEVICE) return LQ_OK;  // already device pointers
    const uint8_t* d = nullptr;
    int rc = resolve(ctx, m->data, m->data_len, &d);
    if (rc) return rc;
    out->data = d;
    if (m->scales && m->scales_len) {
        rc = resolve(ctx, m->scales, m->scales_len, &d);
        if (rc) return rc;
        out->scales = d;
    }
    return LQ_OK;
}

// CTAs of the block-format gather of one token: its CTAs are light (80 registers, 512 bytes of shared memory),
// and what bounds it is how many scattered rows are in flight, so an SM takes several.
int fmt_gather_grid(const lq_ctx* ctx) {
    static const int mult = [] { const char* e = getenv("LARQL_B200_FMT_GATHER_CTAS"); const int v = e ? atoi(e) : 2; return v < 1 ? 1 : (v > 3 ? 3 : v); }();
    return mult * ctx->gather_grid;
}

int check_device_err(lq_ctx* ctx) {
    int h = 0;
    CK(cudaMemcpyAsync(&h, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaStreamSynchronize(ctx->stream));
    if (h == DEV_OK) return LQ_OK;
    CK(cudaMemsetAsync(ctx->d_err, 0, sizeof(int), ctx->stream));
    // a failed fused launch may leave its histogram / counters dirty
    if (ctx->fws) CK(cudaMemsetAsync(ctx->fws, 0, fused_q4k_ws_dirty_bytes(), ctx->stream));
    if (h == DEV_ERR_NAN_SCORE) return fail(ctx, LQ_ERR_NAN_SCORE, "NaN gate score or non-finite activation");
    if (h == DEV_ERR_TMA_TIMEOUT) return fail(ctx, LQ_ERR_TIMEOUT, "a bounded device-side wait ran out");
    return fail(ctx, LQ_ERR_CUDA, "device-side internal error");
}

XPrep xprep_of(const TokenWs& w) { return XPrep{w.xn, w.xa, w.xb, w.bscale, w.bsum, w.babs}; }

// Rounding-count constant of the score error bound: the reference's sum_x-form row has at
// most 43 + nsb roundings on any term's path (product, 32-term chain, scale multiply,
// subtract, 8 group adds, nsb super-block adds) and the fast path at most 64.
float bound_c1(int hidden) {
    const double u = std::ldexp(1.0, -24);
    const double n = 43.0 + hidden / 256 + 64.0;
    return (float)(n * u / (1.0 - n * u) * 1.01);
}

// Reference rows of Q8_0 / MXFP4 / NVFP4 are one f32 chain over the whole row: hidden + 3 roundings on a term's
// path; the fast path has at most 64.  The 2 % margin also covers the rounding of the sum |w x| the bound is
// taken from.
float bound_c1_fmt(int hidden) {
    const double u = std::ldexp(1.0, -24);
    const double n = (double)hidden + 3.0 + 64.0;
    return (float)(n * u / (1.0 - n * u) * 1.02);
}

FmtMat fmtmat_of(const lq_matrix& m) {
    return FmtMat{m.fmt & 0xff, (const uint8_t*)m.data, (const uint8_t*)m.scales, m.tensor_scale, (int)m.rows,
                  (int)m.cols};
}

// The format kernels load whole blocks with vector loads: 2 / 16 / 8 byte alignment of the base.
bool fmt_aligned(const lq_matrix& m) {
    const uintptr_t a = (uintptr_t)m.data;
    switch (m.fmt & 0xff) {
        case LQ_FMT_Q8_0: return (a & 1) == 0;
        case LQ_FMT_Q6_K: return (a & 1) == 0;
        case LQ_FMT_Q4_K: return (a & 15) == 0;
        case LQ_FMT_MXFP4: return (a & 15) == 0;
        case LQ_FMT_NVFP4: return (a & 7) == 0;
    }
    return true;
}

__global__ void scaled_add_kernel(float* __restrict__ out, const float* __restrict__ src, const float* __restrict__ w,
                                  int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fmaf(*w, src[i], out[i]);
}

// Walk of one prepared token for Q8_0 / MXFP4 / NVFP4 (separate kernels).
int enqueue_walk_token_fmt(lq_ctx* ctx, const lq_matrix& gate, const lq_matrix& up, const lq_matrix& down, size_t t,
                           int k, const float* residual, float* out) {
    if (!fmt_aligned(gate) || !fmt_aligned(up) || !fmt_aligned(down))
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "walk: weight base address not block aligned");
    TokenWs& w = ctx->tok[t];
    const int N = (int)gate.rows, H = (int)gate.cols;
    const FmtMat g = fmtmat_of(gate), u = fmtmat_of(up), d = fmtmat_of(down);
    const XPrep xp = xprep_of(w);
    const bool sparse = k < N;
    cudaStream_t st = ctx->stream;
    // The reference rows of these formats are one running f32 sum over the whole row, so the rounding part of a
    // rigorous bound on a re-associated fast score grows with the row length: even with sum |w x| accumulated per
    // row beside the dot, the band at 28672 x 8192 costs more to re-score in the reference's order than scanning
    // every row in that order from the start (measured on B200: 631 against 371 us per NVFP4 layer).  The scan
    // therefore runs in the reference's order and the selection works on exact scores: no bound, no band.
    // LARQL_B200_FMT_FAST_SCAN=1 selects fast scan + band for the FP4 formats.
    static const bool fast_scan = [] { const char* e = getenv("LARQL_B200_FMT_FAST_SCAN"); return e && e[0] == '1'; }();
    const bool force_exact = !fast_scan;
    if (sparse && !force_exact && (g.fmt == LQ_FMT_MXFP4 || g.fmt == LQ_FMT_NVFP4)) {
        CK(launch_scan_fmt(g, xp, w.scores, w.hist, &w.sel->bound_bits, bound_c1_fmt(H), ctx->d_err, ctx->sm_count, st));
        CK(launch_classify(w.scores, N, k, w, ctx->d_err, st));
        CK(launch_rescore_fmt(g, w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, ctx->sm_count, st));
        CK(launch_final_pick(w, ctx->d_err, st));
        CK(launch_gather_fmt(u, d, xp, w.hit_idx, w.hit_score, &w.sel->n_sel, k, ctx->partials, fmt_gather_grid(ctx), st));
        CK(launch_finish(ctx->partials, fmt_gather_grid(ctx), H, residual, out, st));
        ctx->launches += 6;
        return LQ_OK;
    }
    CK(launch_scan_exact_fmt(g, w.xn, w.scores, ctx->d_err, st));
    static const bool mc_on = [] { const char* e = getenv("LARQL_B200_SELECT_MC"); return !(e && e[0] == '0'); }();
    if (sparse && mc_on && N >= 8192 && k > 0) {
        // many rows: histogram of the exact scores, the threshold bucket's rows as the band (their scores are
        // exact already), the rest by several CTAs in row order; the final pick settles the bucket
        CK(launch_hist_abs(w.scores, N, w.hist, st));
        CK(launch_classify_mc(w.scores, N, k, w, st, 1, 0, 1));
        CK(launch_final_pick(w, ctx->d_err, st));
        ctx->launches += 5;
    } else {
        CK(launch_select(w.scores, N, k, w, ctx->d_err, st));
        ctx->launches += 2;
        if (sparse) {
            CK(launch_final_pick(w, ctx->d_err, st));  // ties at the K-th |score|: the lower rows win
            ctx->launches += 1;
        }
    }
    CK(launch_gather_fmt(u, d, xp, w.hit_idx, w.hit_score, &w.sel->n_sel, k, ctx->partials, fmt_gather_grid(ctx), st));
    CK(launch_finish(ctx->partials, fmt_gather_grid(ctx), H, residual, out, st));
    ctx->launches += 3;
    return LQ_OK;
}

// Enqueue the walk of one prepared token.
int enqueue_walk_token(lq_ctx* ctx, const lq_matrix& gate, const lq_matrix& up, const lq_matrix& down, size_t t,
                       size_t top_k, const float* residual, float* out) {
    auto kquant = [](int f) { return f == LQ_FMT_Q4_K || f == LQ_FMT_Q6_K; };
    const bool mixed_kq = kquant(gate.fmt) && kquant(up.fmt) && kquant(down.fmt) &&
                          !(gate.fmt == LQ_FMT_Q4_K && up.fmt == LQ_FMT_Q4_K && down.fmt == LQ_FMT_Q4_K);
    if (!mixed_kq && (gate.fmt != up.fmt || gate.fmt != down.fmt))
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "walk: gate/up/down formats differ (only Q4_K and Q6_K mix)");
    TokenWs& w = ctx->tok[t];
    const int N = (int)gate.rows, H = (int)gate.cols;
    if (mixed_kq) {
        // Q4_K / Q6_K in any mix: the gate by its own format's scan, the rows by the K-quant gather
        if (H % 256 != 0) return fail(ctx, LQ_REFUSED_SHAPE, "walk: K-quant rows need hidden % 256 == 0");
        if (!fmt_aligned(gate) || !fmt_aligned(up) || !fmt_aligned(down))
            return fail(ctx, LQ_ERR_ARGUMENT, "walk: weight base address not block aligned");
        const int k = (int)std::min<size_t>(top_k, (size_t)N);
        cudaStream_t st = ctx->stream;
        if (k == 0) {
            CK(cudaMemsetAsync(w.sel, 0, sizeof(SelHeader), st));
            if (residual) CK(cudaMemcpyAsync(out, residual, (size_t)H * 4, cudaMemcpyDeviceToDevice, st));
            else CK(cudaMemsetAsync(out, 0, (size_t)H * 4, st));
            return LQ_OK;
        }
        const bool sparse = k < N;
        if (gate.fmt == LQ_FMT_Q4_K) {
            const Q4kMat g{(const uint8_t*)gate.data, N, H};
            CK(launch_scan_q4k(g, xprep_of(w), w.scores, sparse ? w.hist : nullptr, &w.sel->bound_bits, bound_c1(H),
                               ctx->d_err, ctx->sm_count, st));
            if (sparse) {
                CK(launch_classify(w.scores, N, k, w, ctx->d_err, st));
                CK(launch_rescore_q4k(g, w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, w, k, 1, ctx->d_err,
                                      ctx->sm_count, st));
                ctx->launches += 1;
            } else
                CK(launch_select(w.scores, N, k, w, ctx->d_err, st));
            ctx->launches += 2;
        } else {
            // the Q6_K matvec kernel runs in the reference's order: its scores are the reference's scores
            CK(launch_q6k_matvec((const uint8_t*)gate.data, w.xn, nullptr, nullptr, N, H, w.scores, ctx->d_err,
                                 ctx->sm_count, st));
            CK(launch_select(w.scores, N, k, w, ctx->d_err, st));
            ctx->launches += 2;
            if (sparse) {
                CK(launch_final_pick(w, ctx->d_err, st));
                ctx->launches += 1;
            }
        }
        CK(launch_gather_kquant(up.fmt, (const uint8_t*)up.data, down.fmt, (const uint8_t*)down.data, w.xn, H, w.hit_idx,
                                w.hit_score, &w.sel->n_sel, k, ctx->partials, ctx->gather_grid, st));
        CK(launch_finish(ctx->partials, ctx->gather_grid, H, residual, out, st));
        ctx->launches += 2;
        return LQ_OK;
    }
    if (gate.fmt != LQ_FMT_Q4_K) {
        const int kk = (int)std::min<size_t>(top_k, (size_t)N);
        if (kk == 0) {
            CK(cudaMemsetAsync(w.sel, 0, sizeof(SelHeader), ctx->stream));
            if (residual) CK(cudaMemcpyAsync(out, residual, (size_t)H * 4, cudaMemcpyDeviceToDevice, ctx->stream));
            else CK(cudaMemsetAsync(out, 0, (size_t)H * 4, ctx->stream));
            return LQ_OK;
        }
        return enqueue_walk_token_fmt(ctx, gate, up, down, t, kk, residual, out);
    }
    const Q4kMat g{(const uint8_t*)gate.data, N, H}, u{(const uint8_t*)up.data, N, H},
        d{(const uint8_t*)down.data, N, H};
    const XPrep xp = xprep_of(w);
    const int k = (int)std::min<size_t>(top_k, (size_t)N);
    if (k == 0) {  // empty selection: zero contribution
        CK(cudaMemsetAsync(w.sel, 0, sizeof(SelHeader), ctx->stream));
        if (residual) CK(cudaMemcpyAsync(out, residual, (size_t)H * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        else CK(cudaMemsetAsync(out, 0, (size_t)H * 4, ctx->stream));
        return LQ_OK;
    }
    const bool sparse = k < N;
    CK(launch_scan_q4k(g, xp, w.scores, sparse ? w.hist : nullptr, &w.sel->bound_bits, bound_c1(H), ctx->d_err,
                       ctx->sm_count, ctx->stream));
    if (sparse) CK(launch_classify(w.scores, N, k, w, ctx->d_err, ctx->stream));
    else CK(launch_select(w.scores, N, k, w, ctx->d_err, ctx->stream));
    ctx->launches += 2;
    if (sparse) {
        CK(launch_rescore_q4k(g, w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, w, k, 1, ctx->d_err,
                              ctx->sm_count, ctx->stream));
        ctx->launches += 1;
    }
    CK(launch_gather_q4k(u, d, xp, w.hit_idx, w.hit_score, &w.sel->n_sel, k, ctx->partials, ctx->gather_grid,
                         ctx->d_err, ctx->stream));
    CK(launch_finish(ctx->partials, ctx->gather_grid, H, residual, out, ctx->stream));
    ctx->launches += 2;
    return LQ_OK;
}

// Fast scores (+ histogram and bound) of every row for nb <= 64 tokens: the tcgen05 scan, 32 tokens per launch,
// or the mma.sync scan.  Never called inside a capture for the first time (the scratch is allocated here).
int batched_scan(lq_ctx* ctx, const Q4kMat& g, const TokenWs& w, size_t ws_stride, int nb, int want_hist, float c1) {
    if (!ctx->use_tc_scan) {
        CK(launch_scan_q4k_mma(g, w, ws_stride, nb, want_hist, c1, ctx->d_err, ctx->sm_count, ctx->stream));
        ctx->launches += 1;
        return LQ_OK;
    }
    const size_t need = scan_q4k_tc_scratch_bytes(g.cols);
    if (need > ctx->tc_scratch_cap) {
        CK(cudaStreamSynchronize(ctx->stream));
        if (ctx->tc_scratch) cudaFree(ctx->tc_scratch);
        ctx->tc_scratch = nullptr;
        ctx->tc_scratch_cap = 0;
        CK(cudaMalloc(&ctx->tc_scratch, need));
        ctx->tc_scratch_cap = need;
    }
    for (int o = 0; o < nb; o += 32) {
        // one scratch for all launches: they run one after the other on the stream
        CK(launch_scan_q4k_tc(g, ws_at(w, ws_stride * (size_t)o), ws_stride, std::min(32, nb - o), want_hist, c1,
                              ctx->tc_scratch, ctx->d_err, ctx->stream));
        ctx->launches += 2;  // the token planes, the scan
    }
    return LQ_OK;
}

size_t effective_k(size_t top_k, size_t n, uint32_t flags) {
    // K >= 80% of the features runs dense (all features) unless the walk is forced
    // (crates/larql-inference/src/vindex/walk_ffn/helpers.rs:18-30, thresholds.rs:29-31).
    if (!(flags & LQ_WALK_FORCE_SPARSE) && top_k >= (n * 4) / 5) return n;
    return std::min(top_k, n);
}

int dev_walk(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down, const float* x,
             size_t batch, size_t top_k, uint32_t flags, float* out, uint32_t* idx_out, uint32_t* count_out) {
    const size_t N = (size_t)gate->rows, H = (size_t)gate->cols;
    if (up->rows != gate->rows || down->rows != gate->rows || up->cols != gate->cols || down->cols != gate->cols)
        return fail(ctx, LQ_REFUSED_SHAPE, "walk: gate/up/down shapes differ");
    if (batch == 0 || H == 0) return LQ_OK;
    if (H > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "walk: hidden > 16384");
    if (H % 32 != 0) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "walk: hidden not a multiple of 32");
    // every Q4_K kernel moves rows with 16-byte vector loads and bulk copies
    for (const lq_matrix* m : {gate, up, down})
        if ((m->fmt & 0xff) == LQ_FMT_Q4_K && N > 0 && ((uintptr_t)m->data & 15) != 0)
            return fail(ctx, LQ_ERR_ARGUMENT, "walk: Q4_K weights not 16-byte aligned");
    int rc = ensure_ws(ctx, batch, H, N);
    if (rc) return rc;
    const size_t k = effective_k(top_k, N, flags);
    if (N > 0 && batch < ctx->batch_min && fused_ok(ctx, *gate, *up, *down, k)) {
        rc = ensure_fused(ctx, H, N);
        if (rc) return rc;
        const uint8_t* single[3] = {(const uint8_t*)gate->data, (const uint8_t*)up->data, (const uint8_t*)down->data};
        for (size_t t = 0; t < batch; ++t) {
            CK(launch_walk_fused_q4k(nullptr, single, 1, (int)N, (int)H, (int)k, flags, bound_c1((int)H), x + t * H,
                                     out + t * H, ctx->fws, idx_out ? idx_out + t * k : nullptr,
                                     count_out ? count_out + t : nullptr, t == 0 ? ctx->stats_dev : nullptr,
                                     ctx->d_err, ctx->sm_count, ctx->stream));
            ctx->launches += 1;
        }
        ctx->last_fused = true;
        return LQ_OK;
    }
    ctx->last_fused = false;
    TokenWs& w0 = ctx->tok[0];
    // Token workspaces are laid out with a constant byte stride; prep takes it in 4-byte words.
    const size_t tok_stride_f =
        batch > 1 ? (size_t)((uint8_t*)ctx->tok[1].xn - (uint8_t*)ctx->tok[0].xn) / sizeof(float) : 0;
    launch_prep(x, (int)batch, (int)H, (flags & LQ_WALK_RMSNORM) ? 1 : 0, 1e-6, w0.xn, w0.xa, w0.xb, w0.bscale,
                w0.bsum, w0.babs, tok_stride_f, ctx->d_err, ctx->stream);
    CK(cudaGetLastError());
    ctx->launches += 1;
    // Batches of Q4_K tokens: one tensor-core scan and one launch of each selection / gather kernel
    // for up to 64 tokens at a time (the gate matrix is read once per chunk instead of once per token).
    if (batch >= ctx->batch_min && N > 0 && k < N && k > 0 && gate->fmt == LQ_FMT_Q4_K && up->fmt == LQ_FMT_Q4_K &&
        down->fmt == LQ_FMT_Q4_K) {
        const Q4kMat g{(const uint8_t*)gate->data, (int)N, (int)H}, u{(const uint8_t*)up->data, (int)N, (int)H},
            d{(const uint8_t*)down->data, (int)N, (int)H};
        const size_t ws_stride = (size_t)((uint8_t*)ctx->tok[1].xn - (uint8_t*)ctx->tok[0].xn);
        for (size_t c0 = 0; c0 < batch; c0 += 64) {
            const int nb = (int)std::min<size_t>(64, batch - c0);
            const TokenWs& w = ctx->tok[c0];
            const int gb = batch_gather_grid(ctx, (size_t)nb);
            const TokStride ts{ws_stride, H, (size_t)gb * H};
            if ((rc = batched_scan(ctx, g, w, ws_stride, nb, 1, bound_c1((int)H)))) return rc;
            CK(launch_classify(w.scores, (int)N, (int)k, w, ctx->d_err, ctx->stream, nb, ws_stride));
            CK(launch_rescore_q4k(g, w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, w, (int)k, 1, ctx->d_err,
                                  ctx->sm_count, ctx->stream, nb, ws_stride));
            CK(launch_gather_q4k(u, d, xprep_of(w), w.hit_idx, w.hit_score, &w.sel->n_sel, (int)k, ctx->partials, gb,
                                 ctx->d_err, ctx->stream, nb, ts));
            CK(launch_finish(ctx->partials, gb, (int)H, (flags & LQ_WALK_RESIDUAL) ? x + c0 * H : nullptr, out + c0 * H,
                             ctx->stream, nb, ts));
            ctx->launches += 4;
            if (idx_out)
                CK(cudaMemcpy2DAsync(idx_out + c0 * k, k * 4, w.hit_idx, ws_stride, k * 4, (size_t)nb,
                                     cudaMemcpyDeviceToDevice, ctx->stream));
            if (count_out)
                CK(cudaMemcpy2DAsync(count_out + c0, 4, &w.sel->n_sel, ws_stride, 4, (size_t)nb, cudaMemcpyDeviceToDevice,
                                     ctx->stream));
        }
        return LQ_OK;
    }
    for (size_t t = 0; t < batch; ++t) {
        if (N == 0) {
            if (flags & LQ_WALK_RESIDUAL)
                CK(cudaMemcpyAsync(out + t * H, x + t * H, H * 4, cudaMemcpyDeviceToDevice, ctx->stream));
            else
                CK(cudaMemsetAsync(out + t * H, 0, H * 4, ctx->stream));
            continue;
        }
        rc = enqueue_walk_token(ctx, *gate, *up, *down, t, k, (flags & LQ_WALK_RESIDUAL) ? x + t * H : nullptr,
                                out + t * H);
        if (rc) return rc;
        if (idx_out)
            CK(cudaMemcpyAsync(idx_out + t * k, ctx->tok[t].hit_idx, k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        if (count_out)
            CK(cudaMemcpyAsync(count_out + t, &ctx->tok[t].sel->n_sel, 4, cudaMemcpyDeviceToDevice, ctx->stream));
    }
    return LQ_OK;
}

}  // namespace

// ------------------------------------------------------------------ context ----
extern "C" {

int lq_create(int device, lq_ctx** out) {
    if (!out) return LQ_ERR_ARGUMENT;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device < 0 || device >= n) return LQ_ERR_CUDA;
    if (cudaSetDevice(device) != cudaSuccess) return LQ_ERR_CUDA;
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return LQ_ERR_CUDA;
    if (p.major < 10) return LQ_REFUSED_UNSUPPORTED;  // kernels are built for sm_100a only
    lq_ctx* ctx = new lq_ctx();
    ctx->device = device;
    ctx->sm_count = p.multiProcessorCount;
    char buf[512];
    snprintf(buf, sizeof buf, "cuda:%d %s sm_%d%d %d SMs %.0f GB", device, p.name, p.major, p.minor,
             p.multiProcessorCount, (double)p.totalGlobalMem / 1e9);
    ctx->info = buf;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&ctx->d_err, 256) != cudaSuccess || cudaMemset(ctx->d_err, 0, 256) != cudaSuccess) {
        delete ctx;
        return LQ_ERR_CUDA;
    }
    if (const char* e = getenv("LARQL_B200_NO_FUSED")) ctx->use_fused = !(e[0] && e[0] != '0');
    if (const char* e = getenv("LARQL_B200_BATCH_SCAN")) ctx->use_tc_scan = strcmp(e, "mma") != 0;
    if (const char* e = getenv("LARQL_B200_BATCH_MIN")) ctx->batch_min = (size_t)std::max(2, atoi(e));
    *out = ctx;
    return LQ_OK;
}

void lq_destroy(lq_ctx* ctx) {
    DevGuard dev_guard(ctx);
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->comm) {
        if (NcclApi* nc = nccl_api()) nc->CommDestroy(ctx->comm);
        ctx->comm = nullptr;
    }
    for (auto& r : ctx->regions) cudaFree(r.dev);
    cudaFree(ctx->ws_raw);
    cudaFree(ctx->fws);
    cudaFree(ctx->stats_dev);
    cudaFree(ctx->tc_scratch);
    cudaFree(ctx->stage);
    cudaFree(ctx->sort_buf);
    cudaFree(ctx->d_err);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char* lq_last_error(lq_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int lq_device_info(lq_ctx* ctx, char* buf, size_t cap) {
    DevGuard dev_guard(ctx);
    if (!ctx || !buf || cap == 0) return LQ_ERR_ARGUMENT;
    snprintf(buf, cap, "%s", ctx->info.c_str());
    return LQ_OK;
}

int lq_supports_quant(lq_ctx* ctx, int fmt) {
    DevGuard dev_guard(ctx);
    (void)ctx;
    return (fmt == LQ_FMT_Q4_K || fmt == LQ_FMT_Q8_0 || fmt == LQ_FMT_MXFP4 || fmt == LQ_FMT_NVFP4) ? 1 : 0;
}

int lq_synchronize(lq_ctx* ctx) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    CK(cudaStreamSynchronize(ctx->stream));
    return check_device_err(ctx);
}

void* lq_stream(lq_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
uint64_t lq_launch_count(lq_ctx* ctx) { return ctx ? ctx->launches : 0; }

int lq_register_weight_region(lq_ctx* ctx, const void* host, size_t len) {
    DevGuard dev_guard(ctx);
    if (!ctx || (!host && len)) return LQ_ERR_ARGUMENT;
    if (ctx->sealed) return fail(ctx, LQ_ERR_ARGUMENT, "regions are sealed");
    const uint8_t* d;
    return resolve(ctx, host, len, &d);
}
int lq_seal_weight_regions(lq_ctx* ctx) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    ctx->sealed = true;
    return LQ_OK;
}
int lq_drop_weight_regions(lq_ctx* ctx) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    CK(cudaStreamSynchronize(ctx->stream));
    for (auto& r : ctx->regions) cudaFree(r.dev);
    ctx->regions.clear();
    ctx->sealed = false;
    return LQ_OK;
}
const void* lq_device_ptr(lq_ctx* ctx, const void* host, size_t len) {
    DevGuard dev_guard(ctx);
    if (!ctx) return nullptr;
    const uint8_t* h = (const uint8_t*)host;
    for (auto& r : ctx->regions)
        if (h >= r.host && h + len <= r.host + r.len) return r.dev + (h - r.host);
    return nullptr;
}

// ------------------------------------------------------------ matvec / matmul ----
int lq_dev_q4k_matvec(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t num_rows, size_t hidden,
                      float* out) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    if (hidden % 256 != 0 || w_len < num_rows * (hidden / 256) * 144)
        return fail(ctx, LQ_REFUSED_SHAPE, "q4k_matvec: geometry");
    if (num_rows == 0) return LQ_OK;
    if (hidden == 0) {
        CK(cudaMemsetAsync(out, 0, num_rows * 4, ctx->stream));
        return LQ_OK;
    }
    if (hidden > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "q4k_matvec: hidden > 16384");
    if (((uintptr_t)w & 15) != 0) return fail(ctx, LQ_ERR_ARGUMENT, "q4k_matvec: weights not 16-byte aligned");
    int rc = ensure_ws(ctx, 1, hidden, 32);
    if (rc) return rc;
    TokenWs& t = ctx->tok[0];
    launch_prep(x, 1, (int)hidden, 0, 0.0, t.xn, t.xa, t.xb, t.bscale, t.bsum, t.babs, 0, nullptr, ctx->stream);
    CK(cudaGetLastError());
    const Q4kMat m{w, (int)num_rows, (int)hidden};
    CK(launch_scan_q4k(m, xprep_of(t), out, nullptr, nullptr, 0.0f, ctx->d_err, ctx->sm_count, ctx->stream));
    ctx->launches += 2;
    return LQ_OK;
}

static int q4k_host_common(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                           size_t num_rows, size_t hidden, size_t seq, float* out, size_t out_len, int exact) {
    if (!ctx) return LQ_ERR_ARGUMENT;
    const size_t needed = (hidden / 256) * 144 * num_rows;
    if (!(out_len == num_rows * seq && x_len == hidden * seq && hidden % 256 == 0 && w_len >= needed))
        return fail(ctx, LQ_REFUSED_SHAPE, "q4k matvec/matmul: shape (KernelShapeError)");
    if (num_rows == 0 || seq == 0) return LQ_OK;
    if (hidden == 0) {
        memset(out, 0, out_len * 4);
        return LQ_OK;
    }
    if (hidden > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "q4k: hidden > 16384");
    const uint8_t* dw;
    int rc = resolve(ctx, w, needed, &dw);
    if (rc) return rc;
    rc = ensure_stage(ctx, (x_len + out_len) * 4 + 512);
    if (rc) return rc;
    float* dx = (float*)ctx->stage;
    float* dout = (float*)(ctx->stage + a256(x_len * 4));
    CK(cudaMemcpyAsync(dx, x, x_len * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (!exact && seq >= 2 && ((uintptr_t)dw & 15) == 0) {
        // q4k_matmul: the integer-MMA scan, up to 64 positions per launch
        rc = ensure_ws(ctx, std::min<size_t>(seq, 64), hidden, num_rows);
        if (rc) return rc;
        const Q4kMat m{dw, (int)num_rows, (int)hidden};
        const size_t tstride = ctx->tok.size() > 1 ? (size_t)((uint8_t*)ctx->tok[1].xn - (uint8_t*)ctx->tok[0].xn) : 0;
        for (size_t c0 = 0; c0 < seq; c0 += 64) {
            const size_t nb = std::min<size_t>(64, seq - c0);
            TokenWs& t0 = ctx->tok[0];
            launch_prep(dx + c0 * hidden, (int)nb, (int)hidden, 0, 0.0, t0.xn, t0.xa, t0.xb, t0.bscale, t0.bsum, t0.babs,
                        tstride / sizeof(float), nullptr, ctx->stream);
            CK(cudaGetLastError());
            if ((rc = batched_scan(ctx, m, t0, tstride, (int)nb, 0, 0.0f))) return rc;
            CK(cudaMemcpy2DAsync(dout + c0 * num_rows, num_rows * 4, t0.scores, tstride ? tstride : num_rows * 4,
                                 num_rows * 4, nb, cudaMemcpyDeviceToDevice, ctx->stream));
            ctx->launches += 1;
        }
        CK(cudaMemcpyAsync(out, dout, out_len * 4, cudaMemcpyDeviceToHost, ctx->stream));
        return lq_synchronize(ctx);
    }
    for (size_t s = 0; s < seq; ++s) {
        if (exact) {
            rc = ensure_ws(ctx, 1, hidden, 32);
            if (rc) return rc;
            const Q4kMat m{dw, (int)num_rows, (int)hidden};
            CK(launch_rescore_q4k(m, dx + s * hidden, nullptr, nullptr, (int)num_rows, dout + s * num_rows,
                                  ctx->tok[0], 0, 0, ctx->d_err, ctx->sm_count, ctx->stream));
            ctx->launches += 1;
        } else {
            rc = lq_dev_q4k_matvec(ctx, dw, needed, dx + s * hidden, num_rows, hidden, dout + s * num_rows);
            if (rc) return rc;
        }
    }
    CK(cudaMemcpyAsync(out, dout, out_len * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_q4k_matvec(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                  size_t hidden, float* out, size_t out_len) {
    DevGuard dev_guard(ctx);
    return q4k_host_common(ctx, w, w_len, x, x_len, num_rows, hidden, 1, out, out_len, 0);
}
int lq_q4k_matvec_exact(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                        size_t hidden, float* out, size_t out_len) {
    DevGuard dev_guard(ctx);
    return q4k_host_common(ctx, w, w_len, x, x_len, num_rows, hidden, 1, out, out_len, 1);
}
int lq_q4k_matmul(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                  size_t hidden, size_t seq_len, float* out, size_t out_len) {
    DevGuard dev_guard(ctx);
    return q4k_host_common(ctx, w, w_len, x, x_len, num_rows, hidden, seq_len, out, out_len, 0);
}

// Dense gemv of one block-format matrix (host pointers): fast path, or the reference's exact order.
int lq_gemv(lq_ctx* ctx, const lq_matrix* m, const float* x, size_t x_len, float* out, size_t out_len, int exact) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    int rc = check_matrix(ctx, m, "gemv");
    if (rc) return rc;
    const int fmt = m->fmt & 0xff;
    const size_t n = (size_t)m->rows, k = (size_t)m->cols;
    if (fmt == LQ_FMT_Q4_K)
        return q4k_host_common(ctx, (const uint8_t*)m->data, m->data_len, x, x_len, n, k, 1, out, out_len, exact);
    if (fmt == LQ_FMT_Q6_K) {
        if (out_len != n) return fail(ctx, LQ_REFUSED_SHAPE, "gemv: out_len != n");
        if (m->fmt & LQ_MAT_DEVICE) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv: Q6_K takes host weights here");
        return lq_q6k_matvec(ctx, (const uint8_t*)m->data, m->data_len, x, x_len, n, k, out);
    }
    if (x_len != k || out_len != n) return fail(ctx, LQ_REFUSED_SHAPE, "gemv: x_len != k or out_len != n");
    if (n == 0) return LQ_OK;
    if (k % 32 != 0 || k > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv: k must be a multiple of 32, <= 16384");
    lq_matrix dm;
    rc = resolve_matrix(ctx, m, &dm);
    if (rc) return rc;
    if (!fmt_aligned(dm)) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv: weight base address not block aligned");
    rc = ensure_ws(ctx, 1, k, 32);
    if (rc) return rc;
    rc = ensure_stage(ctx, (k + n) * 4 + 512);
    if (rc) return rc;
    float* dx = (float*)ctx->stage;
    float* dout = (float*)(ctx->stage + a256(k * 4));
    TokenWs& t = ctx->tok[0];
    CK(cudaMemcpyAsync(dx, x, k * 4, cudaMemcpyHostToDevice, ctx->stream));
    const FmtMat fm = fmtmat_of(dm);
    if (exact) {
        CK(launch_rescore_fmt(fm, dx, nullptr, nullptr, (int)n, dout, ctx->sm_count, ctx->stream));
        ctx->launches += 1;
    } else {
        launch_prep(dx, 1, (int)k, 0, 0.0, t.xn, t.xa, t.xb, t.bscale, t.bsum, t.babs, 0, nullptr, ctx->stream);
        CK(cudaGetLastError());
        CK(launch_scan_fmt(fm, xprep_of(t), dout, nullptr, nullptr, 0.0f, ctx->d_err, ctx->sm_count, ctx->stream));
        ctx->launches += 2;
    }
    CK(cudaMemcpyAsync(out, dout, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_q6k_matvec(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                  size_t hidden, float* out) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    // KernelShapeError-style refusal: the caller falls back to its CPU path
    if (hidden % 256 != 0 || x_len != hidden || w_len < num_rows * (hidden / 256) * 210)
        return fail(ctx, LQ_REFUSED_SHAPE, "q6k_matvec: shape");
    if (num_rows == 0 || hidden == 0) return LQ_OK;
    if (hidden > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "q6k_matvec: hidden > 16384");
    if (!w || !x || !out) return LQ_ERR_ARGUMENT;
    const lq_matrix hm{LQ_FMT_Q6_K, w, w_len, nullptr, 0, 1.0f, (int64_t)num_rows, (int64_t)hidden};
    lq_matrix dm;
    int rc = resolve_matrix(ctx, &hm, &dm);
    if (rc) return rc;
    if (!fmt_aligned(dm)) return fail(ctx, LQ_ERR_ARGUMENT, "q6k_matvec: weights not 2-byte aligned");
    rc = ensure_stage(ctx, (hidden + num_rows) * 4 + 512);
    if (rc) return rc;
    float* dx = (float*)ctx->stage;
    float* dout = (float*)(ctx->stage + a256(hidden * 4));
    CK(cudaMemcpyAsync(dx, x, hidden * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(launch_q6k_matvec((const uint8_t*)dm.data, dx, nullptr, nullptr, (int)num_rows, (int)hidden, dout, nullptr,
                         ctx->sm_count, ctx->stream));
    ctx->launches += 1;
    CK(cudaMemcpyAsync(out, dout, num_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_dequantize_q6k(lq_ctx* ctx, const uint8_t* data, size_t data_len, size_t n_elems, float* out) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    if (n_elems % 256 != 0 || data_len < n_elems / 256 * 210) return fail(ctx, LQ_REFUSED_SHAPE, "dequantize_q6k: shape");
    if (n_elems == 0) return LQ_OK;
    if (!data || !out) return LQ_ERR_ARGUMENT;
    const size_t bytes = n_elems / 256 * 210;
    int rc = ensure_stage(ctx, a256(bytes) + n_elems * 4 + 512);
    if (rc) return rc;
    uint8_t* dsrc = ctx->stage;
    float* dout = (float*)(ctx->stage + a256(bytes));
    CK(cudaMemcpyAsync(dsrc, data, bytes, cudaMemcpyHostToDevice, ctx->stream));
    CK(launch_q6k_dequant(dsrc, n_elems, dout, ctx->stream));
    ctx->launches += 1;
    CK(cudaMemcpyAsync(out, dout, n_elems * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_q4k_dual_matvec(lq_ctx* ctx, const uint8_t* w_a, size_t wa_len, const uint8_t* w_b, size_t wb_len, const float* x,
                       size_t x_len, size_t num_rows, size_t hidden, float* out_a, float* out_b) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    const size_t need = num_rows * (hidden / 256) * 144;
    if (hidden % 256 != 0 || x_len != hidden || wa_len < need || wb_len < need)
        return fail(ctx, LQ_REFUSED_SHAPE, "q4k_dual_matvec: shape");
    if (!out_a || !out_b) return LQ_ERR_ARGUMENT;
    if (num_rows == 0 || hidden == 0) {  // dual.rs:54-58
        for (size_t i = 0; i < num_rows; ++i) out_a[i] = out_b[i] = 0.0f;
        return LQ_OK;
    }
    if (hidden > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "q4k_dual_matvec: hidden > 16384");
    if (!w_a || !w_b || !x) return LQ_ERR_ARGUMENT;
    const lq_matrix ha{LQ_FMT_Q4_K, w_a, wa_len, nullptr, 0, 1.0f, (int64_t)num_rows, (int64_t)hidden};
    const lq_matrix hb{LQ_FMT_Q4_K, w_b, wb_len, nullptr, 0, 1.0f, (int64_t)num_rows, (int64_t)hidden};
    lq_matrix da, db;
    int rc;
    if ((rc = resolve_matrix(ctx, &ha, &da)) || (rc = resolve_matrix(ctx, &hb, &db))) return rc;
    if ((((uintptr_t)da.data | (uintptr_t)db.data) & 15) != 0)
        return fail(ctx, LQ_ERR_ARGUMENT, "q4k_dual_matvec: weights not 16-byte aligned");
    rc = ensure_stage(ctx, a256(hidden * 4) + 2 * a256(num_rows * 4) + 512);
    if (rc) return rc;
    float* dx = (float*)ctx->stage;
    float* doa = (float*)(ctx->stage + a256(hidden * 4));
    float* dob = (float*)((uint8_t*)doa + a256(num_rows * 4));
    CK(cudaMemcpyAsync(dx, x, hidden * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(launch_q4k_dual_matvec((const uint8_t*)da.data, (const uint8_t*)db.data, dx, (int)num_rows, (int)hidden, doa, dob,
                              ctx->sm_count, ctx->stream));
    ctx->launches += 1;
    CK(cudaMemcpyAsync(out_a, doa, num_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaMemcpyAsync(out_b, dob, num_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_q8_0_gemv(lq_ctx* ctx, const uint8_t* blocks, size_t blocks_len, const float* x, size_t x_len, size_t n,
                 size_t k, float* out) {
    DevGuard dev_guard(ctx);
    const lq_matrix m{LQ_FMT_Q8_0, blocks, blocks_len, nullptr, 0, 1.0f, (int64_t)n, (int64_t)k};
    return lq_gemv(ctx, &m, x, x_len, out, n, 0);
}
int lq_mxfp4_gemv(lq_ctx* ctx, const uint8_t* packed, size_t packed_len, const uint8_t* scales, size_t scales_len,
                  const float* x, size_t x_len, size_t n, size_t k, float* out) {
    DevGuard dev_guard(ctx);
    const lq_matrix m{LQ_FMT_MXFP4, packed, packed_len, scales, scales_len, 1.0f, (int64_t)n, (int64_t)k};
    return lq_gemv(ctx, &m, x, x_len, out, n, 0);
}
int lq_nvfp4_gemv(lq_ctx* ctx, const uint8_t* packed, size_t packed_len, const uint8_t* scales, size_t scales_len,
                  float tensor_scale, const float* x, size_t x_len, size_t n, size_t k, float* out) {
    DevGuard dev_guard(ctx);
    const lq_matrix m{LQ_FMT_NVFP4, packed, packed_len, scales, scales_len, tensor_scale, (int64_t)n, (int64_t)k};
    return lq_gemv(ctx, &m, x, x_len, out, n, 0);
}

// Several block-format matrices against ONE input vector in one submission: the input is uploaded
// once, every gemv is enqueued back to back and the call waits once.
int lq_gemv_multi(lq_ctx* ctx, const lq_matrix* mats, size_t n_mats, const float* x, size_t x_len, float* const* outs,
                  int exact) {
    DevGuard dev_guard(ctx);
    if (!ctx || (n_mats && (!mats || !outs))) return LQ_ERR_ARGUMENT;
    if (n_mats == 0) return LQ_OK;
    size_t total_out = 0;
    int rc;
    std::vector<lq_matrix> dm(n_mats);
    for (size_t i = 0; i < n_mats; ++i) {
        if ((rc = check_matrix(ctx, &mats[i], "gemv_multi"))) return rc;
        const int fmt = mats[i].fmt & 0xff;
        const size_t k = (size_t)mats[i].cols;
        if (x_len != k) return fail(ctx, LQ_REFUSED_SHAPE, "gemv_multi: every k must equal x_len");
        if (fmt == LQ_FMT_Q4_K ? (k % 256 != 0) : (k % 32 != 0) || k > 16384 || k == 0)
            return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv_multi: k must be a block multiple, 1..16384");
        if ((rc = resolve_matrix(ctx, &mats[i], &dm[i]))) return rc;
        if (fmt == LQ_FMT_Q4_K ? (((uintptr_t)dm[i].data & 15) != 0) : !fmt_aligned(dm[i]))
            return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv_multi: weight base address not block aligned");
        total_out += a256((size_t)mats[i].rows * 4);
    }
    const size_t k = x_len;
    if ((rc = ensure_ws(ctx, 1, k, 32))) return rc;
    if ((rc = ensure_stage(ctx, a256(k * 4) + total_out + 512))) return rc;
    float* dx = (float*)ctx->stage;
    uint8_t* dout = ctx->stage + a256(k * 4);
    TokenWs& t = ctx->tok[0];
    CK(cudaMemcpyAsync(dx, x, k * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (!exact) {
        launch_prep(dx, 1, (int)k, 0, 0.0, t.xn, t.xa, t.xb, t.bscale, t.bsum, t.babs, 0, nullptr, ctx->stream);
        CK(cudaGetLastError());
        ctx->launches += 1;
    }
    size_t off = 0;
    for (size_t i = 0; i < n_mats; ++i) {
        const size_t n = (size_t)dm[i].rows;
        float* o = (float*)(dout + off);
        if (n) {
            if ((dm[i].fmt & 0xff) == LQ_FMT_Q4_K) {
                const Q4kMat m{(const uint8_t*)dm[i].data, (int)n, (int)k};
                if (exact)
                    CK(launch_rescore_q4k(m, dx, nullptr, nullptr, (int)n, o, t, 0, 0, ctx->d_err, ctx->sm_count,
                                          ctx->stream));
                else
                    CK(launch_scan_q4k(m, xprep_of(t), o, nullptr, nullptr, 0.0f, ctx->d_err, ctx->sm_count, ctx->stream));
            } else {
                const FmtMat fm = fmtmat_of(dm[i]);
                if (exact) CK(launch_rescore_fmt(fm, dx, nullptr, nullptr, (int)n, o, ctx->sm_count, ctx->stream));
                else CK(launch_scan_fmt(fm, xprep_of(t), o, nullptr, nullptr, 0.0f, ctx->d_err, ctx->sm_count, ctx->stream));
            }
            ctx->launches += 1;
            CK(cudaMemcpyAsync(outs[i], o, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        }
        off += a256(n * 4);
    }
    return lq_synchronize(ctx);
}

int lq_mxfp4_gemv_multi(lq_ctx* ctx, const lq_matrix* mats, size_t n_mats, const float* x, size_t x_len,
                        float* const* outs) {
    for (size_t i = 0; mats && i < n_mats; ++i)
        if ((mats[i].fmt & 0xff) != LQ_FMT_MXFP4) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "mxfp4_gemv_multi: not MXFP4");
    return lq_gemv_multi(ctx, mats, n_mats, x, x_len, outs, 0);
}
int lq_nvfp4_gemv_multi(lq_ctx* ctx, const lq_matrix* mats, size_t n_mats, const float* x, size_t x_len,
                        float* const* outs) {
    for (size_t i = 0; mats && i < n_mats; ++i)
        if ((mats[i].fmt & 0xff) != LQ_FMT_NVFP4) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "nvfp4_gemv_multi: not NVFP4");
    return lq_gemv_multi(ctx, mats, n_mats, x, x_len, outs, 0);
}

// f16 (kind 0) / bf16 (kind 1) gemv, single and multi, and the LM-head top-k forms.
static int gemv16_check(lq_ctx* ctx, size_t w_len, size_t x_len, size_t n, size_t k, int kind, int exact) {
    if (kind != 0 && kind != 1) return fail(ctx, LQ_ERR_ARGUMENT, "gemv16: kind must be 0 (f16) or 1 (bf16)");
    if (w_len < n * k * 2 || x_len != k) return fail(ctx, LQ_REFUSED_SHAPE, "gemv16: w_len < n*k*2 or x_len != k");
    if (n > 0x7fffffffu || k > 0x7fffffffu || (exact && k > 32768))
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv16: size");
    return LQ_OK;
}

int lq_gemv16_multi(lq_ctx* ctx, int kind, size_t n_mats, const uint8_t* const* ws, const size_t* w_lens,
                    const size_t* ns, size_t k, const float* x, size_t x_len, float* const* outs, int exact) {
    DevGuard dev_guard(ctx);
    if (!ctx || (n_mats && (!ws || !w_lens || !ns || !outs))) return LQ_ERR_ARGUMENT;
    int rc;
    size_t total_out = 0;
    std::vector<const uint8_t*> dw(n_mats);
    for (size_t i = 0; i < n_mats; ++i) {
        if ((rc = gemv16_check(ctx, w_lens[i], x_len, ns[i], k, kind, exact))) return rc;
        if ((rc = resolve(ctx, ws[i], ns[i] * k * 2, &dw[i]))) return rc;
        if (((uintptr_t)dw[i] & 1) != 0) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv16: weights not 2-byte aligned");
        total_out += a256(ns[i] * 4);
    }
    if (n_mats == 0 || k == 0) {
        for (size_t i = 0; i < n_mats; ++i) memset(outs[i], 0, ns[i] * 4);
        return LQ_OK;
    }
    if ((rc = ensure_stage(ctx, a256(k * 4) + total_out + 512))) return rc;
    float* dx = (float*)ctx->stage;
    uint8_t* dout = ctx->stage + a256(k * 4);
    CK(cudaMemcpyAsync(dx, x, k * 4, cudaMemcpyHostToDevice, ctx->stream));
    size_t off = 0;
    for (size_t i = 0; i < n_mats; ++i) {
        float* o = (float*)(dout + off);
        if (ns[i]) {
            CK(launch_gemv16(dw[i], dx, (int)ns[i], (int)k, kind, exact, o, ctx->stream));
            ctx->launches += 1;
            CK(cudaMemcpyAsync(outs[i], o, ns[i] * 4, cudaMemcpyDeviceToHost, ctx->stream));
        }
        off += a256(ns[i] * 4);
    }
    return lq_synchronize(ctx);
}

int lq_gemv16(lq_ctx* ctx, int kind, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n, size_t k,
              float* out, int exact) {
    return lq_gemv16_multi(ctx, kind, 1, &w, &w_len, &n, k, x, x_len, &out, exact);
}
int lq_f16_gemv(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n, size_t k,
                float* out) {
    return lq_gemv16(ctx, 0, w, w_len, x, x_len, n, k, out, 0);
}
int lq_bf16_gemv(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n, size_t k,
                 float* out) {
    return lq_gemv16(ctx, 1, w, w_len, x, x_len, n, k, out, 0);
}

// Scores on the device (reference order), top-k by value on the device, k pairs back.
static int topk_from_scores(lq_ctx* ctx, float* dscores, size_t n, size_t top_k, uint32_t* idx_out, float* val_out,
                            size_t* count) {
    const size_t kk = std::min(top_k, n);
    uint32_t* di = (uint32_t*)((uint8_t*)dscores + a256(n * 4));
    float* dv = (float*)((uint8_t*)di + a256(kk * 4));
    CK(launch_topk_value_sorted(dscores, (int)n, (int)kk, di, dv, ctx->d_err, ctx->stream));
    ctx->launches += 1;
    CK(cudaMemcpyAsync(idx_out, di, kk * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaMemcpyAsync(val_out, dv, kk * 4, cudaMemcpyDeviceToHost, ctx->stream));
    int rc = lq_synchronize(ctx);
    if (rc) return rc;
    *count = kk;
    return LQ_OK;
}

int lq_q4k_matvec_topk(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                       size_t hidden, size_t top_k, uint32_t* idx_out, float* val_out, size_t* count) {
    DevGuard dev_guard(ctx);
    if (!ctx || !count) return LQ_ERR_ARGUMENT;
    *count = 0;
    const size_t needed = (hidden / 256) * 144 * num_rows;
    if (!(x_len == hidden && hidden % 256 == 0 && w_len >= needed))
        return fail(ctx, LQ_REFUSED_SHAPE, "q4k_matvec_topk: shape (KernelShapeError)");
    if (num_rows == 0 || top_k == 0) return LQ_OK;
    if (hidden == 0 || hidden > 16384 || num_rows > 0x7fffffffu)
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "q4k_matvec_topk: hidden 256..16384");
    if (std::min(top_k, num_rows) > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "q4k_matvec_topk: top_k > 16384");
    if (!idx_out || !val_out) return LQ_ERR_ARGUMENT;
    const uint8_t* dw;
    int rc = resolve(ctx, w, needed, &dw);
    if (rc) return rc;
    if (((uintptr_t)dw & 15) != 0) return fail(ctx, LQ_ERR_ARGUMENT, "q4k_matvec_topk: weights not 16-byte aligned");
    const size_t kk = std::min(top_k, num_rows);
    if ((rc = ensure_ws(ctx, 1, hidden, 32))) return rc;
    if ((rc = ensure_stage(ctx, a256(hidden * 4) + a256(num_rows * 4) + 2 * a256(kk * 4) + 512))) return rc;
    float* dx = (float*)ctx->stage;
    float* ds = (float*)(ctx->stage + a256(hidden * 4));
    CK(cudaMemcpyAsync(dx, x, hidden * 4, cudaMemcpyHostToDevice, ctx->stream));
    const Q4kMat m{dw, (int)num_rows, (int)hidden};
    // scores in the CPU backend's exact order, so that the selected rows are the ones q4k_matvec + a CPU
    // reduce would pick
    CK(launch_rescore_q4k(m, dx, nullptr, nullptr, (int)num_rows, ds, ctx->tok[0], 0, 0, ctx->d_err, ctx->sm_count,
                          ctx->stream));
    ctx->launches += 1;
    return topk_from_scores(ctx, ds, num_rows, top_k, idx_out, val_out, count);
}

int lq_gemv16_topk(lq_ctx* ctx, int kind, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n,
                   size_t k, size_t top_k, uint32_t* idx_out, float* val_out, size_t* count) {
    DevGuard dev_guard(ctx);
    if (!ctx || !count) return LQ_ERR_ARGUMENT;
    *count = 0;
    int rc = gemv16_check(ctx, w_len, x_len, n, k, kind, 1);
    if (rc) return rc;
    if (n == 0 || top_k == 0) return LQ_OK;
    if (k == 0) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv16_topk: k == 0");
    if (std::min(top_k, n) > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv16_topk: top_k > 16384");
    if (!idx_out || !val_out) return LQ_ERR_ARGUMENT;
    const uint8_t* dw;
    if ((rc = resolve(ctx, w, n * k * 2, &dw))) return rc;
    if (((uintptr_t)dw & 1) != 0) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "gemv16_topk: weights not 2-byte aligned");
    const size_t kk = std::min(top_k, n);
    if ((rc = ensure_stage(ctx, a256(k * 4) + a256(n * 4) + 2 * a256(kk * 4) + 512))) return rc;
    float* dx = (float*)ctx->stage;
    float* ds = (float*)(ctx->stage + a256(k * 4));
    CK(cudaMemcpyAsync(dx, x, k * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(launch_gemv16(dw, dx, (int)n, (int)k, kind, 1, ds, ctx->stream));
    ctx->launches += 1;
    return topk_from_scores(ctx, ds, n, top_k, idx_out, val_out, count);
}
int lq_f16_gemv_topk(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n, size_t k,
                     size_t top_k, uint32_t* idx_out, float* val_out, size_t* count) {
    return lq_gemv16_topk(ctx, 0, w, w_len, x, x_len, n, k, top_k, idx_out, val_out, count);
}

int lq_moe_route(lq_ctx* ctx, const float* logits, size_t n_tokens, size_t n_experts, size_t top_k, int renormalise,
                 uint32_t* idx_out, float* w_out) {
    DevGuard dev_guard(ctx);
    if (!ctx || !logits || !idx_out || !w_out) return LQ_ERR_ARGUMENT;
    if (n_experts == 0 || n_experts > 256) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "moe_route: 1..256 experts");
    if (n_tokens == 0 || top_k == 0) return LQ_OK;
    const size_t k = std::min(top_k, n_experts);
    int rc = ensure_stage(ctx, a256(n_tokens * n_experts * 4) + 2 * a256(n_tokens * k * 4));
    if (rc) return rc;
    float* dl = (float*)ctx->stage;
    uint32_t* di = (uint32_t*)(ctx->stage + a256(n_tokens * n_experts * 4));
    float* dw = (float*)((uint8_t*)di + a256(n_tokens * k * 4));
    CK(cudaMemcpyAsync(dl, logits, n_tokens * n_experts * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(launch_moe_route(dl, (int)n_tokens, (int)n_experts, (int)k, renormalise, di, dw, ctx->stream));
    ctx->launches += 1;
    CK(cudaMemcpyAsync(idx_out, di, n_tokens * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaMemcpyAsync(w_out, dw, n_tokens * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_topk_abs(lq_ctx* ctx, const float* scores, size_t n, size_t top_k, uint32_t* idx_out, float* val_out,
                size_t* count) {
    DevGuard dev_guard(ctx);
    if (!ctx || !count) return LQ_ERR_ARGUMENT;
    *count = 0;
    if (n == 0 || top_k == 0) return LQ_OK;
    if (n > (1u << 30)) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "topk: n too large");
    const size_t k = std::min(n, top_k);
    int rc = ensure_ws(ctx, 1, 256, n);
    if (rc) return rc;
    rc = ensure_sort(ctx, k);
    if (rc) return rc;
    rc = ensure_stage(ctx, n * 4 + k * 8 + 1024);
    if (rc) return rc;
    float* ds = (float*)ctx->stage;
    uint32_t* di = (uint32_t*)(ctx->stage + a256(n * 4));
    float* dv = (float*)(ctx->stage + a256(n * 4) + a256(k * 4));
    CK(cudaMemcpyAsync(ds, scores, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(launch_topk_abs_sorted(ds, (int)n, (int)k, ctx->tok[0], di, dv, nullptr, ctx->sort_buf, ctx->d_err,
                              ctx->stream));
    ctx->launches += 3;
    CK(cudaMemcpyAsync(idx_out, di, k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaMemcpyAsync(val_out, dv, k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    rc = lq_synchronize(ctx);
    if (rc) return rc;
    *count = k;
    return LQ_OK;
}

int lq_rms_norm(lq_ctx* ctx, const float* x, size_t rows, size_t cols, double eps, float* out) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    if (rows == 0 || cols == 0) return LQ_OK;
    if (cols % 32 != 0 || cols > 16384) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "rms_norm: cols % 32 != 0");
    int rc = ensure_ws(ctx, 1, cols, 32);
    if (rc) return rc;
    rc = ensure_stage(ctx, cols * 4);
    if (rc) return rc;
    TokenWs& t = ctx->tok[0];
    for (size_t r = 0; r < rows; ++r) {
        CK(cudaMemcpyAsync(ctx->stage, x + r * cols, cols * 4, cudaMemcpyHostToDevice, ctx->stream));
        launch_prep((const float*)ctx->stage, 1, (int)cols, 1, eps, t.xn, t.xa, t.xb, t.bscale, t.bsum, t.babs, 0,
                    nullptr, ctx->stream);
        CK(cudaGetLastError());
        ctx->launches += 1;
        CK(cudaMemcpyAsync(out + r * cols, t.xn, cols * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return lq_synchronize(ctx);
}

int lq_dequantize(lq_ctx* ctx, const lq_matrix* m, float* out, size_t out_len) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    int rc = check_matrix(ctx, m, "dequantize");
    if (rc) return rc;
    const size_t n = (size_t)m->rows * (size_t)m->cols;
    if (out_len != n) return fail(ctx, LQ_REFUSED_SHAPE, "dequantize: out_len != rows*cols");
    if (n == 0) return LQ_OK;
    lq_matrix dm;
    rc = resolve_matrix(ctx, m, &dm);
    if (rc) return rc;
    rc = ensure_stage(ctx, n * 4);
    if (rc) return rc;
    CK(launch_dequantize(dm, (float*)ctx->stage, ctx->stream));
    ctx->launches += 1;
    CK(cudaMemcpyAsync(out, ctx->stage, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

// ------------------------------------------------------------------ the walk ----
int lq_dev_walk_ffn(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down_fm,
                    const float* x, size_t batch, size_t top_k, uint32_t flags, float* out, uint32_t* idx_out,
                    uint32_t* count_out) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    int rc;
    if ((rc = check_matrix(ctx, gate, "gate")) || (rc = check_matrix(ctx, up, "up")) ||
        (rc = check_matrix(ctx, down_fm, "down")))
        return rc;
    lq_matrix g = *gate, u = *up, d = *down_fm;
    g.fmt &= 0xff;
    u.fmt &= 0xff;
    d.fmt &= 0xff;
    return dev_walk(ctx, &g, &u, &d, x, batch, top_k, flags, out, idx_out, count_out);
}

int lq_walk_ffn(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down_fm, const float* x,
                size_t batch, size_t top_k, uint32_t flags, float* out, uint32_t* idx_out, uint32_t* count_out) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    int rc;
    if ((rc = check_matrix(ctx, gate, "gate")) || (rc = check_matrix(ctx, up, "up")) ||
        (rc = check_matrix(ctx, down_fm, "down")))
        return rc;
    lq_matrix g, u, d;
    if ((rc = resolve_matrix(ctx, gate, &g)) || (rc = resolve_matrix(ctx, up, &u)) ||
        (rc = resolve_matrix(ctx, down_fm, &d)))
        return rc;
    const size_t H = (size_t)gate->cols, N = (size_t)gate->rows;
    const size_t k = effective_k(top_k, N, flags);
    const size_t xb = a256(batch * H * 4), ib = a256(batch * std::max<size_t>(k, 1) * 4), cb = a256(batch * 4);
    rc = ensure_stage(ctx, 2 * xb + ib + cb);
    if (rc) return rc;
    float* dx = (float*)ctx->stage;
    float* dout = (float*)(ctx->stage + xb);
    uint32_t* didx = (uint32_t*)(ctx->stage + 2 * xb);
    uint32_t* dcnt = (uint32_t*)(ctx->stage + 2 * xb + ib);
    if (batch * H) CK(cudaMemcpyAsync(dx, x, batch * H * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = dev_walk(ctx, &g, &u, &d, dx, batch, top_k, flags, dout, idx_out ? didx : nullptr,
                  count_out ? dcnt : nullptr);
    if (rc) return rc;
    if (batch * H) CK(cudaMemcpyAsync(out, dout, batch * H * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (idx_out && batch * k) CK(cudaMemcpyAsync(idx_out, didx, batch * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (count_out && batch) {
        if (N == 0) memset(count_out, 0, batch * 4);
        else CK(cudaMemcpyAsync(count_out, dcnt, batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    rc = lq_synchronize(ctx);
    if (rc) return rc;
    if (N && batch && H) {
        if (ctx->last_fused) {
            CK(cudaMemcpy(&ctx->stats, ctx->stats_dev, sizeof(lq_walk_stats), cudaMemcpyDeviceToHost));
        } else {
            SelHeader h;
            CK(cudaMemcpy(&h, ctx->tok[0].sel, sizeof h, cudaMemcpyDeviceToHost));
            ctx->stats = lq_walk_stats{h.n_in, h.n_band, h.n_sel, h.need, h.tau, h.bound};
        }
    }
    return LQ_OK;
}

// MoE expert walk: route each token to its top experts, walk each selected expert's
// gate/up/down with the per-expert top-K, combine with the routing weights.
int lq_moe_walk_ffn(lq_ctx* ctx, const lq_matrix* gates, const lq_matrix* ups, const lq_matrix* downs_fm,
                    size_t n_experts, const float* logits, const float* x, size_t batch, size_t top_e, int renormalise,
                    size_t top_k, uint32_t flags, float* out, uint32_t* expert_idx_out, float* expert_w_out) {
    DevGuard dev_guard(ctx);
    if (!ctx || !gates || !ups || !downs_fm || !logits || !x || !out) return LQ_ERR_ARGUMENT;
    if (n_experts == 0 || n_experts > 256) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "moe_walk: 1..256 experts");
    if (flags & (LQ_WALK_RMSNORM | LQ_WALK_RESIDUAL))
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "moe_walk: norm/residual belong to the caller");
    int rc;
    std::vector<lq_matrix> g(n_experts), u(n_experts), d(n_experts);
    for (size_t e = 0; e < n_experts; ++e) {
        if ((rc = check_matrix(ctx, gates + e, "gate")) || (rc = check_matrix(ctx, ups + e, "up")) ||
            (rc = check_matrix(ctx, downs_fm + e, "down")))
            return rc;
        if (gates[e].cols != gates[0].cols) return fail(ctx, LQ_REFUSED_SHAPE, "moe_walk: experts differ in hidden");
        if ((rc = resolve_matrix(ctx, gates + e, &g[e])) || (rc = resolve_matrix(ctx, ups + e, &u[e])) ||
            (rc = resolve_matrix(ctx, downs_fm + e, &d[e])))
            return rc;
    }
    const size_t H = (size_t)gates[0].cols, ke = std::min(top_e, n_experts);
    if (batch == 0 || H == 0) return LQ_OK;
    const size_t lb = a256(batch * n_experts * 4), rb = a256(batch * std::max<size_t>(ke, 1) * 4), xb = a256(batch * H * 4);
    rc = ensure_stage(ctx, lb + 2 * rb + 2 * xb + a256(H * 4));
    if (rc) return rc;
    float* dl = (float*)ctx->stage;
    uint32_t* di = (uint32_t*)(ctx->stage + lb);
    float* dw = (float*)(ctx->stage + lb + rb);
    float* dx = (float*)(ctx->stage + lb + 2 * rb);
    float* dout = (float*)(ctx->stage + lb + 2 * rb + xb);
    float* dtmp = (float*)(ctx->stage + lb + 2 * rb + 2 * xb);
    CK(cudaMemcpyAsync(dl, logits, batch * n_experts * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(cudaMemcpyAsync(dx, x, batch * H * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(cudaMemsetAsync(dout, 0, batch * H * 4, ctx->stream));
    // Experts in one block format and one shape (what a mixture-of-experts layer holds): every (token, expert)
    // pair is walked by the same few launches, pair y reading its expert's matrices through a device table, and
    // nothing comes back to the host between routing and the result.  LARQL_B200_MOE_GROUPED=0 keeps the
    // per-pair walks below (also the route for Q4_K experts and mixed shapes).
    static const bool grouped_on = [] { const char* e = getenv("LARQL_B200_MOE_GROUPED"); return !(e && e[0] == '0'); }();
    bool uniform = grouped_on && ke > 0 && gates[0].fmt != LQ_FMT_Q4_K && gates[0].fmt != LQ_FMT_Q6_K;
    for (size_t e = 0; uniform && e < n_experts; ++e) {
        uniform = g[e].fmt == g[0].fmt && u[e].fmt == g[0].fmt && d[e].fmt == g[0].fmt && g[e].rows == g[0].rows &&
                  u[e].rows == g[0].rows && d[e].rows == g[0].rows && u[e].cols == H && d[e].cols == H &&
                  fmt_aligned(g[e]) && fmt_aligned(u[e]) && fmt_aligned(d[e]);
    }
    if (uniform && g[0].rows > 0 && H % 32 == 0 && H <= 16384) {
        const size_t N = (size_t)g[0].rows, n_pairs = batch * ke;
        const int kk = (int)std::min<size_t>(top_k, N);
        // gather CTAs per pair: about six CTAs per SM over all pairs (what a narrow gather CTA lets an SM hold)
        const int gx = (int)std::max<size_t>(1, std::min<size_t>(16, (size_t)(6 * ctx->sm_count) / n_pairs));
        if ((rc = ensure_ws(ctx, n_pairs, H, N))) return rc;
        // (ensure_ws may have moved nothing the pointers above use: they live in the staging buffer)
        const size_t tb = a256(3 * n_experts * sizeof(FmtMat)), xpb = a256(n_pairs * H * 4),
                     pb = a256(n_pairs * (size_t)gx * H * 4);
        const size_t base = lb + 2 * rb + 2 * xb + a256(H * 4);
        if (base + tb + xpb + pb > ctx->stage_cap) {
            // grow the staging buffer once, before anything is enqueued into it
            if ((rc = ensure_stage(ctx, base + tb + xpb + pb))) return rc;
            dl = (float*)ctx->stage;
            di = (uint32_t*)(ctx->stage + lb);
            dw = (float*)(ctx->stage + lb + rb);
            dx = (float*)(ctx->stage + lb + 2 * rb);
            dout = (float*)(ctx->stage + lb + 2 * rb + xb);
            CK(cudaMemcpyAsync(dl, logits, batch * n_experts * 4, cudaMemcpyHostToDevice, ctx->stream));
            CK(cudaMemcpyAsync(dx, x, batch * H * 4, cudaMemcpyHostToDevice, ctx->stream));
        }
        FmtMat* dtab = (FmtMat*)(ctx->stage + base);
        float* dxp = (float*)(ctx->stage + base + tb);
        float* dpart = (float*)(ctx->stage + base + tb + xpb);
        std::vector<FmtMat> tab(3 * n_experts);
        for (size_t e = 0; e < n_experts; ++e) {
            tab[e] = fmtmat_of(g[e]);
            tab[n_experts + e] = fmtmat_of(u[e]);
            tab[2 * n_experts + e] = fmtmat_of(d[e]);
        }
        CK(cudaMemcpyAsync(dtab, tab.data(), tab.size() * sizeof(FmtMat), cudaMemcpyHostToDevice, ctx->stream));
        CK(cudaStreamSynchronize(ctx->stream));  // (the table is a local: its copy must have left before it goes away)
        cudaStream_t st = ctx->stream;
        const TokenWs& w0 = ctx->tok[0];
        const size_t ws_stride = n_pairs > 1 ? (size_t)((uint8_t*)ctx->tok[1].xn - (uint8_t*)ctx->tok[0].xn) : 0;
        CK(launch_moe_route(dl, (int)batch, (int)n_experts, (int)ke, renormalise, di, dw, st));
        CK(launch_moe_replicate(dx, (int)batch, (int)ke, (int)H, dxp, st));
        launch_prep(dxp, (int)n_pairs, (int)H, 0, 1e-6, w0.xn, w0.xa, w0.xb, w0.bscale, w0.bsum, w0.babs,
                    ws_stride / sizeof(float), ctx->d_err, st);
        CK(cudaGetLastError());
        CK(launch_scan_exact_pairs(g[0].fmt, dtab, di, (int)n_pairs, (int)N, (int)H, w0, ws_stride, ctx->d_err, st));
        CK(launch_select(w0.scores, (int)N, kk, w0, ctx->d_err, st, (int)n_pairs, ws_stride));
        if ((size_t)kk < N) CK(launch_final_pick(w0, ctx->d_err, st, (int)n_pairs, ws_stride));
        CK(launch_gather_fmt_pairs(g[0].fmt, dtab + n_experts, dtab + 2 * n_experts, di, (int)n_pairs, (int)H, w0, ws_stride,
                                   dpart, gx, st));
        CK(launch_moe_combine(dpart, dw, (int)batch, (int)ke, gx, (int)H, dout, st));
        ctx->launches += 8;
        if (expert_idx_out) CK(cudaMemcpyAsync(expert_idx_out, di, batch * ke * 4, cudaMemcpyDeviceToHost, st));
        if (expert_w_out) CK(cudaMemcpyAsync(expert_w_out, dw, batch * ke * 4, cudaMemcpyDeviceToHost, st));
        CK(cudaMemcpyAsync(out, dout, batch * H * 4, cudaMemcpyDeviceToHost, st));
        return lq_synchronize(ctx);
    }
    std::vector<uint32_t> hi(batch * ke);
    if (ke) {
        CK(launch_moe_route(dl, (int)batch, (int)n_experts, (int)ke, renormalise, di, dw, ctx->stream));
        ctx->launches += 1;
        CK(cudaMemcpyAsync(hi.data(), di, batch * ke * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (expert_w_out) CK(cudaMemcpyAsync(expert_w_out, dw, batch * ke * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CK(cudaStreamSynchronize(ctx->stream));
        if (expert_idx_out) memcpy(expert_idx_out, hi.data(), batch * ke * 4);
    }
    for (size_t t = 0; t < batch; ++t) {
        for (size_t j = 0; j < ke; ++j) {
            const uint32_t e = hi[t * ke + j];
            if (e >= n_experts) return fail(ctx, LQ_ERR_CUDA, "moe_walk: router returned a bad expert");
            rc = dev_walk(ctx, &g[e], &u[e], &d[e], dx + t * H, 1, top_k, flags, dtmp, nullptr, nullptr);
            if (rc) return rc;
            scaled_add_kernel<<<(unsigned)((H + 255) / 256), 256, 0, ctx->stream>>>(dout + t * H, dtmp, dw + t * ke + j,
                                                                                  (int)H);
            CK(cudaGetLastError());
            ctx->launches += 1;
        }
    }
    CK(cudaMemcpyAsync(out, dout, batch * H * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

int lq_fused_phase_us(lq_ctx* ctx, float* us, size_t n) {
    DevGuard dev_guard(ctx);
    if (!ctx || !us) return LQ_ERR_ARGUMENT;
    if (!ctx->stats_dev) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "no fused walk has run");
    CK(cudaStreamSynchronize(ctx->stream));
    int khz = 0;
    CK(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
    const double clk_mhz = khz > 0 ? khz * 1e-3 : 1965.0;  // stamps are SM cycles
    unsigned long long t[16];
    CK(cudaMemcpy(t, (uint8_t*)ctx->stats_dev + 64, sizeof t, cudaMemcpyDeviceToHost));
    const size_t n_phase = (size_t)fused_q4k_stamp_count() - 1;
    for (size_t i = 0; i < n; ++i) us[i] = i < n_phase ? (float)((double)(t[i + 1] - t[i]) / clk_mhz) : 0.0f;
    return LQ_OK;
}

int lq_last_walk_stats(lq_ctx* ctx, lq_walk_stats* out) {
    DevGuard dev_guard(ctx);
    if (!ctx || !out) return LQ_ERR_ARGUMENT;
    *out = ctx->stats;
    return LQ_OK;
}

int lq_dev_quantize_q4k(lq_ctx* ctx, const float* src, size_t n_elems, uint8_t* dst) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    if (n_elems % 256 != 0) return fail(ctx, LQ_REFUSED_SHAPE, "quantize_q4k: length % 256 != 0");
    if (((uintptr_t)dst & 15) != 0) return fail(ctx, LQ_ERR_ARGUMENT, "quantize_q4k: dst not 16-byte aligned");
    CK(launch_quantize_q4k(src, n_elems, dst, ctx->stream));
    ctx->launches += 1;
    return LQ_OK;
}

int lq_profile_walk(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down_fm,
                    const float* x, size_t top_k, uint32_t flags, float* out, float* ms) {
    DevGuard dev_guard(ctx);
    if (!ctx || !ms) return LQ_ERR_ARGUMENT;
    int rc;
    if ((rc = check_matrix(ctx, gate, "gate")) || (rc = check_matrix(ctx, up, "up")) ||
        (rc = check_matrix(ctx, down_fm, "down")))
        return rc;
    if ((gate->fmt & 0xff) != LQ_FMT_Q4_K) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "profile: Q4_K only");
    const int N = (int)gate->rows, H = (int)gate->cols;
    if (N == 0 || H == 0) return fail(ctx, LQ_REFUSED_SHAPE, "profile: empty layer");
    rc = ensure_ws(ctx, 1, H, N);
    if (rc) return rc;
    cudaEvent_t ev[7];
    for (auto& e : ev) CK(cudaEventCreate(&e));
    TokenWs& w = ctx->tok[0];
    const Q4kMat g{(const uint8_t*)gate->data, N, H}, u{(const uint8_t*)up->data, N, H},
        d{(const uint8_t*)down_fm->data, N, H};
    const XPrep xp = xprep_of(w);
    const int k = (int)effective_k(top_k, (size_t)N, flags);
    cudaStream_t st = ctx->stream;
    CK(cudaEventRecord(ev[0], st));
    launch_prep(x, 1, H, (flags & LQ_WALK_RMSNORM) ? 1 : 0, 1e-6, w.xn, w.xa, w.xb, w.bscale, w.bsum, w.babs, 0,
                ctx->d_err, st);
    CK(cudaEventRecord(ev[1], st));
    CK(launch_scan_q4k(g, xp, w.scores, k < N ? w.hist : nullptr, &w.sel->bound_bits, bound_c1(H), ctx->d_err,
                       ctx->sm_count, st));
    CK(cudaEventRecord(ev[2], st));
    if (k < N) CK(launch_classify(w.scores, N, k, w, ctx->d_err, st));
    else CK(launch_select(w.scores, N, k, w, ctx->d_err, st));
    CK(cudaEventRecord(ev[3], st));
    if (k < N)
        CK(launch_rescore_q4k(g, w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, w, k, 1, ctx->d_err,
                              ctx->sm_count, st));
    CK(cudaEventRecord(ev[4], st));
    CK(launch_gather_q4k(u, d, xp, w.hit_idx, w.hit_score, &w.sel->n_sel, k, ctx->partials, ctx->gather_grid,
                         ctx->d_err, st));
    CK(cudaEventRecord(ev[5], st));
    CK(launch_finish(ctx->partials, ctx->gather_grid, H, (flags & LQ_WALK_RESIDUAL) ? x : nullptr, out, st));
    CK(cudaEventRecord(ev[6], st));
    ctx->launches += 6;
    rc = lq_synchronize(ctx);
    for (int i = 0; i < 6; ++i) {
        float t = 0.0f;
        cudaEventElapsedTime(&t, ev[i], ev[i + 1]);
        ms[i] = t;
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return rc;
}

// ------------------------------------------------------- feature-sharded walk ----
static int shard_check(lq_ctx* ctx, const lq_matrix* m, const char* name) {
    int rc = check_matrix(ctx, m, name);
    if (rc) return rc;
    if (m->cols > 16384 || m->cols == 0 || m->cols % 32 != 0 || m->rows == 0)
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "sharded walk: shape");
    if ((m->fmt & 0xff) == LQ_FMT_Q4_K ? (((uintptr_t)m->data & 15) != 0) : !fmt_aligned(*m))
        return fail(ctx, LQ_ERR_ARGUMENT, "sharded walk: weights not block aligned");
    return LQ_OK;
}

int lq_dev_shard_scan(lq_ctx* ctx, const lq_matrix* gate_shard, const float* x, uint32_t flags, int rank, int world,
                      uint32_t* hist_buf) {
    DevGuard dev_guard(ctx);
    if (!ctx || !hist_buf || rank < 0 || world < 1 || rank >= world || world > 16) return LQ_ERR_ARGUMENT;
    int rc = shard_check(ctx, gate_shard, "gate shard");
    if (rc) return rc;
    const int N = (int)gate_shard->rows, H = (int)gate_shard->cols;
    rc = ensure_ws(ctx, 1, H, N);
    if (rc) return rc;
    TokenWs& w = ctx->tok[0];
    cudaStream_t st = ctx->stream;
    CK(cudaMemsetAsync(hist_buf + LQ_HIST_BINS, 0, 64 * 4, st));
    launch_prep(x, 1, H, (flags & LQ_WALK_RMSNORM) ? 1 : 0, 1e-6, w.xn, w.xa, w.xb, w.bscale, w.bsum, w.babs, 0,
                ctx->d_err, st);
    CK(cudaGetLastError());
    if ((gate_shard->fmt & 0xff) != LQ_FMT_Q4_K) {
        // exact-order scores: the bound slot stays zero
        CK(launch_scan_exact_fmt(fmtmat_of(*gate_shard), w.xn, w.scores, ctx->d_err, st));
        CK(launch_hist_abs(w.scores, N, hist_buf, st));
        ctx->launches += 3;
        return LQ_OK;
    }
    const Q4kMat g{(const uint8_t*)gate_shard->data, N, H};
    CK(launch_scan_q4k(g, xprep_of(w), w.scores, hist_buf, &w.sel->bound_bits, bound_c1(H), ctx->d_err, ctx->sm_count,
                       st));
    CK(cudaMemcpyAsync(hist_buf + LQ_HIST_BINS + rank, &w.sel->bound_bits, 4, cudaMemcpyDeviceToDevice, st));
    ctx->launches += 2;
    return LQ_OK;
}

int lq_dev_shard_classify(lq_ctx* ctx, const lq_matrix* gate_shard, uint32_t* hist_buf, int world, size_t top_k,
                          size_t row_offset, int32_t* pack, size_t cap) {
    DevGuard dev_guard(ctx);
    if (!ctx || !hist_buf || !pack || world < 1 || world > 16 || cap == 0) return LQ_ERR_ARGUMENT;
    int rc = shard_check(ctx, gate_shard, "gate shard");
    if (rc) return rc;
    const int N = (int)gate_shard->rows, H = (int)gate_shard->cols;
    if (top_k == 0) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "sharded walk: top_k == 0");
    if ((size_t)N > ctx->ws_feat || (size_t)H > ctx->ws_hidden) return fail(ctx, LQ_ERR_ARGUMENT, "shard_scan first");
    TokenWs w = ctx->tok[0];
    cudaStream_t st = ctx->stream;
    CK(launch_shard_bound_max(hist_buf + LQ_HIST_BINS, world, &w.sel->bound_bits, st));
    TokenWs wh = w;
    wh.hist = hist_buf;  // global histogram; the classify kernel clears it for the next layer
    CK(launch_classify(w.scores, N, (int)top_k, wh, ctx->d_err, st));
    if ((gate_shard->fmt & 0xff) != LQ_FMT_Q4_K) {
        CK(launch_rescore_fmt(fmtmat_of(*gate_shard), w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, ctx->sm_count, st));
    } else {
        const Q4kMat g{(const uint8_t*)gate_shard->data, N, H};
        CK(launch_rescore_q4k(g, w.xn, w.band_idx, &w.sel->n_band, 0, w.band_exact, w, (int)top_k, 0, ctx->d_err,
                              ctx->sm_count, st));
    }
    CK(launch_shard_pack(w, (uint32_t)row_offset, (int)cap, pack, ctx->d_err, st));
    ctx->launches += 4;
    return LQ_OK;
}

int lq_dev_shard_gather(lq_ctx* ctx, const lq_matrix* up_shard, const lq_matrix* down_shard, const int32_t* packs,
                        int world, int rank, size_t cap, size_t top_k, size_t row_offset, float* out_partial) {
    DevGuard dev_guard(ctx);
    if (!ctx || !packs || !out_partial || world < 1 || world > 16 || rank < 0 || rank >= world) return LQ_ERR_ARGUMENT;
    int rc;
    if ((rc = shard_check(ctx, up_shard, "up shard")) || (rc = shard_check(ctx, down_shard, "down shard"))) return rc;
    const int N = (int)up_shard->rows, H = (int)up_shard->cols;
    if (down_shard->rows != up_shard->rows || down_shard->cols != up_shard->cols)
        return fail(ctx, LQ_REFUSED_SHAPE, "sharded walk: up/down shapes differ");
    if ((size_t)N > ctx->ws_feat || (size_t)H > ctx->ws_hidden) return fail(ctx, LQ_ERR_ARGUMENT, "shard_scan first");
    TokenWs w = ctx->tok[0];
    cudaStream_t st = ctx->stream;
    CK(launch_shard_pick(packs, world, rank, (int)cap, (int)top_k, (uint32_t)row_offset, w, ctx->d_err, st));
    if ((up_shard->fmt & 0xff) != (down_shard->fmt & 0xff))
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "sharded walk: up/down formats differ");
    if ((up_shard->fmt & 0xff) != LQ_FMT_Q4_K) {
        CK(launch_gather_fmt(fmtmat_of(*up_shard), fmtmat_of(*down_shard), xprep_of(w), w.hit_idx, w.hit_score,
                             &w.sel->n_sel, N, ctx->partials, ctx->gather_grid, st));
    } else {
        const Q4kMat u{(const uint8_t*)up_shard->data, N, H}, d{(const uint8_t*)down_shard->data, N, H};
        CK(launch_gather_q4k(u, d, xprep_of(w), w.hit_idx, w.hit_score, &w.sel->n_sel, N, ctx->partials,
                             ctx->gather_grid, ctx->d_err, st));
    }
    CK(launch_finish(ctx->partials, ctx->gather_grid, H, nullptr, out_partial, st));
    ctx->launches += 3;
    return LQ_OK;
}

int lq_dev_shard_hits(lq_ctx* ctx, uint32_t* idx_out_host, size_t cap, size_t* count) {
    DevGuard dev_guard(ctx);
    if (!ctx || !count) return LQ_ERR_ARGUMENT;
    if (const lq_stack* xs = ctx->last_xstack) {
        uint32_t n = 0;
        CK(cudaMemcpyAsync(&n, xs->xhits + xs->top_k, 4, cudaMemcpyDeviceToHost, ctx->stream));
        CK(cudaStreamSynchronize(ctx->stream));
        if (n > xs->top_k) return fail(ctx, LQ_ERR_CUDA, "shard_hits: bad count");
        *count = (size_t)n;
        const size_t m = std::min((size_t)n, cap);
        if (m && idx_out_host) CK(cudaMemcpy(idx_out_host, xs->xhits, m * 4, cudaMemcpyDeviceToHost));
        return LQ_OK;
    }
    if (ctx->tok.empty()) return LQ_ERR_ARGUMENT;
    TokenWs w = ctx->tok[0];
    int n = 0;
    CK(cudaMemcpyAsync(&n, &w.sel->n_sel, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaStreamSynchronize(ctx->stream));
    if (n < 0 || (size_t)n > ctx->ws_feat) return fail(ctx, LQ_ERR_CUDA, "shard_hits: bad count");
    *count = (size_t)n;
    const size_t m = std::min((size_t)n, cap);
    if (m && idx_out_host) CK(cudaMemcpy(idx_out_host, w.hit_idx, m * 4, cudaMemcpyDeviceToHost));
    return LQ_OK;
}

// ----------------------------------------------------------------- layer stack ----
// One token of a feature-sharded stack: per layer three device steps with an NCCL exchange after each
// (histogram + bound slots, band packs, partial outputs), all enqueued on the context's stream.
static int sharded_enqueue_token(lq_ctx* ctx, lq_stack* s, const float* h_in, float* h_out) {
    NcclApi* nc = nccl_api();
    if (!nc || !ctx->comm) return fail(ctx, LQ_ERR_ARGUMENT, "sharded stack: lq_comm_init first");
    const size_t L = s->gates.size();
    const int H = s->hidden;
    const size_t stride = 2 + 2 * s->cap;
    const uint32_t flags = s->flags;
    const float* cur = h_in;
#define NCK(call)                                                                                   \
    do {                                                                                            \
        ncclResult_t r__ = (call);                                                                  \
        if (r__ != ncclSuccess) return fail(ctx, LQ_ERR_CUDA, std::string(#call) + ": " + nc->GetErrorString(r__)); \
    } while (0)
    for (size_t l = 0; l < L; ++l) {
        float* nxt = (l + 1 == L) ? h_out : s->h_buf[l & 1];
        int rc = lq_dev_shard_scan(ctx, &s->gates[l], cur, flags & LQ_WALK_RMSNORM, ctx->rank, ctx->world, s->hist_buf);
        if (rc) return rc;
        NCK(nc->AllReduce(s->hist_buf, s->hist_buf, LQ_HIST_WORDS, ncclUint32, ncclSum, ctx->comm, ctx->stream));
        rc = lq_dev_shard_classify(ctx, &s->gates[l], s->hist_buf, ctx->world, s->top_k, s->row_offset, s->pack, s->cap);
        if (rc) return rc;
        NCK(nc->AllGather(s->pack, s->packs, stride, ncclInt32, ctx->comm, ctx->stream));
        rc = lq_dev_shard_gather(ctx, &s->ups[l], &s->downs[l], s->packs, ctx->world, ctx->rank, s->cap, s->top_k,
                                 s->row_offset, s->out_partial);
        if (rc) return rc;
        NCK(nc->AllReduce(s->out_partial, s->out_partial, (size_t)H, ncclFloat, ncclSum, ctx->comm, ctx->stream));
        if (flags & LQ_WALK_RESIDUAL) {
            add_vec_kernel<<<(H + 255) / 256, 256, 0, ctx->stream>>>(nxt, cur, s->out_partial, H);
            CK(cudaGetLastError());
        } else {
            CK(cudaMemcpyAsync(nxt, s->out_partial, (size_t)H * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        }
        ctx->launches += 4;
        cur = nxt;
    }
#undef NCK
    return LQ_OK;
}

static int stack_enqueue(lq_ctx* ctx, lq_stack* s) {
    const size_t L = s->gates.size();
    if (s->xfused) {
        // The ranks' kernels wait for one another: a tiny all-reduce first, so that they start together
        // (and after every rank's previous launch on these areas has ended).
        NcclApi* nc = nccl_api();
        if (!nc || !ctx->comm) return fail(ctx, LQ_ERR_ARGUMENT, "sharded stack: lq_comm_init first");
        if (ctx->world > 1 &&
            nc->AllReduce(s->sync_word, s->sync_word, 1, ncclUint32, ncclSum, ctx->comm, ctx->stream) != ncclSuccess)
            return fail(ctx, LQ_ERR_CUDA, "sharded stack: launch rendezvous failed");
        const int H = s->hidden, Nl = (int)s->gates[0].rows;
        for (size_t t = 0; t < s->batch; ++t) {
            const bool last = t + 1 == s->batch;
            CK(launch_walk_fused_q4k_sharded(s->layers_dev, (int)L, Nl, (int)s->n_global, H, (int)s->top_k, s->flags,
                                             bound_c1(H), s->h_in + t * H, s->h_out + t * H, ctx->fws,
                                             last ? s->xhits : nullptr, last ? s->xhits + s->top_k : nullptr,
                                             t == 0 ? ctx->stats_dev : nullptr, ctx->d_err, ctx->sm_count, ctx->world,
                                             ctx->rank, s->areas.data(), s->row_offs.data(), s->xepoch, ctx->stream));
            s->xepoch += (uint32_t)L;
            ctx->launches += 1;
        }
        ctx->last_xstack = s;
        return LQ_OK;
    }
    if (s->sharded) {
        ctx->last_xstack = nullptr;
        for (size_t t = 0; t < s->batch; ++t) {
            int rc = sharded_enqueue_token(ctx, s, s->h_in + t * s->hidden, s->h_out + t * s->hidden);
            if (rc) return rc;
        }
        return LQ_OK;
    }
    if (s->fused) {
        const int N = (int)s->gates[0].rows, H = s->hidden;
        const size_t k = effective_k(s->top_k, (size_t)N, s->flags);
        for (size_t t = 0; t < s->batch; ++t) {
            CK(launch_walk_fused_q4k(s->layers_dev, nullptr, (int)L, N, H, (int)k, s->flags, bound_c1(H),
                                     s->h_in + t * H, s->h_out + t * H, ctx->fws, nullptr, nullptr,
                                     t == 0 ? ctx->stats_dev : nullptr, ctx->d_err,
                                     ctx->sm_count, ctx->stream));
            ctx->launches += 1;
        }
        return LQ_OK;
    }
    const float* cur = s->h_in;
    for (size_t l = 0; l < L; ++l) {
        float* nxt = (l + 1 == L) ? s->h_out : s->h_buf[l & 1];
        int rc = dev_walk(ctx, &s->gates[l], &s->ups[l], &s->downs[l], cur, s->batch, s->top_k, s->flags, nxt,
                          nullptr, nullptr);
        if (rc) return rc;
        cur = nxt;
    }
    return LQ_OK;
}

int lq_stack_create(lq_ctx* ctx, const lq_matrix* gates, const lq_matrix* ups, const lq_matrix* downs_fm,
                    size_t n_layers, size_t batch, size_t top_k, uint32_t flags, lq_stack** out) {
    DevGuard dev_guard(ctx);
    if (!ctx || !out || !n_layers || !batch) return LQ_ERR_ARGUMENT;
    *out = nullptr;
    int rc;
    for (size_t l = 0; l < n_layers; ++l) {
        if ((rc = check_matrix(ctx, &gates[l], "gate")) || (rc = check_matrix(ctx, &ups[l], "up")) ||
            (rc = check_matrix(ctx, &downs_fm[l], "down")))
            return rc;
        if (gates[l].cols != gates[0].cols) return fail(ctx, LQ_REFUSED_SHAPE, "stack: hidden differs per layer");
    }
    lq_stack* s = new lq_stack();
    s->gates.resize(n_layers);
    s->ups.resize(n_layers);
    s->downs.resize(n_layers);
    for (size_t l = 0; l < n_layers; ++l) {
        // host matrices are uploaded once through the weight cache, device matrices are taken as they are
        if ((rc = resolve_matrix(ctx, &gates[l], &s->gates[l])) || (rc = resolve_matrix(ctx, &ups[l], &s->ups[l])) ||
            (rc = resolve_matrix(ctx, &downs_fm[l], &s->downs[l]))) {
            delete s;
            return rc;
        }
    }
    s->batch = batch;
    s->top_k = top_k;
    s->flags = flags | LQ_WALK_RMSNORM | LQ_WALK_RESIDUAL;
    s->hidden = (int)gates[0].cols;
    const size_t bytes = a256(batch * s->hidden * 4);
    uint8_t* raw = nullptr;
    cudaError_t e = cudaMalloc(&raw, 4 * bytes);
    if (e != cudaSuccess) {
        delete s;
        return cuda_fail(ctx, e, "stack buffers");
    }
    s->h_in = (float*)raw;
    s->h_out = (float*)(raw + bytes);
    s->h_buf[0] = (float*)(raw + 2 * bytes);
    s->h_buf[1] = (float*)(raw + 3 * bytes);
    // Fused path: every layer the same shape and Q4_K -> one cooperative launch per token.
    {
        bool same = true;
        for (size_t l = 0; l < n_layers; ++l)
            same = same && gates[l].rows == gates[0].rows && gates[l].cols == gates[0].cols;
        const size_t k = effective_k(top_k, (size_t)gates[0].rows, s->flags);
        bool ok = same && batch < ctx->batch_min;  // batches take the tensor-core scan, layer by layer
        for (size_t l = 0; ok && l < n_layers; ++l) ok = fused_ok(ctx, s->gates[l], s->ups[l], s->downs[l], k);
        if (ok) {
            rc = ensure_fused(ctx, (size_t)s->hidden, (size_t)gates[0].rows);
            if (rc) {
                lq_stack_destroy(ctx, s);
                return rc;
            }
            std::vector<const void*> ptrs(3 * n_layers);
            for (size_t l = 0; l < n_layers; ++l) {
                ptrs[3 * l] = s->gates[l].data;
                ptrs[3 * l + 1] = s->ups[l].data;
                ptrs[3 * l + 2] = s->downs[l].data;
            }
            e = cudaMalloc(&s->layers_dev, ptrs.size() * sizeof(void*));
            if (e == cudaSuccess)
                e = cudaMemcpy(s->layers_dev, ptrs.data(), ptrs.size() * sizeof(void*), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                lq_stack_destroy(ctx, s);
                return cuda_fail(ctx, e, "stack layer table");
            }
            s->fused = true;
        }
    }
    // One eager pass on a harmless input grows the workspace and sets kernel attributes,
    // neither of which may happen inside a capture.
    cudaMemsetAsync(s->h_in, 0x3f, bytes, ctx->stream);
    rc = stack_enqueue(ctx, s);
    if (!rc) rc = lq_synchronize(ctx);
    if (!rc && !s->fused) {
        e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            rc = stack_enqueue(ctx, s);
            cudaError_t e2 = cudaStreamEndCapture(ctx->stream, &s->graph);
            if (!rc && e2 != cudaSuccess) rc = cuda_fail(ctx, e2, "end capture");
            if (!rc) {
                e2 = cudaGraphInstantiate(&s->exec, s->graph, 0);
                if (e2 != cudaSuccess) rc = cuda_fail(ctx, e2, "graph instantiate");
            }
        } else
            rc = cuda_fail(ctx, e, "begin capture");
    }
    if (rc) {
        lq_stack_destroy(ctx, s);
        return rc;
    }
    *out = s;
    return LQ_OK;
}

int lq_stack_run(lq_ctx* ctx, lq_stack* s, const float* h_in, float* h_out) {
    DevGuard dev_guard(ctx);
    if (!ctx || !s || (!s->exec && !s->fused && !s->sharded)) return LQ_ERR_ARGUMENT;
    const size_t bytes = s->batch * s->hidden * 4;
    CK(cudaMemcpyAsync(s->h_in, h_in, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    if (s->fused || s->sharded) {
        int rc = stack_enqueue(ctx, s);
        if (rc) return rc;
    } else
        CK(cudaGraphLaunch(s->exec, ctx->stream));
    CK(cudaMemcpyAsync(h_out, s->h_out, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return LQ_OK;
}

int lq_stack_run_host(lq_ctx* ctx, lq_stack* s, const float* h_in_host, float* h_out_host) {
    DevGuard dev_guard(ctx);
    if (!ctx || !s || (!s->exec && !s->fused && !s->sharded) || !h_in_host || !h_out_host) return LQ_ERR_ARGUMENT;
    const size_t bytes = s->batch * s->hidden * 4;
    CK(cudaMemcpyAsync(s->h_in, h_in_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    if (s->fused || s->sharded) {
        int rc = stack_enqueue(ctx, s);
        if (rc) return rc;
    } else
        CK(cudaGraphLaunch(s->exec, ctx->stream));
    CK(cudaMemcpyAsync(h_out_host, s->h_out, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return lq_synchronize(ctx);
}

// ------------------------------------------------------------- multi-GPU (NCCL) ----
int lq_comm_unique_id(void* id_out, size_t cap) {
    if (!id_out || cap < sizeof(ncclUniqueId)) return LQ_ERR_ARGUMENT;
    NcclApi* nc = nccl_api();
    if (!nc) return LQ_REFUSED_UNSUPPORTED;
    ncclUniqueId id;
    if (nc->GetUniqueId(&id) != ncclSuccess) return LQ_ERR_CUDA;
    memcpy(id_out, &id, sizeof id);
    return LQ_OK;
}

int lq_comm_init(lq_ctx* ctx, int rank, int world, const void* unique_id, size_t id_len) {
    DevGuard dev_guard(ctx);
    if (!ctx || !unique_id || id_len < sizeof(ncclUniqueId) || world < 1 || world > 16 || rank < 0 || rank >= world)
        return LQ_ERR_ARGUMENT;
    if (ctx->comm) return fail(ctx, LQ_ERR_ARGUMENT, "comm_init: this context already has a communicator");
    NcclApi* nc = nccl_api();
    if (!nc) return fail(ctx, LQ_REFUSED_UNSUPPORTED, "comm_init: libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    ncclResult_t r = nc->CommInitRank(&ctx->comm, world, id, rank);
    if (r != ncclSuccess) {
        ctx->comm = nullptr;
        return fail(ctx, LQ_ERR_CUDA, std::string("ncclCommInitRank: ") + nc->GetErrorString(r));
    }
    ctx->rank = rank;
    ctx->world = world;
    return LQ_OK;
}

int lq_comm_destroy(lq_ctx* ctx) {
    DevGuard dev_guard(ctx);
    if (!ctx) return LQ_ERR_ARGUMENT;
    if (ctx->comm) {
        cudaStreamSynchronize(ctx->stream);
        if (NcclApi* nc = nccl_api()) nc->CommDestroy(ctx->comm);
        ctx->comm = nullptr;
    }
    ctx->rank = 0;
    ctx->world = 1;
    return LQ_OK;
}

// Puts a sharded stack on the fused persistent kernel when every rank can: Q4_K layers of one shape that the
// kernel supports, and every rank's exchange area mapped into every other rank's process (CUDA IPC, one
// process per GPU).  All ranks take the same decision (the conditions are all-reduced), so a stack never
// runs fused on one rank and through NCCL on another.  Leaves s->xfused false and returns LQ_OK when the
// fused path is not available; a non-zero status is a failure of the set-up itself.
static int try_xfused(lq_ctx* ctx, lq_stack* s) {
    NcclApi* nc = nccl_api();
    const int world = ctx->world, rank = ctx->rank;
    const size_t L = s->gates.size();
    const int H = s->hidden, Nl = (int)s->gates[0].rows;
    bool ok = ctx->use_fused && world <= 8 && getenv("LARQL_B200_SHARDED_NCCL") == nullptr;
    for (size_t l = 0; ok && l < L; ++l)
        ok = s->gates[l].fmt == LQ_FMT_Q4_K && s->ups[l].fmt == LQ_FMT_Q4_K && s->downs[l].fmt == LQ_FMT_Q4_K &&
             s->gates[l].rows == s->gates[0].rows && s->ups[l].rows == s->gates[0].rows &&
             s->downs[l].rows == s->gates[0].rows && s->gates[l].cols == s->gates[0].cols;
    ok = ok && fused_q4k_sharded_supported(H, Nl, (int)s->n_global, (int)s->top_k, world, ctx->sm_count);
    // scratch for the small exchanges: [0, 1024) send, [1024, ...) receive
    uint8_t* tmp = nullptr;
    CK(cudaMalloc(&tmp, 1024 + 1024 * 16));
    struct Hello {
        int ok, row_offset, n_rows, pad;
        cudaIpcMemHandle_t handle;
    };
    static_assert(sizeof(Hello) <= 1024, "hello record");
    Hello mine;
    memset(&mine, 0, sizeof mine);
    mine.row_offset = (int)s->row_offset;
    mine.n_rows = Nl;
    cudaError_t e = cudaSuccess;
    if (ok) {
        const size_t xb = fused_q4k_xarea_bytes(H, (int)s->n_global, world);
        e = cudaMalloc(&s->xarea, xb);
        if (e == cudaSuccess) e = cudaMemset(s->xarea, 0, xb);
        if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(&mine.handle, s->xarea);
        if (e != cudaSuccess) {
            cudaGetLastError();
            ok = false;
        }
    }
    mine.ok = ok ? 1 : 0;
    std::vector<Hello> all((size_t)world);
    auto exchange = [&]() -> int {
        CK(cudaMemcpyAsync(tmp, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream));
        if (nc->AllGather(tmp, tmp + 1024, sizeof(Hello), ncclChar, ctx->comm, ctx->stream) != ncclSuccess)
            return fail(ctx, LQ_ERR_CUDA, "sharded stack: all-gather of the set-up records failed");
        CK(cudaMemcpyAsync(all.data(), tmp + 1024, sizeof(Hello) * (size_t)world, cudaMemcpyDeviceToHost, ctx->stream));
        CK(cudaStreamSynchronize(ctx->stream));
        return LQ_OK;
    };
    int rc = exchange();
    if (!rc) {
        for (int r = 0; r < world; ++r) ok = ok && all[(size_t)r].ok;
        s->row_offs.resize((size_t)world);
        s->areas.assign((size_t)world, nullptr);
        long long rows = 0;
        for (int r = 0; r < world; ++r) {
            s->row_offs[(size_t)r] = all[(size_t)r].row_offset;
            rows += all[(size_t)r].n_rows;
        }
        ok = ok && rows == (long long)s->n_global;  // the ranks' row ranges make up the whole layer
        if (ok) {
            s->areas[(size_t)rank] = s->xarea;
            for (int r = 0; r < world && ok; ++r) {
                if (r == rank) continue;
                void* ptr = nullptr;
                e = cudaIpcOpenMemHandle(&ptr, all[(size_t)r].handle, cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) {
                    cudaGetLastError();
                    ok = false;
                } else
                    s->areas[(size_t)r] = (uint8_t*)ptr;
            }
        }
        // second round: did every rank map every area?
        mine.ok = ok ? 1 : 0;
        rc = exchange();
        if (!rc)
            for (int r = 0; r < world; ++r) ok = ok && all[(size_t)r].ok;
    }
    cudaFree(tmp);
    if (rc) return rc;
    if (!ok) {
        for (int r = 0; r < world; ++r)
            if (r != rank && r < (int)s->areas.size() && s->areas[(size_t)r]) cudaIpcCloseMemHandle(s->areas[(size_t)r]);
        s->areas.clear();
        if (s->xarea) cudaFree(s->xarea);
        s->xarea = nullptr;
        return LQ_OK;
    }
    rc = ensure_fused(ctx, (size_t)H, (size_t)Nl);
    if (rc) return rc;
    std::vector<const void*> ptrs(3 * L);
    for (size_t l = 0; l < L; ++l) {
        ptrs[3 * l] = s->gates[l].data;
        ptrs[3 * l + 1] = s->ups[l].data;
        ptrs[3 * l + 2] = s->downs[l].data;
    }
    CK(cudaMalloc(&s->layers_dev, ptrs.size() * sizeof(void*)));
    CK(cudaMemcpy(s->layers_dev, ptrs.data(), ptrs.size() * sizeof(void*), cudaMemcpyHostToDevice));
    CK(cudaMalloc(&s->xhits, (s->top_k + 2) * 4));
    CK(cudaMemset(s->xhits, 0, (s->top_k + 2) * 4));
    s->sync_word = s->xhits + s->top_k + 1;
    s->xfused = true;
    return LQ_OK;
}

int lq_stack_create_sharded(lq_ctx* ctx, const lq_matrix* gate_shards, const lq_matrix* up_shards,
                            const lq_matrix* down_shards_fm, size_t n_layers, size_t batch, size_t top_k,
                            size_t n_features_global, size_t row_offset, uint32_t flags, size_t cap, lq_stack** out) {
    DevGuard dev_guard(ctx);
    if (!ctx || !out || !n_layers || !batch || !cap) return LQ_ERR_ARGUMENT;
    *out = nullptr;
    if (!ctx->comm) return fail(ctx, LQ_ERR_ARGUMENT, "sharded stack: lq_comm_init first");
    if (top_k == 0 || top_k >= n_features_global)
        return fail(ctx, LQ_REFUSED_UNSUPPORTED, "sharded stack: 0 < top_k < global feature count");
    int rc;
    lq_stack* s = new lq_stack();
    s->gates.resize(n_layers);
    s->ups.resize(n_layers);
    s->downs.resize(n_layers);
    for (size_t l = 0; l < n_layers; ++l) {
        if ((rc = shard_check(ctx, &gate_shards[l], "gate shard")) || (rc = shard_check(ctx, &up_shards[l], "up shard")) ||
            (rc = shard_check(ctx, &down_shards_fm[l], "down shard")) ||
            (rc = resolve_matrix(ctx, &gate_shards[l], &s->gates[l])) || (rc = resolve_matrix(ctx, &up_shards[l], &s->ups[l])) ||
            (rc = resolve_matrix(ctx, &down_shards_fm[l], &s->downs[l]))) {
            delete s;
            return rc;
        }
        if (gate_shards[l].cols != gate_shards[0].cols || row_offset + (size_t)gate_shards[l].rows > n_features_global) {
            delete s;
            return fail(ctx, LQ_REFUSED_SHAPE, "sharded stack: shard geometry");
        }
    }
    s->sharded = true;
    s->batch = batch;
    s->top_k = top_k;
    s->flags = flags | LQ_WALK_RMSNORM | LQ_WALK_RESIDUAL;
    s->hidden = (int)gate_shards[0].cols;
    s->row_offset = row_offset;
    s->cap = cap;
    const size_t H = (size_t)s->hidden, stride = 2 + 2 * cap;
    const size_t hb = a256(batch * H * 4);
    cudaError_t e = cudaMalloc(&s->h_in, 4 * hb);
    uint8_t* raw = nullptr;
    const size_t aux = a256(LQ_HIST_WORDS * 4) + a256(stride * 4) + a256((size_t)ctx->world * stride * 4) + a256(H * 4);
    if (e == cudaSuccess) e = cudaMalloc(&raw, aux);
    if (e == cudaSuccess) e = cudaMemset(raw, 0, aux);
    if (e != cudaSuccess) {
        if (s->h_in) cudaFree(s->h_in);
        if (raw) cudaFree(raw);
        s->h_in = nullptr;
        delete s;
        return cuda_fail(ctx, e, "sharded stack buffers");
    }
    uint8_t* hraw = (uint8_t*)s->h_in;
    s->h_out = (float*)(hraw + hb);
    s->h_buf[0] = (float*)(hraw + 2 * hb);
    s->h_buf[1] = (float*)(hraw + 3 * hb);
    s->hist_buf = (uint32_t*)raw;
    s->pack = (int32_t*)(raw + a256(LQ_HIST_WORDS * 4));
    s->packs = (int32_t*)((uint8_t*)s->pack + a256(stride * 4));
    s->out_partial = (float*)((uint8_t*)s->packs + a256((size_t)ctx->world * stride * 4));
    s->n_global = n_features_global;
    rc = try_xfused(ctx, s);
    if (!rc && s->xfused) {
        // one pass on a harmless input: kernel attributes, module load, and a check that the ranks meet
        cudaMemsetAsync(s->h_in, 0x3f, hb, ctx->stream);
        rc = stack_enqueue(ctx, s);
        if (!rc) rc = lq_synchronize(ctx);
    }
    if (rc) {
        lq_stack_destroy(ctx, s);
        return rc;
    }
    *out = s;
    return LQ_OK;
}

int lq_stack_path(const lq_stack* s) {
    if (!s) return LQ_ERR_ARGUMENT;
    if (s->xfused) return LQ_STACK_PATH_SHARDED_FUSED;
    if (s->sharded) return LQ_STACK_PATH_SHARDED_NCCL;
    return s->fused ? LQ_STACK_PATH_FUSED : LQ_STACK_PATH_GRAPH;
}

void lq_stack_destroy(lq_ctx* ctx, lq_stack* s) {
    DevGuard dev_guard(ctx);
    if (!s) return;
    if (ctx) cudaStreamSynchronize(ctx->stream);
    if (s->exec) cudaGraphExecDestroy(s->exec);
    if (s->graph) cudaGraphDestroy(s->graph);
    if (s->h_in) cudaFree(s->h_in);
    if (s->layers_dev) cudaFree(s->layers_dev);
    if (s->hist_buf) cudaFree(s->hist_buf);
    if (ctx && ctx->last_xstack == s) ctx->last_xstack = nullptr;
    for (size_t r = 0; r < s->areas.size(); ++r)
        if (s->areas[r] && s->areas[r] != s->xarea) cudaIpcCloseMemHandle(s->areas[r]);
    if (s->xfused && ctx && ctx->comm && ctx->world > 1) {
        // an area is freed only after every rank has unmapped it: the ranks destroy a stack together
        if (NcclApi* nc = nccl_api()) {
            nc->AllReduce(s->sync_word, s->sync_word, 1, ncclUint32, ncclSum, ctx->comm, ctx->stream);
            cudaStreamSynchronize(ctx->stream);
        }
    }
    if (s->xarea) cudaFree(s->xarea);
    if (s->xhits) cudaFree(s->xhits);
    delete s;
}

}  // extern "C"
