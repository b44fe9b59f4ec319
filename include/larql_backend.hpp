// C++ host-side mirror of the reference's backend trait for the walk path, over the C ABI in
// larql_cuda.h.  Method names, argument meaning and refusal behaviour follow the Rust traits
//   QuantMatVec  crates/larql-compute/src/backend/quant_matvec.rs:252-427
//   MatMul       crates/larql-compute/src/backend/matmul.rs:207-235
//   ComputeBackend  crates/larql-compute/src/backend/mod.rs:49-144
// with Option<T> rendered as std::optional<T>: a refusal (positive status: shape rule violated,
// format or size unsupported) is std::nullopt, exactly where the trait returns None; a device or
// runtime failure (negative status) and the reference's panic case (NaN score in top_k_by_abs,
// crates/larql-vindex/src/index/compute/gate_knn/mod.rs:47-49) throw BackendError.  There is no CPU
// fallback: constructing the backend without the CUDA library or a device throws.
#pragma once
#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "larql_cuda.h"

namespace larql {

struct BackendError : std::runtime_error {
    int status;
    BackendError(int st, const std::string& what) : std::runtime_error(what), status(st) {}
};

enum class QuantFormat : int { Q4_K = LQ_FMT_Q4_K, Q8_0 = LQ_FMT_Q8_0, MXFP4 = LQ_FMT_MXFP4, NVFP4 = LQ_FMT_NVFP4 };

// A quantised [rows, cols] matrix in host memory (the reference's mmap slices) or, with
// `on_device`, raw device pointers.
struct QuantMatrix {
    QuantFormat fmt = QuantFormat::Q4_K;
    const uint8_t* data = nullptr;
    size_t data_len = 0;
    const uint8_t* scales = nullptr;  // MXFP4 e8m0 / NVFP4 e4m3 stream
    size_t scales_len = 0;
    float tensor_scale = 1.0f;        // NVFP4
    int64_t rows = 0, cols = 0;
    bool on_device = false;

    lq_matrix c() const {
        lq_matrix m;
        m.fmt = static_cast<int>(fmt) | (on_device ? LQ_MAT_DEVICE : 0);
        m.data = data;
        m.data_len = data_len;
        m.scales = scales;
        m.scales_len = scales_len;
        m.tensor_scale = tensor_scale;
        m.rows = rows;
        m.cols = cols;
        return m;
    }
};

struct WalkResult {
    std::vector<float> out;                   // [batch, hidden]
    std::vector<std::vector<uint32_t>> hits;  // selected features per token (order unspecified)
};

class CudaBackend {
public:
    explicit CudaBackend(int device = 0) {
        const int rc = lq_create(device, &ctx_);
        if (rc != LQ_OK || !ctx_) throw BackendError(rc, "lq_create failed: no CUDA device or library (no CPU fallback)");
    }
    ~CudaBackend() {
        if (ctx_) lq_destroy(ctx_);
    }
    CudaBackend(const CudaBackend&) = delete;
    CudaBackend& operator=(const CudaBackend&) = delete;

    // ComputeBackend
    std::string name() const { return "cuda-b200"; }
    std::string device_info() const {
        char buf[256] = {0};
        lq_device_info(ctx_, buf, sizeof buf);
        return buf;
    }
    bool supports_quant(QuantFormat f) const { return lq_supports_quant(ctx_, static_cast<int>(f)) != 0; }
    void register_weight_region(const uint8_t* host, size_t len) { check(lq_register_weight_region(ctx_, host, len)); }
    void seal_weight_regions() { check(lq_seal_weight_regions(ctx_)); }
    void drop_weight_regions() { check(lq_drop_weight_regions(ctx_)); }
    const std::string& last_refusal() const { return last_refusal_; }

    // QuantMatVec::q4k_matvec: out[num_rows] = Q4_K[num_rows, hidden] . x
    std::optional<std::vector<float>> q4k_matvec(const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                                                 size_t num_rows, size_t hidden) {
        std::vector<float> out(num_rows);
        return ok(lq_q4k_matvec(ctx_, w, w_len, x, x_len, num_rows, hidden, out.data(), out.size())) ? std::optional(std::move(out))
                                                                                                     : std::nullopt;
    }
    // QuantMatVec::q4k_matmul: x [seq_len, hidden] -> out [seq_len, num_rows]
    std::optional<std::vector<float>> q4k_matmul(const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                                                 size_t num_rows, size_t hidden, size_t seq_len) {
        std::vector<float> out(num_rows * seq_len);
        return ok(lq_q4k_matmul(ctx_, w, w_len, x, x_len, num_rows, hidden, seq_len, out.data(), out.size()))
                   ? std::optional(std::move(out))
                   : std::nullopt;
    }
    // QuantMatVec::q8_0_gemv
    std::optional<std::vector<float>> q8_0_gemv(const uint8_t* blocks, size_t blocks_len, const float* x, size_t x_len,
                                                size_t n, size_t k) {
        std::vector<float> out(n);
        return ok(lq_q8_0_gemv(ctx_, blocks, blocks_len, x, x_len, n, k, out.data())) ? std::optional(std::move(out))
                                                                                       : std::nullopt;
    }
    // QuantMatVec::nvfp4_gemv
    std::optional<std::vector<float>> nvfp4_gemv(const uint8_t* packed, size_t packed_len, const uint8_t* scales,
                                                 size_t scales_len, float tensor_scale, const float* x, size_t x_len,
                                                 size_t n, size_t k) {
        std::vector<float> out(n);
        return ok(lq_nvfp4_gemv(ctx_, packed, packed_len, scales, scales_len, tensor_scale, x, x_len, n, k, out.data()))
                   ? std::optional(std::move(out))
                   : std::nullopt;
    }
    // MatMul::mxfp4_gemv
    std::optional<std::vector<float>> mxfp4_gemv(const uint8_t* packed, size_t packed_len, const uint8_t* scales,
                                                 size_t scales_len, const float* x, size_t x_len, size_t n, size_t k) {
        std::vector<float> out(n);
        return ok(lq_mxfp4_gemv(ctx_, packed, packed_len, scales, scales_len, x, x_len, n, k, out.data()))
                   ? std::optional(std::move(out))
                   : std::nullopt;
    }
    // MatMul::f16_gemv / bf16_gemv (kind 0 / 1): w holds n*k little-endian 16-bit words
    std::optional<std::vector<float>> gemv16(int kind, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n,
                                             size_t k, bool exact = false) {
        std::vector<float> out(n);
        return ok(lq_gemv16(ctx_, kind, w, w_len, x, x_len, n, k, out.data(), exact ? 1 : 0)) ? std::optional(std::move(out))
                                                                                           : std::nullopt;
    }
    // MatMul::mxfp4_gemv_multi / nvfp4_gemv_multi: several matrices against one input, one submission
    std::optional<std::vector<std::vector<float>>> gemv_multi(const std::vector<QuantMatrix>& mats, const float* x,
                                                              size_t x_len, bool exact = false) {
        std::vector<lq_matrix> cm;
        std::vector<std::vector<float>> outs;
        std::vector<float*> ptrs;
        for (const auto& m : mats) {
            cm.push_back(m.c());
            outs.emplace_back(static_cast<size_t>(m.rows));
        }
        for (auto& o : outs) ptrs.push_back(o.data());
        return ok(lq_gemv_multi(ctx_, cm.data(), cm.size(), x, x_len, ptrs.data(), exact ? 1 : 0)) ? std::optional(std::move(outs))
                                                                                                : std::nullopt;
    }
    // QuantMatVec::q6k_matvec
    std::optional<std::vector<float>> q6k_matvec(const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                                                 size_t num_rows, size_t hidden) {
        std::vector<float> out(num_rows);
        if (!ok(lq_q6k_matvec(ctx_, w, w_len, x, x_len, num_rows, hidden, out.data()))) return std::nullopt;
        return out;
    }
    // QuantMatVec::q4k_dual_matvec: gate and up against one activation
    std::optional<std::pair<std::vector<float>, std::vector<float>>> q4k_dual_matvec(const uint8_t* w_a, size_t wa_len,
                                                                                     const uint8_t* w_b, size_t wb_len,
                                                                                     const float* x, size_t x_len,
                                                                                     size_t num_rows, size_t hidden) {
        std::vector<float> a(num_rows), b(num_rows);
        if (!ok(lq_q4k_dual_matvec(ctx_, w_a, wa_len, w_b, wb_len, x, x_len, num_rows, hidden, a.data(), b.data())))
            return std::nullopt;
        return std::make_pair(std::move(a), std::move(b));
    }
    // QuantMatVec::q4k_matvec_topk: (row, score) sorted by score descending, ties to the lower row
    std::optional<std::vector<std::pair<uint32_t, float>>> q4k_matvec_topk(const uint8_t* w, size_t w_len, const float* x,
                                                                           size_t x_len, size_t num_rows, size_t hidden,
                                                                           size_t top_k) {
        const size_t k = top_k < num_rows ? top_k : num_rows;
        std::vector<uint32_t> idx(k ? k : 1);
        std::vector<float> val(k ? k : 1);
        size_t count = 0;
        if (!ok(lq_q4k_matvec_topk(ctx_, w, w_len, x, x_len, num_rows, hidden, top_k, idx.data(), val.data(), &count)))
            return std::nullopt;
        std::vector<std::pair<uint32_t, float>> r(count);
        for (size_t i = 0; i < count; ++i) r[i] = {idx[i], val[i]};
        return r;
    }
    // top_k_by_abs: (index, signed score) of the top_k largest |score|, ties to the lower index
    std::optional<std::vector<std::pair<uint32_t, float>>> top_k_by_abs(const float* scores, size_t n, size_t top_k) {
        const size_t k = top_k < n ? top_k : n;
        std::vector<uint32_t> idx(k ? k : 1);
        std::vector<float> val(k ? k : 1);
        size_t count = 0;
        if (!ok(lq_topk_abs(ctx_, scores, n, top_k, idx.data(), val.data(), &count))) return std::nullopt;
        std::vector<std::pair<uint32_t, float>> r(count);
        for (size_t i = 0; i < count; ++i) r[i] = {idx[i], val[i]};
        return r;
    }
    // The walk of one layer (walk_ffn_sparse, crates/larql-inference/src/vindex/walk_ffn/sparse.rs:60-306):
    // x [batch, hidden] -> out [batch, hidden] and the selected features of every token.
    std::optional<WalkResult> walk_ffn(const QuantMatrix& gate, const QuantMatrix& up, const QuantMatrix& down_fm,
                                       const float* x, size_t batch, size_t top_k, uint32_t flags) {
        const lq_matrix g = gate.c(), u = up.c(), d = down_fm.c();
        const size_t hidden = static_cast<size_t>(gate.cols), n = static_cast<size_t>(gate.rows);
        const size_t cap = top_k < n ? top_k : n;  // the dense rewrite may select all n features
        WalkResult r;
        r.out.resize(batch * hidden);
        std::vector<uint32_t> idx(batch * (n ? n : 1));
        std::vector<uint32_t> cnt(batch ? batch : 1);
        // idx rows are laid out with the effective K of the call: K itself, or n when K >= 80 % of n
        const bool dense = !(flags & LQ_WALK_FORCE_SPARSE) && top_k >= (n * 4) / 5;
        const size_t stride = dense ? n : cap;
        if (!ok(lq_walk_ffn(ctx_, &g, &u, &d, x, batch, top_k, flags, r.out.data(), idx.data(), cnt.data()))) return std::nullopt;
        r.hits.resize(batch);
        for (size_t t = 0; t < batch; ++t) r.hits[t].assign(idx.begin() + t * stride, idx.begin() + t * stride + cnt[t]);
        return r;
    }

    lq_ctx* raw() const { return ctx_; }

private:
    // status -> Option: 0 Some, positive None (refusal), negative / NaN-score throw
    bool ok(int rc) {
        if (rc == LQ_OK) return true;
        const char* msg = lq_last_error(ctx_);
        if (rc > 0 && rc != LQ_ERR_NAN_SCORE) {
            last_refusal_ = msg ? msg : "";
            return false;
        }
        throw BackendError(rc, msg ? msg : "device error");
    }
    void check(int rc) {
        if (!ok(rc)) throw BackendError(rc, last_refusal_);
    }
    lq_ctx* ctx_ = nullptr;
    std::string last_refusal_;
};

}  // namespace larql
