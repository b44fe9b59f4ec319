/*
 * larql_cuda.h — C ABI of the B200 (sm_100a) backend for LARQL's vindex FFN walk.
 *
 * This is the boundary a `larql-compute-cuda` crate binds (extern "C", plain
 * pointers and sizes).  Every entry point names the reference trait method or
 * function it stands in for (paths relative to the reference repository).
 *
 * Conventions
 *   - Status: 0 = ok.  > 0 = refusal, which the Rust shim maps to `None` ("cannot
 *     compute this": bad geometry, unsupported format) — never a wrong or zero-filled
 *     answer (crates/larql-compute/src/backend/quant_matvec.rs:378-427,
 *     crates/larql-compute/src/cpu/ops/kernel_shape.rs:1-17).  < 0 = device / runtime
 *     error; lq_last_error() has the text.
 *   - Host entry points (lq_*) take HOST pointers.  Weights are long-lived, immutable
 *     byte ranges (mmap slices in the reference, backend/mod.rs:68-89); they are
 *     uploaded once and cached by (address, length) exactly like the reference's GPU
 *     backend does (crates/larql-compute-metal/src/buffers/mod.rs:107-160).
 *     Activations are copied per call; outputs are written to caller memory.
 *   - Device entry points (lq_dev_*) take DEVICE pointers, enqueue on the context's
 *     stream and do not synchronise; call lq_synchronize() to wait and collect errors.
 *   - Device weight pointers are block aligned: 16 bytes for Q4_K and MXFP4 codes, 8 for NVFP4
 *     codes, 2 for Q8_0 blocks (LQ_ERR_ARGUMENT / LQ_REFUSED_UNSUPPORTED otherwise, before any
 *     launch).  Host weight ranges may sit at any address: a range that would land misaligned
 *     inside a registered region is given an aligned device copy of its own.
 *   - Every call makes its context's device current for its duration: one process may hold
 *     contexts on several GPUs.
 *   - There is no CPU fallback anywhere: without a CUDA device lq_create fails.
 *   - A context is used by one thread at a time (the reference serialises device
 *     calls behind a mutex, crates/larql-vindex/src/format/vindex3/opplan/exec/device.rs:39-42).
 */
#ifndef LARQL_CUDA_H
#define LARQL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LQ_API __attribute__((visibility("default")))

typedef struct lq_ctx lq_ctx;

enum lq_status {
    LQ_OK = 0,
    LQ_REFUSED_SHAPE = 1,       /* geometry does not describe the operands (-> None) */
    LQ_REFUSED_UNSUPPORTED = 2, /* no kernel for this format / size (-> None) */
    LQ_ERR_NAN_SCORE = 3,       /* a gate score is NaN: the reference's top_k_by_abs panics */
    LQ_ERR_CUDA = -1,
    LQ_ERR_TIMEOUT = -2,        /* a bounded device-side wait ran out */
    LQ_ERR_ARGUMENT = -3,
};

/* Weight formats (layouts as in the reference):
 *   Q4_K  : 144-byte super-blocks of 256 (crates/larql-models/src/quant/ggml/q4_k.rs:9-21)
 *   Q8_0  : ggml 34-byte blocks of 32    (crates/larql-compute/src/cpu/kquant_gemv.rs:1-10)
 *   MXFP4 : packed [rows,K/32,16] + e8m0 scales [rows,K/32] (crates/larql-models/src/quant/mxfp4.rs:1-9)
 *   NVFP4 : packed [rows,K/16,8] + e4m3 scales [rows,K/16] + f32 tensor scale
 *           (crates/larql-models/src/quant/nvfp4.rs:24-36)                              */
enum lq_format { LQ_FMT_Q4_K = 0, LQ_FMT_Q8_0 = 1, LQ_FMT_MXFP4 = 2, LQ_FMT_NVFP4 = 3, LQ_FMT_Q6_K = 4 };
/* OR-ed into lq_matrix.fmt: data/scales are DEVICE pointers already (resident weights handed to
 * a host-pointer entry point; activations and outputs stay host memory). */
#define LQ_MAT_DEVICE 0x100

typedef struct lq_matrix {
    int32_t fmt;          /* enum lq_format */
    const void* data;     /* blocks (Q4_K/Q8_0) or packed codes (MXFP4/NVFP4) */
    size_t data_len;      /* bytes */
    const void* scales;   /* MXFP4/NVFP4 scale stream, else NULL */
    size_t scales_len;
    float tensor_scale;   /* NVFP4 only */
    int64_t rows, cols;
} lq_matrix;

/* Walk flags. */
#define LQ_WALK_RMSNORM 1u      /* input is the raw residual: RMS-normalise it first (unit weight,
                                   eps 1e-6; crates/larql-compute/src/residual.rs:56-78) */
#define LQ_WALK_RESIDUAL 2u     /* out = input + walk(...)  (run_ffn,
                                   crates/larql-compute/src/forward/layer.rs:109-124) */
#define LQ_WALK_FORCE_SPARSE 4u /* keep the sparse walk even when K >= 80% of the features
                                   (WalkFfnConfig::force_walk; default rewrites to dense,
                                   crates/larql-inference/src/vindex/walk_ffn/helpers.rs:18-30) */

/* ---- context ----------------------------------------------------------------- */
/* BackendCtor for BackendKind::Cuda (crates/larql-compute/src/backend/factory.rs:127-130):
 * a non-zero return means "no device" and the registry entry yields None. */
LQ_API int lq_create(int device, lq_ctx** out);
LQ_API void lq_destroy(lq_ctx* ctx);
/* Text of the last failure on this context ("" if none). */
LQ_API const char* lq_last_error(lq_ctx* ctx);
/* ComputeBackend::device_info (backend/mod.rs:54-56). */
LQ_API int lq_device_info(lq_ctx* ctx, char* buf, size_t cap);
/* QuantMatVec::supports_quant (backend/quant_matvec.rs:367-370): 1 or 0. */
LQ_API int lq_supports_quant(lq_ctx* ctx, int fmt);
/* Waits for the context's stream and reports any device-side error recorded since the last call. */
LQ_API int lq_synchronize(lq_ctx* ctx);
/* The context's cudaStream_t (for callers that enqueue their own work around lq_dev_* calls). */
LQ_API void* lq_stream(lq_ctx* ctx);
/* MatMul::submission_clock (backend/matmul.rs:209-218; the SubmissionClock it returns: 25-42): kernel launches
 * issued by this context. */
LQ_API uint64_t lq_launch_count(lq_ctx* ctx);

/* ---- weight residency ---------------------------------------------------------- */
/* ComputeBackend::register_weight_region / seal_weight_regions (backend/mod.rs:68-89) and
 * MatMul::wire_resident (backend/matmul.rs:207): upload a host byte range once.  Any later
 * host-pointer call whose weight slice lies inside a registered range uses the device copy. */
LQ_API int lq_register_weight_region(lq_ctx* ctx, const void* host, size_t len);
LQ_API int lq_seal_weight_regions(lq_ctx* ctx);
LQ_API int lq_drop_weight_regions(lq_ctx* ctx);
/* Device address of a registered host range (NULL if not resident). */
LQ_API const void* lq_device_ptr(lq_ctx* ctx, const void* host, size_t len);

/* ---- dense quantised matvec / matmul (host pointers) --------------------------- */
/* QuantMatVec::q4k_matvec (backend/quant_matvec.rs:252-260) -> CpuBackend::q4k_matvec
 * (crates/larql-compute/src/cpu/mod.rs:95-114).  Shape rule = KernelShapeError::check:
 * out_len == num_rows, x_len == hidden, hidden % 256 == 0, w_len >= needed. */
LQ_API int lq_q4k_matvec(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                         size_t num_rows, size_t hidden, float* out, size_t out_len);
/* QuantMatVec::q4k_matmul (backend/quant_matvec.rs:324-333): x [seq,hidden] -> out [seq,num_rows]. */
LQ_API int lq_q4k_matmul(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                         size_t num_rows, size_t hidden, size_t seq_len, float* out, size_t out_len);
/* The same matvec in the reference's exact f32 order (bit-identical to the CPU backend);
 * slower, used to resolve top-K boundary cases and by the parity tests.  No trait counterpart. */
LQ_API int lq_q4k_matvec_exact(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len,
                               size_t num_rows, size_t hidden, float* out, size_t out_len);

/* Dense gemv of one block-format matrix (any of the four formats): out[n] = W[n,k] . x[k].
 * exact = 0: fast path (integer / table dots, error within the bound the walk uses);
 * exact = 1: the CPU backend's f32 order, bit-identical to q8_0_gemv
 * (crates/larql-compute/src/cpu/kquant_gemv.rs:67-109), nvfp4_gemv (cpu/nvfp4_gemv.rs:29-65), the
 * MXFP4 test loop (crates/larql-vindex/src/format/vindex3/opplan/exec/tests/device.rs:105-127) and
 * q4k_matvec.  Refuses (LQ_REFUSED_SHAPE) where those return None. */
LQ_API int lq_gemv(lq_ctx* ctx, const lq_matrix* m, const float* x, size_t x_len, float* out, size_t out_len,
                   int exact);
/* q8_0_gemv (crates/larql-compute/src/cpu/kquant_gemv.rs:67-109; the reference calls it directly, no
 * trait method carries ggml Q8_0 with f32 activations): blocks [n, k/32, 34]. */
LQ_API int lq_q8_0_gemv(lq_ctx* ctx, const uint8_t* blocks, size_t blocks_len, const float* x, size_t x_len, size_t n,
                        size_t k, float* out);
/* MatMul::mxfp4_gemv (backend/matmul.rs:226-235): packed [n, k/2], e8m0 scales [n, k/32]. */
LQ_API int lq_mxfp4_gemv(lq_ctx* ctx, const uint8_t* packed, size_t packed_len, const uint8_t* scales,
                         size_t scales_len, const float* x, size_t x_len, size_t n, size_t k, float* out);
/* MatMul::nvfp4_gemv (backend/matmul.rs:263-273) -> cpu/nvfp4_gemv.rs:29-65: packed [n, k/2], e4m3 scales
 * [n, k/16], one f32 tensor scale. */
LQ_API int lq_nvfp4_gemv(lq_ctx* ctx, const uint8_t* packed, size_t packed_len, const uint8_t* scales,
                         size_t scales_len, float tensor_scale, const float* x, size_t x_len, size_t n, size_t k,
                         float* out);

/* Several block-format matrices against ONE input vector, one submission (the input is uploaded once, the
 * call waits once): MatMul::mxfp4_gemv_multi / nvfp4_gemv_multi (backend/matmul.rs:242-251, 279-286) as
 * DevicePlanBackend calls them (crates/larql-vindex/src/format/vindex3/opplan/exec/device.rs:256-341).  Every
 * matrix's cols must equal x_len; outs[i] receives rows_i floats.  Results are those of the single gemvs. */
LQ_API int lq_gemv_multi(lq_ctx* ctx, const lq_matrix* mats, size_t n_mats, const float* x, size_t x_len,
                         float* const* outs, int exact);
LQ_API int lq_mxfp4_gemv_multi(lq_ctx* ctx, const lq_matrix* mats, size_t n_mats, const float* x, size_t x_len,
                               float* const* outs);
LQ_API int lq_nvfp4_gemv_multi(lq_ctx* ctx, const lq_matrix* mats, size_t n_mats, const float* x, size_t x_len,
                               float* const* outs);

/* Dense gemv over f16 (kind 0) or bf16 (kind 1) weights [n, k], little-endian 16-bit words:
 * MatMul::f16_gemv(_force) / bf16_gemv(_force) / f16_gemv_multi / bf16_gemv_multi (backend/matmul.rs:124-205).
 * Refuses (LQ_REFUSED_SHAPE) when w_len < n*k*2 or x_len != k.  exact = 1: one running f32 sum per row, k
 * ascending, the loop of the reference's test device (…/opplan/exec/tests/device.rs:68-84; the CPU backend has
 * no f16 / bf16 gemv of its own); exact = 0: warp-per-row tree sum (any order, f32). */
LQ_API int lq_gemv16(lq_ctx* ctx, int kind, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n,
                     size_t k, float* out, int exact);
LQ_API int lq_gemv16_multi(lq_ctx* ctx, int kind, size_t n_mats, const uint8_t* const* ws, const size_t* w_lens,
                           const size_t* ns, size_t k, const float* x, size_t x_len, float* const* outs, int exact);
LQ_API int lq_f16_gemv(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n, size_t k,
                       float* out);
LQ_API int lq_bf16_gemv(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n, size_t k,
                        float* out);

/* Q6_K (210-byte super-blocks of 256; rows need 2-byte alignment).  A walk takes Q6_K for any of gate / up /
 * down beside Q4_K (the Ollama convention keeps down as Q6_K): the gate is scanned in the backend matvec's
 * order, up and down rows go through the per-format row functions (crates/larql-vindex/src/quant/registry.rs;
 * q6k_row_dot / q6k_row_scaled_add, crates/larql-models/src/quant/ggml/q6_k.rs:44-168).
 *   lq_q6k_matvec     QuantMatVec::q6k_matvec (backend/quant_matvec.rs:336-344); arithmetic and order of
 *                     crates/larql-compute/src/cpu/ops/q6k_matvec.rs:45-96 (bit-identical)
 *   lq_dequantize_q6k dequantize_q6_k (crates/larql-models/src/quant/ggml/q6_k.rs:171-195)
 *   lq_q4k_dual_matvec QuantMatVec::q4k_dual_matvec (backend/quant_matvec.rs:287-296): gate and up against one
 *                     activation in one launch; order of crates/larql-compute/src/cpu/ops/q4_common/dual.rs:22-167 (one
 *                     running sum per row; bit-identical) */
LQ_API int lq_q6k_matvec(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                         size_t hidden, float* out);
LQ_API int lq_dequantize_q6k(lq_ctx* ctx, const uint8_t* data, size_t data_len, size_t n_elems, float* out);
LQ_API int lq_q4k_dual_matvec(lq_ctx* ctx, const uint8_t* w_a, size_t wa_len, const uint8_t* w_b, size_t wb_len,
                              const float* x, size_t x_len, size_t num_rows, size_t hidden, float* out_a, float* out_b);

/* ---- on-disk K-quant FFN weights of a vindex directory (host only; needs no context) ----------------
 * interleaved_kquant.bin + interleaved_kquant_manifest.json hold, per layer, gate [features, padded hidden],
 * up [features, padded hidden] and down [hidden, padded features] as Q4_K / Q6_K
 * (write_interleaved_ffn_kquant, crates/larql-vindex/src/format/weights/write_kquant/ffn.rs:25-117; read by
 * load_interleaved_kquant, crates/larql-vindex/src/index/storage/ffn_store/interleaved_kquant.rs:64-106);
 * down_features_kquant.bin + manifest hold the feature-major down [padded features, padded hidden] the walk
 * wants (crates/larql-vindex/src/format/weights/write_kquant/feature_major_down.rs:48-104; read by
 * load_down_features_q4k, crates/larql-vindex/src/index/storage/ffn_store/interleaved_kquant.rs:115-159).  The legacy
 * file names (interleaved_q4k.bin, down_features_q4k.bin) are looked for second.  Rows are padded to whole
 * 256-element super-blocks (k_quant_padded_cols, crates/larql-models/src/quant/ggml/mod.rs:105-114), so a
 * matrix's `cols` is the padded width: a caller pads its activation with zeros to that width.
 *   lq_vindex_open    maps the files read-only and checks every manifest entry (format known to the registry,
 *                     shape, length, range); *out is NULL and err holds the reason on any refusal
 *   lq_vindex_layer   the layer's matrices, pointing into the mappings (valid until lq_vindex_close);
 *                     down_fm->fmt = -1 when the directory has no feature-major sidecar
 *   lq_nvfp4_pack_split  the three regions {codes | scales | f32 tensor scale} of a stored NVFP4 tensor
 *                     (PackLayout::derive and split, crates/larql-vindex/src/format/vindex3/represent/nvfp4_pack.rs:43-164) */
typedef struct lq_vindex lq_vindex;
LQ_API size_t lq_k_quant_padded_cols(size_t cols);
LQ_API int lq_vindex_open(const char* dir, lq_vindex** out, char* err, size_t err_cap);
LQ_API size_t lq_vindex_num_layers(const lq_vindex* v);
LQ_API int lq_vindex_layer(const lq_vindex* v, size_t layer, lq_matrix* gate, lq_matrix* up, lq_matrix* down,
                           lq_matrix* down_fm);
LQ_API void lq_vindex_close(lq_vindex* v);
LQ_API int lq_nvfp4_pack_split(const uint8_t* bytes, size_t len, size_t rows, size_t k, lq_matrix* out);

/* LM-head style scan + top-k: QuantMatVec::q4k_matvec_topk (backend/quant_matvec.rs:268-277) and
 * MatMul::f16_gemv_topk (backend/matmul.rs:100-109).  Up to top_k (row, score) pairs sorted by score
 * descending, ties to the lower row; *count = min(top_k, rows).  Scores are computed in the reference
 * order (q4k_matvec's / the f16 loop's), so the rows are the ones the caller's fallback (full matvec + CPU
 * reduce) would pick.  top_k <= 16384.  LQ_ERR_NAN_SCORE if a score is NaN. */
LQ_API int lq_q4k_matvec_topk(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t num_rows,
                              size_t hidden, size_t top_k, uint32_t* idx_out, float* val_out, size_t* count);
LQ_API int lq_gemv16_topk(lq_ctx* ctx, int kind, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n,
                          size_t k, size_t top_k, uint32_t* idx_out, float* val_out, size_t* count);
LQ_API int lq_f16_gemv_topk(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t x_len, size_t n,
                            size_t k, size_t top_k, uint32_t* idx_out, float* val_out, size_t* count);

/* MoE routing (crates/larql-compute/src/cpu/ops/moe/math.rs:130-164, mod.rs:127-189): per token a
 * max-subtracted softmax over n_experts logits, the top_k experts by probability (ties to the lower
 * index, descending), weights renormalised over the selected when renormalise != 0.
 * logits [n_tokens, n_experts]; idx_out, w_out [n_tokens, min(top_k, n_experts)].  n_experts <= 256. */
LQ_API int lq_moe_route(lq_ctx* ctx, const float* logits, size_t n_tokens, size_t n_experts, size_t top_k,
                        int renormalise, uint32_t* idx_out, float* w_out);

/* top_k_by_abs (crates/larql-vindex/src/index/compute/gate_knn/mod.rs:50-108): the top_k largest
 * |score|, ties to the lower index, sorted by |score| descending then index.  *count = min(top_k, n).
 * LQ_ERR_NAN_SCORE if a score is NaN. */
LQ_API int lq_topk_abs(lq_ctx* ctx, const float* scores, size_t n, size_t top_k, uint32_t* idx_out,
                       float* val_out, size_t* count);

/* rms_norm_eps with unit weight (crates/larql-compute/src/residual.rs:56-78): x,out [rows,cols]. */
LQ_API int lq_rms_norm(lq_ctx* ctx, const float* x, size_t rows, size_t cols, double eps, float* out);

/* Block decoders on the device, for the bit-exact weight check: dequantize_q4_k
 * (crates/larql-models/src/quant/ggml/q4_k.rs:286-338), dequantize_q8_0 (ggml/legacy.rs:68-83),
 * mxfp4::dequantize_expert (quant/mxfp4.rs:42-95), nvfp4::dequantize_into (quant/nvfp4.rs:192-222).
 * out holds rows*cols floats. */
LQ_API int lq_dequantize(lq_ctx* ctx, const lq_matrix* m, float* out, size_t out_len);

/* ---- the walk (host pointers) --------------------------------------------------- */
/* One FFN layer for `batch` tokens: gate scan -> top-K by |score| -> SiLU-gated up/down
 * accumulate; WalkFfn::forward (crates/larql-inference/src/vindex/walk_ffn/mod.rs:535-542) ->
 * walk_ffn_sparse (…/walk_ffn/sparse.rs:60-306).  gate, up: [features, hidden];
 * down_fm: feature-major [features, hidden] (…/write_kquant/feature_major_down.rs:46-90).
 * x, out: [batch, hidden].  idx_out (optional): [batch, min(top_k, features)] selected feature
 * ids per token, in no particular order (the SET is the reference's); count_out (optional):
 * hits per token. */
LQ_API int lq_walk_ffn(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down_fm,
                       const float* x, size_t batch, size_t top_k, uint32_t flags, float* out,
                       uint32_t* idx_out, uint32_t* count_out);

/* ---- device-pointer variants (async on the context's stream) --------------------- */
LQ_API int lq_dev_q4k_matvec(lq_ctx* ctx, const uint8_t* w, size_t w_len, const float* x, size_t num_rows,
                             size_t hidden, float* out);
LQ_API int lq_dev_walk_ffn(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down_fm,
                           const float* x, size_t batch, size_t top_k, uint32_t flags, float* out,
                           uint32_t* idx_out, uint32_t* count_out);

/* A stack of walk layers run back to back on the device, h <- h + walk_l(rmsnorm(h)) for
 * l = 0..n_layers (run_ffn per layer, forward/layer.rs:61-127), replayed from a CUDA graph.
 * Matrices are DEVICE resident.  h_in/h_out: [batch, hidden] device pointers. */
typedef struct lq_stack lq_stack;
LQ_API int lq_stack_create(lq_ctx* ctx, const lq_matrix* gates, const lq_matrix* ups, const lq_matrix* downs_fm,
                           size_t n_layers, size_t batch, size_t top_k, uint32_t flags, lq_stack** out);
LQ_API int lq_stack_run(lq_ctx* ctx, lq_stack* stack, const float* h_in, float* h_out);
/* The same with HOST residuals: one upload, every layer on the device, one download; returns when
 * h_out_host is written (device or NaN-score errors come back as the status). */
LQ_API int lq_stack_run_host(lq_ctx* ctx, lq_stack* stack, const float* h_in_host, float* h_out_host);
LQ_API void lq_stack_destroy(lq_ctx* ctx, lq_stack* stack);

/* quantize_q4_k (crates/larql-compute/src/cpu/ops/q4_common/quantize.rs:89-189) on the device:
 * src [n_elems] f32 (n_elems % 256 == 0) -> dst [n_elems/256*144] bytes, byte-identical to the CPU
 * encoder.  Device pointers, dst 16-byte aligned.  Builds synthetic layers directly in HBM. */
LQ_API int lq_dev_quantize_q4k(lq_ctx* ctx, const float* src, size_t n_elems, uint8_t* dst);

/* One token of lq_dev_walk_ffn with CUDA events between the phases; ms[6] receives the device
 * time of {prepare, gate scan, select, exact re-score + final pick, gather, finish}.  Synchronises.
 * No trait counterpart (the reference's equivalent is PhaseTimingsHandle,
 * crates/larql-inference/src/vindex/walk_ffn/timings.rs:12-33). */
LQ_API int lq_profile_walk(lq_ctx* ctx, const lq_matrix* gate, const lq_matrix* up, const lq_matrix* down_fm,
                           const float* x, size_t top_k, uint32_t flags, float* out, float* ms);

/* Diagnostics of the last walk on this context (token 0): rows certainly selected, rows in the
 * boundary band that were re-scored exactly, threshold and error bound. */
typedef struct lq_walk_stats {
    int32_t n_certain, n_band, n_hits, need;
    float tau, bound;
} lq_walk_stats;
LQ_API int lq_last_walk_stats(lq_ctx* ctx, lq_walk_stats* out);

/* Phase times (microseconds, CTA 0, last layer but one when the launch covers several) of the last
 * fused persistent walk, 13 values: prepare, scan, barrier A, threshold + classify, re-score,
 * gather, wait for barrier B, pick, gather of band winners, merge, barrier C, finish, barrier D.
 * The reference's counterpart is PhaseTimingsHandle (crates/larql-inference/src/vindex/walk_ffn/timings.rs:12-33). */
LQ_API int lq_fused_phase_us(lq_ctx* ctx, float* us, size_t n);

/* ---- feature-sharded walk over the GPUs of one box (device pointers, one token) --------------
 * The reference shards layers or experts over HTTP/gRPC (docs/ffn/distributed.md:14-40) and has no
 * feature sharding; these three steps sit between the caller's collectives (NCCL over NVLink):
 *   scan     -> all-reduce(sum) of hist_buf [LQ_HIST_BINS + 64] u32
 *   classify -> all-gather of pack [2 + 2*cap] i32 per rank
 *   gather   -> all-reduce(sum) of out_partial [hidden] f32 (the caller adds the residual).
 * Each rank passes its contiguous row range [row_offset, row_offset + rows) of gate / up / down and
 * the GLOBAL top_k; the union of the ranks' selections is the unsharded reference's top-K set. */
#define LQ_HIST_WORDS (16384 + 64)
LQ_API int lq_dev_shard_scan(lq_ctx* ctx, const lq_matrix* gate_shard, const float* x, uint32_t flags, int rank,
                             int world, uint32_t* hist_buf);
LQ_API int lq_dev_shard_classify(lq_ctx* ctx, const lq_matrix* gate_shard, uint32_t* hist_buf, int world,
                                 size_t top_k, size_t row_offset, int32_t* pack, size_t cap);
LQ_API int lq_dev_shard_gather(lq_ctx* ctx, const lq_matrix* up_shard, const lq_matrix* down_shard,
                               const int32_t* packs, int world, int rank, size_t cap, size_t top_k,
                               size_t row_offset, float* out_partial);

/* The same protocol run by the library itself: one NCCL communicator per context, the three exchanges
 * enqueued on the context's stream between the device steps (no host round trip per layer).
 *   lq_comm_unique_id   rank 0 makes the 128-byte id and hands it to the other ranks by any channel
 *   lq_comm_init        every rank, collectively (ncclCommInitRank); one rank = one context = one GPU
 *   lq_stack_create_sharded   this rank's row range [row_offset, row_offset + rows) of every layer's gate / up /
 *                       feature-major down, the GLOBAL top_k and feature count; cap = band rows a rank can publish
 *                       per token (a band that does not fit fails the token on every rank: LQ_ERR_CUDA)
 * lq_stack_run / lq_stack_run_host then run h <- h + walk_l(rmsnorm(h)) over all layers on every rank; all ranks
 * call them in the same order and receive the same h.  libnccl.so.2 is loaded on the first of these calls.
 *
 * With one process per GPU, Q4_K layers of one shape and up to 8 ranks, a sharded stack runs on the fused
 * persistent kernel (LQ_STACK_PATH_SHARDED_FUSED): each rank's kernel walks all layers in one launch and the
 * ranks exchange histogram, band rows and partial outputs through each other's memory (CUDA IPC mappings,
 * ordinary peer stores, flag barriers with bounded waits); NCCL then only carries the set-up records and a
 * one-word rendezvous before each launch.  Otherwise (other formats, ranks that cannot map each other's
 * memory, LARQL_B200_SHARDED_NCCL set) the three exchanges per layer are NCCL collectives
 * (LQ_STACK_PATH_SHARDED_NCCL).  All ranks take the same path, and create and destroy a stack together. */
LQ_API int lq_comm_unique_id(void* id_out, size_t cap);
LQ_API int lq_comm_init(lq_ctx* ctx, int rank, int world, const void* unique_id, size_t id_len);
LQ_API int lq_comm_destroy(lq_ctx* ctx);
LQ_API int lq_stack_create_sharded(lq_ctx* ctx, const lq_matrix* gate_shards, const lq_matrix* up_shards,
                                   const lq_matrix* down_shards_fm, size_t n_layers, size_t batch, size_t top_k,
                                   size_t n_features_global, size_t row_offset, uint32_t flags, size_t cap,
                                   lq_stack** out);

/* Which implementation a stack runs on (lq_stack_create picks by shape, format and batch). */
#define LQ_STACK_PATH_GRAPH 0          /* one CUDA graph of per-layer kernels */
#define LQ_STACK_PATH_FUSED 1          /* one persistent kernel per token (Q4_K, batch 1) */
#define LQ_STACK_PATH_SHARDED_NCCL 2   /* per-layer kernels with three NCCL exchanges per layer */
#define LQ_STACK_PATH_SHARDED_FUSED 3  /* one persistent kernel per token and rank, exchange in peer memory */
LQ_API int lq_stack_path(const lq_stack* stack);

/* The rows this rank selected in its last lq_dev_shard_gather or in the last layer of its last sharded stack run, LOCAL to its shard (add the shard's row
 * offset for global rows), unordered; *count is their number, at most cap of them are copied to the host. */
LQ_API int lq_dev_shard_hits(lq_ctx* ctx, uint32_t* idx_out_host, size_t cap, size_t* count);

/* MoE expert walk (cpu_moe_forward's combine, crates/larql-compute/src/cpu/ops/moe/forward.rs:24-140,
 * over walked experts): out[t] = sum_j w[t,j] * walk(expert idx[t,j], x[t]) with lq_moe_route's
 * selection and lq_walk_ffn's per-expert top_k.  gates/ups/downs_fm: n_experts matrices each.
 * flags: LQ_WALK_FORCE_SPARSE only.  expert_idx_out / expert_w_out may be NULL.
 * Experts of one block format (Q8_0 / MXFP4 / NVFP4) and one shape are walked for all (token, expert) pairs at
 * once, the experts' matrices reached through a table on the device and nothing read back between routing and
 * the result; Q4_K / Q6_K experts and experts of different shapes pair by pair after one read-back of the routing.
 * The results are the same either way (the experts' outputs are combined in selection order). */
LQ_API int lq_moe_walk_ffn(lq_ctx* ctx, const lq_matrix* gates, const lq_matrix* ups, const lq_matrix* downs_fm,
                           size_t n_experts, const float* logits, const float* x, size_t batch, size_t top_e,
                           int renormalise, size_t top_k, uint32_t flags, float* out, uint32_t* expert_idx_out,
                           float* expert_w_out);

/* ---- allocation-free entry point ---------------------------------------------------- */
/* Has no counterpart in the reference.  A Q4_K matvec (same arithmetic and kernels as
 * lq_dev_q4k_matvec) for hosts that must not allocate device memory while running: processes
 * that gave all free HBM to their own pools at start-up, plugins under a framework allocator
 * that forbids raw cudaMalloc, loops that cannot take cudaMalloc's device-wide synchronisation.
 * It needs no context and calls no cudaMalloc / cudaFree: its scratch (the prepared activation)
 * is a fixed 128 KiB array inside the library's device image, one per GPU, kept until exit.
 *   - w, x, out are DEVICE pointers (w 16-byte aligned); out[num_rows] = Q4_K[num_rows, hidden] . x.
 *   - hidden must be a multiple of 256 and at most 16384 (LQ_REFUSED_UNSUPPORTED beyond that,
 *     with the reason in errbuf).
 *   - Enqueues on `stream` (a cudaStream_t, NULL = default stream), then waits for it: the
 *     result is ready on return.
 *   - The first call on a device looks up the array's device address; make that call outside
 *     any stream capture.
 *   - All calls on a GPU share the one array (it keeps the previous call's contents; the call
 *     clears what must start at zero): calls that overlap on the same GPU race, serialise them.
 *   - errbuf (optional, errcap bytes) receives the text of a failure. */
LQ_API int lq_q4k_matvec_static(const uint8_t* w, size_t w_len, const float* x, size_t num_rows, size_t hidden,
                                float* out, void* stream, char* errbuf, size_t errcap);

#ifdef __cplusplus
}
#endif
#endif /* LARQL_CUDA_H */
