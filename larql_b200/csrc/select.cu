// Selection kernels: threshold + band classification of the fast gate scores, the
// final pick kernel, and the stand-alone sorted top-K by |score|.
#include "select.cuh"

#include <cstdlib>

namespace lq {

namespace {

constexpr int SEL_T = 1024;
constexpr int SEL_SMEM_VALS_MAX = 40 * 1024;  // floats cached in shared memory (160 KB)

// Classifies every row of one token against the K-th largest fast |score| tau and
// the error bound B = max_r bounds[r]:
//   |s| >  tau + 2B  -> certainly in the reference's top-K        (hit list, ascending)
//   |s| >= tau - 2B  -> membership depends on the reference bits  (band list, ascending)
//   else             -> certainly out.
// Proof sketch: |s_ref - s| <= B for every row, so a row above tau + 2B beats, in
// reference scores, every row at or below tau (fewer than K rows are above tau); a
// row below tau - 2B is beaten by the >= K rows at or above tau.
__global__ void __launch_bounds__(SEL_T, 1)
select_kernel(const float* __restrict__ scores, int n, int top_k, TokenWs ws, int* err, int use_smem, size_t ws_stride) {
    ws = ws_at(ws, ws_stride * blockIdx.y);  // (batched launches: workspace blockIdx.y, a constant stride apart)
    scores = tok_off(scores, ws_stride * blockIdx.y);
    extern __shared__ __align__(16) float s_vals[];
    __shared__ SelectSmem<SEL_T> sm;
    __shared__ float s_red[SEL_T / 32];
    __shared__ int s_nan;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_nan = 0;
    __syncthreads();

    float bmax = 0.0f;
    bool nan = false;
    for (int i = tid; i < n; i += SEL_T) {
        const float v = scores[i];
        nan |= (v != v);
        if (use_smem) s_vals[i] = v;
    }
    for (int o = 16; o > 0; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
    if (lane == 0) s_red[warp] = bmax;
    if (nan) s_nan = 1;
    __syncthreads();
    if (warp == 0) {
        float t = s_red[lane];
        for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
        if (lane == 0) sm.fbcast[0] = t;
    }
    __syncthreads();
    const float B = sm.fbcast[0];
    if (s_nan) set_err(err, DEV_ERR_NAN_SCORE);
    const float* vals = use_smem ? s_vals : scores;

    if (top_k <= 0 || n <= 0) {
        if (tid == 0) *ws.sel = SelHeader{0, 0, 0, 0, 0.0f, B, 0, 0};
        return;
    }
    if (top_k >= n) {
        for (int i = tid; i < n; i += SEL_T) {
            ws.hit_idx[i] = (uint32_t)i;
            ws.hit_score[i] = vals[i];
        }
        if (tid == 0) *ws.sel = SelHeader{n, 0, n, 0, 0.0f, B, 0, 0};
        return;
    }

    uint32_t tau_key;
    int cnt_gt, need_eq;
    block_kth_largest<SEL_T>(vals, n, top_k, sm, tau_key, cnt_gt, need_eq);
    const float tau = __uint_as_float(tau_key);
    const float two_b = __fmul_ru(2.0f, B);
    const float hi = __fadd_ru(tau, two_b), lo = __fadd_rd(tau, -two_b);

    int na, nb;
    block_compact2<SEL_T>(
        n, sm, n,
        [&](int i) {
            const float a = fabsf(vals[i]);
            return a > hi ? 1 : (a >= lo ? 2 : 0);
        },
        [&](int pos, int i) {
            ws.hit_idx[pos] = (uint32_t)i;
            ws.hit_score[pos] = vals[i];
        },
        [&](int pos, int i) {
            ws.band_idx[pos] = (uint32_t)i;
            ws.band_exact[pos] = vals[i];  // replaced by the exact score when a re-score runs
        },
        na, nb);
    if (tid == 0) *ws.sel = SelHeader{na, nb, top_k, top_k - na, tau, B, 0, 0};
}

// Walk-path classification from the coarse histogram the scan kernel filled: the bucket
// [t_lo, t_hi) that holds the K-th largest fast |score| is found with one suffix scan
// over the bins; with B the scan's bound on |fast - reference| per row,
//   |s| >  t_hi + 2B  -> certainly in the reference's top-K   (fewer than K rows reach t_hi)
//   |s| >= t_lo - 2B  -> needs the reference's exact score    (band)
//   else              -> certainly out                        (at least K rows reach t_lo).
// The histogram and the bound word are cleared for the next scan.
__global__ void __launch_bounds__(SEL_T, 1)
classify_kernel(const float* __restrict__ scores_g, int n, int top_k, TokenWs ws, int* err, int use_smem,
                size_t ws_stride) {
    ws = ws_at(ws, ws_stride * blockIdx.y);
    scores_g = tok_off(scores_g, ws_stride * blockIdx.y);
    extern __shared__ __align__(16) float s_vals[];
    __shared__ SelectSmem<SEL_T> sm;
    __shared__ uint32_t s_wsum[SEL_T / 32];
    constexpr int PER = LQ_HIST_BINS / SEL_T;  // bins per thread, contiguous
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // top_k above the number of counted scores (a shard step called with the global K): no bin holds the K-th
    // score; bin 0 then makes every row a candidate, which is the "take all" answer
    if (tid == 0) sm.bcast[0] = 0;
    // stage the scores in shared memory (independent loads), so the two compaction passes
    // do not pay a global-memory round trip per element
    if (use_smem)
        for (int i = tid; i < n; i += SEL_T) s_vals[i] = scores_g[i];
    const float* scores = use_smem ? s_vals : scores_g;
    uint32_t bins[PER];
    uint32_t own = 0;
#pragma unroll
    for (int b = 0; b < PER; ++b) {
        bins[b] = ws.hist[tid * PER + b];
        own += bins[b];
        ws.hist[tid * PER + b] = 0;
    }
    // inclusive suffix sum over threads (higher thread = larger keys)
    uint32_t suf = own;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += v;
    }
    if (lane == 0) s_wsum[warp] = suf;
    __syncthreads();
    uint32_t higher = 0;
    for (int w = warp + 1; w < SEL_T / 32; ++w) higher += s_wsum[w];
    suf += higher;
    const uint32_t above = suf - own;
    if (above < (uint32_t)top_k && (uint32_t)top_k <= suf) {
        uint32_t acc = above;
        int b = PER - 1;
        for (; b >= 0; --b) {
            if (acc + bins[b] >= (uint32_t)top_k) break;
            acc += bins[b];
        }
        sm.bcast[0] = tid * PER + b;
    }
    __syncthreads();
    const uint32_t bstar = (uint32_t)sm.bcast[0];
    const float B = __uint_as_float(ws.sel->bound_bits);
    const float t_lo = __uint_as_float(bstar << LQ_HIST_SHIFT);
    const uint32_t hi_bits = (bstar + 1u) << LQ_HIST_SHIFT;
    const float t_hi = __uint_as_float(hi_bits > 0x7F800000u ? 0x7F800000u : hi_bits);
    const float two_b = __fmul_ru(2.0f, B);
    const float hi = __fadd_ru(t_hi, two_b), lo = __fadd_rd(t_lo, -two_b);
    __syncthreads();
    int na, nb;
    block_compact2<SEL_T>(
        n, sm, n,
        [&](int i) {
            const float a = fabsf(scores[i]);
            return a > hi ? 1 : (a >= lo ? 2 : 0);
        },
        [&](int pos, int i) {
            ws.hit_idx[pos] = (uint32_t)i;
            ws.hit_score[pos] = scores[i];
        },
        [&](int pos, int i) { ws.band_idx[pos] = (uint32_t)i; }, na, nb);
    if (tid == 0) *ws.sel = SelHeader{na, nb, top_k, top_k - na, t_lo, B, 0, 0u};
    (void)err;
}

// ---- the same classification by several CTAs per token ------------------------------------------
// One CTA needs some 30 us to compact 28672 scores in order.  Here MC_MAX_CTAS CTAs share a token: every CTA finds
// the threshold bucket from the histogram (the same answer everywhere), counts the certainly-in and the band rows
// of ITS contiguous chunk of rows (first launch), and, once all counts are known, writes them at the offsets the
// counts of the chunks before it give (second launch): the lists come out in ascending row order, exactly as one
// CTA writes them.  Counts and thresholds travel in the spare words of the token's selection page.
constexpr int MC_T = 256;
constexpr int MC_MAX_CTAS = 24;  // 2 counts per CTA behind the header and four threshold words: 32 + 16 + 192 <= 256 bytes
enum { MC_W_BSTAR = 8, MC_W_LO = 9, MC_W_HI = 10, MC_W_B = 11, MC_W_COUNTS = 12 };

struct McSmem {
    uint32_t wsum[MC_T / 32];
    int bstar;
    int wcnt_a[MC_T / 32], wcnt_b[MC_T / 32];
    int tot[2];
};

// The bucket of the K-th largest key (every thread gets it).
__device__ __forceinline__ uint32_t mc_find_bucket(const uint32_t* __restrict__ hist, int top_k, McSmem& sm) {
    constexpr int PER = LQ_HIST_BINS / MC_T;  // bins per thread, contiguous; higher thread = larger keys
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) sm.bstar = 0;  // top_k above the number of counted scores: bin 0 makes every row a candidate
    uint32_t own = 0;
    const uint4* h4 = reinterpret_cast<const uint4*>(hist + tid * PER);
#pragma unroll 4
    for (int b = 0; b < PER / 4; ++b) {
        const uint4 v = __ldcg(h4 + b);
        own += v.x + v.y + v.z + v.w;
    }
    uint32_t suf = own;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += v;
    }
    if (lane == 0) sm.wsum[warp] = suf;
    __syncthreads();
    uint32_t higher = 0;
    for (int w = warp + 1; w < MC_T / 32; ++w) higher += sm.wsum[w];
    suf += higher;
    const uint32_t above = suf - own;
    if (above < (uint32_t)top_k && (uint32_t)top_k <= suf) {
        uint32_t acc = above;
        int b = PER - 1;
        for (; b > 0; --b) {
            const uint32_t v = __ldcg(hist + tid * PER + b);
            if (acc + v >= (uint32_t)top_k) break;
            acc += v;
        }
        sm.bstar = tid * PER + b;
    }
    __syncthreads();
    return (uint32_t)sm.bstar;
}

__global__ void __launch_bounds__(MC_T) classify_mc_count_kernel(const float* __restrict__ scores_g, int n, int top_k,
                                                                TokenWs ws, size_t ws_stride) {
    ws = ws_at(ws, ws_stride * blockIdx.y);
    const float* scores = tok_off(scores_g, ws_stride * blockIdx.y);
    __shared__ McSmem sm;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bstar = mc_find_bucket(ws.hist, top_k, sm);
    const float B = __uint_as_float(ws.sel->bound_bits);
    const float t_lo = __uint_as_float(bstar << LQ_HIST_SHIFT);
    const uint32_t hi_bits = (bstar + 1u) << LQ_HIST_SHIFT;
    const float t_hi = __uint_as_float(hi_bits > 0x7F800000u ? 0x7F800000u : hi_bits);
    const float two_b = __fmul_ru(2.0f, B);
    const float hi = __fadd_ru(t_hi, two_b), lo = __fadd_rd(t_lo, -two_b);
    int* words = reinterpret_cast<int*>(ws.sel);
    const int per = ((n + (int)gridDim.x - 1) / (int)gridDim.x + 31) / 32 * 32;
    const int beg = blockIdx.x * per, end = min(n, beg + per);
    int ca = 0, cb = 0;
    for (int i0 = beg + warp * 32; i0 < end; i0 += MC_T) {
        const int i = i0 + lane;
        const float a = i < end ? fabsf(scores[i]) : -1.0f;
        ca += __popc(__ballot_sync(0xffffffffu, a > hi));
        cb += __popc(__ballot_sync(0xffffffffu, !(a > hi) && a >= lo));
    }
    if (lane == 0) {
        sm.wcnt_a[warp] = ca;
        sm.wcnt_b[warp] = cb;
    }
    __syncthreads();
    if (tid == 0) {
        int ta = 0, tb = 0;
        for (int w = 0; w < MC_T / 32; ++w) {
            ta += sm.wcnt_a[w];
            tb += sm.wcnt_b[w];
        }
        words[MC_W_COUNTS + 2 * blockIdx.x] = ta;
        words[MC_W_COUNTS + 2 * blockIdx.x + 1] = tb;
        if (blockIdx.x == 0) {
            words[MC_W_BSTAR] = (int)bstar;
            words[MC_W_LO] = __float_as_int(lo);
            words[MC_W_HI] = __float_as_int(hi);
            words[MC_W_B] = __float_as_int(B);
        }
    }
}

__global__ void __launch_bounds__(MC_T) classify_mc_write_kernel(const float* __restrict__ scores_g, int n, int top_k,
                                                                TokenWs ws, size_t ws_stride, int band_scores) {
    ws = ws_at(ws, ws_stride * blockIdx.y);
    const float* scores = tok_off(scores_g, ws_stride * blockIdx.y);
    __shared__ McSmem sm;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int* words = reinterpret_cast<const int*>(ws.sel);
    const float lo = __int_as_float(words[MC_W_LO]), hi = __int_as_float(words[MC_W_HI]);
    int oa = 0, ob = 0, ta = 0, tb = 0;
    for (int c = 0; c < (int)gridDim.x; ++c) {
        const int a = words[MC_W_COUNTS + 2 * c], b = words[MC_W_COUNTS + 2 * c + 1];
        if (c < (int)blockIdx.x) {
            oa += a;
            ob += b;
        }
        ta += a;
        tb += b;
    }
    const int per = ((n + (int)gridDim.x - 1) / (int)gridDim.x + 31) / 32 * 32;
    const int beg = blockIdx.x * per, end = min(n, beg + per);
    // rounds of MC_T rows: warp w of a round holds rows [i0 + 32 w, i0 + 32 w + 32); offsets inside a round from the
    // warps' ballot counts
    for (int i0 = beg; i0 < end; i0 += MC_T) {
        const int i = i0 + warp * 32 + lane;
        const float v = i < end ? scores[i] : 0.0f;
        const float a = i < end ? fabsf(v) : -1.0f;
        const int cls = a > hi ? 1 : (a >= lo ? 2 : 0);
        const uint32_t ba = __ballot_sync(0xffffffffu, cls == 1), bb = __ballot_sync(0xffffffffu, cls == 2);
        if (lane == 0) {
            sm.wcnt_a[warp] = __popc(ba);
            sm.wcnt_b[warp] = __popc(bb);
        }
        __syncthreads();
        int wa = 0, wb = 0, ra = 0, rb = 0;
        for (int w = 0; w < MC_T / 32; ++w) {
            if (w < warp) {
                wa += sm.wcnt_a[w];
                wb += sm.wcnt_b[w];
            }
            ra += sm.wcnt_a[w];
            rb += sm.wcnt_b[w];
        }
        const uint32_t lt = (1u << lane) - 1u;
        if (cls == 1) {
            const int pos = oa + wa + __popc(ba & lt);
            ws.hit_idx[pos] = (uint32_t)i;
            ws.hit_score[pos] = v;
        } else if (cls == 2) {
            const int pos = ob + wb + __popc(bb & lt);
            ws.band_idx[pos] = (uint32_t)i;
            if (band_scores) ws.band_exact[pos] = v;
        }
        oa += ra;
        ob += rb;
        __syncthreads();
    }
    // the histogram is cleared for the next scan (every CTA a slice); the header last
    for (int i = blockIdx.x * MC_T + tid; i < LQ_HIST_BINS / 4; i += gridDim.x * MC_T)
        reinterpret_cast<uint4*>(ws.hist)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (blockIdx.x == 0 && tid == 0)
        *ws.sel = SelHeader{ta, tb, top_k, top_k - ta, __uint_as_float((uint32_t)words[MC_W_BSTAR] << LQ_HIST_SHIFT),
                            __int_as_float(words[MC_W_B]), 0, 0u};
}

__global__ void __launch_bounds__(256) final_pick_kernel(TokenWs ws, int* err, size_t ws_stride) {
    __shared__ SelectSmem<256> sm;
    final_pick_block<256>(ws_at(ws, ws_stride * blockIdx.y), err, sm);
}

// Sort the hit list by (|v| desc, idx asc) with a bitonic network over 64-bit keys
// (~|v| bits, row) held in `buf` (shared memory, or global scratch for very large K),
// n_pad a power of two >= count; writes the sorted rows and their signed scores.
__global__ void __launch_bounds__(1024) sort_hits_kernel(const uint32_t* hit_idx, const float* hit_val,
                                                        const SelHeader* sel, const float* scores,
                                                        unsigned long long* gbuf, int n_pad, int use_smem,
                                                        uint32_t* idx_out, float* val_out, int* count_out) {
    extern __shared__ __align__(16) unsigned long long s_buf[];
    unsigned long long* buf = use_smem ? s_buf : gbuf;
    const int count = sel->n_sel;
    const int tid = threadIdx.x;
    for (int i = tid; i < n_pad; i += 1024) {
        unsigned long long k = ~0ull;  // pads sort to the end
        if (i < count) k = ((unsigned long long)(~abs_key(hit_val[i])) << 32) | (unsigned long long)hit_idx[i];
        buf[i] = k;
    }
    __syncthreads();
    for (int size = 2; size <= n_pad; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < n_pad / 2; t += 1024) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool up = ((lo & size) == 0);
                const unsigned long long a = buf[lo], b = buf[hi];
                if ((a > b) == up) {
                    buf[lo] = b;
                    buf[hi] = a;
                }
            }
            __syncthreads();
        }
    }
    for (int i = tid; i < count; i += 1024) {
        const uint32_t r = (uint32_t)(buf[i] & 0xffffffffull);
        idx_out[i] = r;
        val_out[i] = scores[r];
    }
    if (tid == 0 && count_out) *count_out = count;
}

// Top-K by VALUE (descending, ties to the lower index), sorted: the order of the LM-head style calls
// q4k_matvec_topk / f16_gemv_topk (crates/larql-compute/src/backend/quant_matvec.rs:268-277,
// backend/matmul.rs:100-109).  One CTA: radix select of the K-th largest ordered key, index-ordered
// compaction of the winners into 64-bit (key, row) words, bitonic sort in shared memory.
__device__ __forceinline__ uint32_t value_key(float v) {  // larger value -> larger key
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(SEL_T, 1)
topk_value_kernel(const float* __restrict__ scores, int n, int top_k, int n_pad, uint32_t* __restrict__ idx_out,
                  float* __restrict__ val_out, int* err) {
    extern __shared__ __align__(16) unsigned long long t_buf[];  // [n_pad]
    __shared__ SelectSmem<SEL_T> sm;
    __shared__ int s_cut, s_nan;
    const int tid = threadIdx.x;
    if (tid == 0) {
        s_cut = n;
        s_nan = 0;
    }
    for (int i = tid; i < n_pad; i += SEL_T) t_buf[i] = ~0ull;  // pads sort to the end
    __syncthreads();
    bool nan = false;
    for (int i = tid; i < n; i += SEL_T) nan |= scores[i] != scores[i];
    if (nan) s_nan = 1;
    __syncthreads();
    if (s_nan) {
        set_err(err, DEV_ERR_NAN_SCORE);
        return;
    }
    const int k = min(top_k, n);
    auto keyf = [scores](int i) { return value_key(scores[i]); };
    uint32_t tau_key = 0;
    int cnt_gt = 0, need_eq = k;
    if (k < n) block_kth_largest_keys<SEL_T, 0>(keyf, n, k, sm, tau_key, cnt_gt, need_eq);
    int na, nb;
    if (k < n) {
        // the need_eq lowest rows among those equal to the threshold
        block_compact2<SEL_T>(
            n, sm, need_eq, [&](int i) { return keyf(i) == tau_key ? 2 : 0; }, [&](int, int) {},
            [&](int pos, int i) { if (pos == need_eq - 1) s_cut = i + 1; }, na, nb);
        __syncthreads();
    }
    const int cut = s_cut;
    block_compact2<SEL_T>(
        n, sm, 0,
        [&](int i) {
            if (k >= n) return 1;
            const uint32_t key = keyf(i);
            return (key > tau_key || (key == tau_key && i < cut)) ? 1 : 0;
        },
        [&](int pos, int i) { t_buf[pos] = ((unsigned long long)(~keyf(i)) << 32) | (unsigned long long)(uint32_t)i; },
        [&](int, int) {}, na, nb);
    __syncthreads();
    for (int size = 2; size <= n_pad; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < n_pad / 2; t += SEL_T) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool up = ((lo & size) == 0);
                const unsigned long long a = t_buf[lo], b = t_buf[hi];
                if ((a > b) == up) {
                    t_buf[lo] = b;
                    t_buf[hi] = a;
                }
            }
            __syncthreads();
        }
    }
    for (int i = tid; i < k; i += SEL_T) {
        const uint32_t r = (uint32_t)(t_buf[i] & 0xffffffffull);
        idx_out[i] = r;
        val_out[i] = scores[r];
    }
}

}  // namespace

// top_k <= 16384 (the sort runs in shared memory)
cudaError_t launch_topk_value_sorted(const float* scores, int n, int top_k, uint32_t* idx_out, float* val_out, int* err,
                                     cudaStream_t st) {
    const int k = top_k < n ? top_k : n;
    if (k <= 0) return cudaSuccess;
    if (k > 16384) return cudaErrorInvalidValue;
    int n_pad = 1;
    while (n_pad < k) n_pad <<= 1;
    cudaError_t e = set_max_dyn_smem((const void*)topk_value_kernel, 16384 * 8);
    if (e != cudaSuccess) return e;
    topk_value_kernel<<<1, SEL_T, (size_t)n_pad * 8, st>>>(scores, n, top_k, n_pad, idx_out, val_out, err);
    return cudaGetLastError();
}

cudaError_t launch_select(const float* scores, int n, int top_k, TokenWs ws, int* err, cudaStream_t st, int batch,
                          size_t ws_stride) {
    cudaError_t e = set_max_dyn_smem((const void*)select_kernel, SEL_SMEM_VALS_MAX * 4);
    if (e != cudaSuccess) return e;
    const int use_smem = n <= SEL_SMEM_VALS_MAX;
    const size_t smem = use_smem ? (size_t)((n + 3) / 4 * 4) * sizeof(float) : 0;
    select_kernel<<<dim3(1, batch), SEL_T, smem, st>>>(scores, n, top_k, ws, err, use_smem, ws_stride);
    return cudaGetLastError();
}

// band_scores: the band rows' entries of band_exact are filled with their (already exact) scores.
cudaError_t launch_classify_mc(const float* scores, int n, int top_k, TokenWs ws, cudaStream_t st, int batch,
                               size_t ws_stride, int band_scores) {
    int g = (n + 1023) / 1024;
    if (g > MC_MAX_CTAS) g = MC_MAX_CTAS;
    if (g < 1) g = 1;
    classify_mc_count_kernel<<<dim3(g, batch), MC_T, 0, st>>>(scores, n, top_k, ws, ws_stride);
    classify_mc_write_kernel<<<dim3(g, batch), MC_T, 0, st>>>(scores, n, top_k, ws, ws_stride, band_scores);
    return cudaGetLastError();
}

cudaError_t launch_classify(const float* scores, int n, int top_k, TokenWs ws, int* err, cudaStream_t st, int batch,
                            size_t ws_stride) {
    // many rows: several CTAs per token (the lists come out the same)
    static const bool mc_on = [] { const char* e = getenv("LARQL_B200_SELECT_MC"); return !(e && e[0] == '0'); }();
    // (many tokens fill the GPU with one CTA each: measured slower with several at batch 64)
    if (mc_on && n >= 8192 && top_k > 0 && top_k < n && batch <= 16)
        return launch_classify_mc(scores, n, top_k, ws, st, batch, ws_stride, 0);
    cudaError_t e = set_max_dyn_smem((const void*)classify_kernel, SEL_SMEM_VALS_MAX * 4);
    if (e != cudaSuccess) return e;
    const int use_smem = n <= SEL_SMEM_VALS_MAX;
    const size_t smem = use_smem ? (size_t)((n + 3) / 4 * 4) * sizeof(float) : 0;
    classify_kernel<<<dim3(1, batch), SEL_T, smem, st>>>(scores, n, top_k, ws, err, use_smem, ws_stride);
    return cudaGetLastError();
}

cudaError_t launch_final_pick(TokenWs ws, int* err, cudaStream_t st, int batch, size_t ws_stride) {
    final_pick_kernel<<<dim3(1, batch), 256, 0, st>>>(ws, err, ws_stride);
    return cudaGetLastError();
}

cudaError_t launch_topk_abs_sorted(const float* scores, int n, int top_k, TokenWs ws, uint32_t* idx_out,
                                   float* val_out, int* count_out, unsigned long long* sort_buf, int* err,
                                   cudaStream_t st) {
    cudaError_t e = launch_select(scores, n, top_k, ws, err, st, 1, 0);
    if (e != cudaSuccess) return e;
    e = launch_final_pick(ws, err, st, 1, 0);
    if (e != cudaSuccess) return e;
    const int count = top_k < n ? top_k : n;
    if (count <= 0) {
        if (count_out) return cudaMemsetAsync(count_out, 0, sizeof(int), st);
        return cudaSuccess;
    }
    int n_pad = 1;
    while (n_pad < count) n_pad <<= 1;
    e = set_max_dyn_smem((const void*)sort_hits_kernel, 16384 * 8);
    if (e != cudaSuccess) return e;
    const int use_smem = n_pad <= 16384;
    sort_hits_kernel<<<1, 1024, use_smem ? (size_t)n_pad * 8 : 0, st>>>(ws.hit_idx, ws.hit_score, ws.sel, scores,
                                                                        sort_buf, n_pad, use_smem, idx_out, val_out,
                                                                        count_out);
    return cudaGetLastError();
}

}  // namespace lq
