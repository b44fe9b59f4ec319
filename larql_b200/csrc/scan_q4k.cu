// Q4_K gate scan for one token (batch-1, HBM-bound) and the exact re-score.
//
// scan_q4k_kernel — persistent CTAs stream tiles of whole rows from HBM into a ring
// of shared-memory stages with TMA bulk copies (cp.async.bulk + mbarrier), and decode
// them in registers: each thread owns one "cell" = one 32-byte nibble group of one
// super-block column (64 weights: sub-blocks 2g and 2g+1), keeps the matching 64
// activations in registers as two dp4a byte planes, and walks down the rows of the
// tile.  The per-row sum over cells is a fixed-order shared-memory + shuffle tree.
// It produces a FAST score (any-order integer dot products, sum_x form) and a rigorous
// bound on |fast - reference| per row; the selection kernels use the bound to find the
// few rows whose top-K membership needs the reference's exact bits.
//
// rescore_q4k_kernel — those rows (or all rows) in the reference's exact f32 order:
// Association A of the CPU backend, process_q4k_superblock
// (crates/larql-compute/src/cpu/ops/q4_common/matvec_f32.rs:116-155) with the scalar
// q4_dual_dot_32 (…/q4_common/dual.rs:186-198): per 32-element sub-block a sequential
// sum of q*x (separate multiply and add, never fused), `acc += sc*dot - mn*sumx` for the
// low then the high sub-block of each group, super-block partials added in order.
#include "q4k_exact.cuh"
#include "select.cuh"

namespace lq {

namespace {

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_MAX_STAGES = 6;
constexpr int SCAN_TILE_TARGET = 32 * 1024;
constexpr int SCAN_SMEM_BUDGET = 200 * 1024;

struct ScanGeom {
    int nsb;         // super-blocks per row
    int G;           // cells per row = 4 * nsb
    int P;           // rows processed side by side = SCAN_THREADS / G
    int R;           // rows per tile
    int row_bytes;
    int tile_bytes;
    int stages;
    int part_floats; // R * G
    int smem_bytes;
};

__host__ __device__ inline int align_up(int v, int a) { return (v + a - 1) / a * a; }

__host__ inline bool scan_geom(int hidden, ScanGeom& g) {
    if (hidden <= 0 || hidden % 256 != 0) return false;
    g.nsb = hidden / 256;
    g.G = 4 * g.nsb;
    if (g.G > SCAN_THREADS) return false;
    g.P = SCAN_THREADS / g.G;
    g.row_bytes = g.nsb * 144;
    int r = SCAN_TILE_TARGET / g.row_bytes;
    r = r / g.P * g.P;
    if (r < g.P) r = g.P;
    g.R = r;
    g.tile_bytes = g.R * g.row_bytes;
    g.part_floats = g.R * g.G;
    const int fixed = 128 + 2 * 2 * g.part_floats * 4;  // barriers + double-buffered (score,bound) partials
    int st = (SCAN_SMEM_BUDGET - align_up(fixed, 128)) / g.tile_bytes;
    if (st > SCAN_MAX_STAGES) st = SCAN_MAX_STAGES;
    if (st < 2) return false;
    g.stages = st;
    g.smem_bytes = align_up(fixed, 128) + st * g.tile_bytes;
    return true;
}

__global__ void __launch_bounds__(SCAN_THREADS, 1)
scan_q4k_kernel(const uint8_t* __restrict__ W, int n_rows, ScanGeom gm, XPrep xp, float* __restrict__ scores,
                uint32_t* __restrict__ hist, uint32_t* __restrict__ bound_bits, float c1, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    float* part = reinterpret_cast<float*>(smem + 128);  // [2 buffers][2 kinds][R*G]
    uint8_t* stage0 = smem + align_up(128 + 2 * 2 * gm.part_floats * 4, 128);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gm.G, P = gm.P, R = gm.R;
    const int c = tid % G, prow = tid / G;
    const bool active = prow < P;
    const int s = c >> 2, g = c & 3;

    // This thread's 64 activations: sub-blocks (s*8 + 2g) and (s*8 + 2g + 1).
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
    const float ab_lo = xp.abs[blk_lo], ab_hi = xp.abs[blk_hi];
    const float qe_lo = xp.scale[blk_lo] * (15.0f * 32.0f * LQ_XQ_ERR_STEPS);
    const float qe_hi = xp.scale[blk_hi] * (15.0f * 32.0f * LQ_XQ_ERR_STEPS);

    const int n_tiles = (n_rows + R - 1) / R;
    const int my_first = blockIdx.x;
    const int my_count = my_first < n_tiles ? (n_tiles - my_first + gridDim.x - 1) / gridDim.x : 0;

    if (tid == 0) {
        for (int i = 0; i < gm.stages; ++i) mbar_init(&full[i], 1);
        fence_mbar_init();
    }
    __syncthreads();

    auto issue = [&](int k) {
        const int tile = my_first + k * gridDim.x;
        const int row0 = tile * R;
        const int rows_here = min(R, n_rows - row0);
        const uint32_t bytes = (uint32_t)rows_here * (uint32_t)gm.row_bytes;
        const int stg = k % gm.stages;
        mbar_expect_tx(&full[stg], bytes);
        tma_bulk_g2s(stage0 + (size_t)stg * gm.tile_bytes, W + (size_t)row0 * gm.row_bytes, bytes, &full[stg]);
    };
    if (tid == 0) {
        const int pre = min(my_count, gm.stages);
        for (int k = 0; k < pre; ++k) issue(k);
    }

    bool timed_out = false;
    float bmax = 0.0f;  // largest row bound seen by this warp's lane 0
    for (int k = 0; k < my_count; ++k) {
        const int stg = k % gm.stages;
        const uint32_t parity = (uint32_t)((k / gm.stages) & 1);
        // A thread whose wait ran out keeps walking through the barriers (its results are
        // garbage and the error word says so) so that the CTA never splits at a barrier.
        if (!timed_out && !mbar_wait(&full[stg], parity)) timed_out = true;
        const int tile = my_first + k * gridDim.x;
        const int row0 = tile * R;
        const int rows_here = min(R, n_rows - row0);
        const uint8_t* tb = stage0 + (size_t)stg * gm.tile_bytes;
        float* p_sc = part + (size_t)(k & 1) * 2 * gm.part_floats;
        float* p_bd = p_sc + gm.part_floats;

        if (active) {
            for (int r = prow; r < rows_here; r += P) {
                const uint8_t* cell = tb + (size_t)r * gm.row_bytes + s * 144;
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
                const float sc_lo = (float)(sc2 & 0xff), sc_hi = (float)(sc2 >> 8);
                const float m_lo = (float)(m2 & 0xff), m_hi = (float)(m2 >> 8);
                const float dot_lo = st_lo * (float)(ia_lo * 256 + ib_lo);
                // hi nibbles entered dp4a as 16*q: the sum is an exact multiple of 16
                const float dot_hi = st_hi * (float)((ia_hi * 256 + ib_hi) >> 4);
                const float val = d * (sc_lo * dot_lo + sc_hi * dot_hi) - dmin * (m_lo * su_lo + m_hi * su_hi);
                const float ad = fabsf(d), am = fabsf(dmin);
                const float tb_ = ad * 15.0f * (sc_lo * ab_lo + sc_hi * ab_hi) + am * (m_lo * ab_lo + m_hi * ab_hi);
                const float qb = ad * (sc_lo * qe_lo + sc_hi * qe_hi);
                p_sc[r * G + c] = val;
                p_bd[r * G + c] = c1 * tb_ + qb;
            }
        }
        __syncthreads();
        if (tid == 0 && k + gm.stages < my_count) issue(k + gm.stages);
        // Row sums: one warp per row, fixed order.
        for (int r = warp; r < rows_here; r += SCAN_THREADS / 32) {
            float a = 0.0f, b = 0.0f;
            for (int i = lane; i < G; i += 32) {
                a += p_sc[r * G + i];
                b += p_bd[r * G + i];
            }
            for (int o = 16; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
            }
            if (lane == 0) {
                scores[row0 + r] = a;
                if (hist) {
                    if (a != a) set_err(err, DEV_ERR_NAN_SCORE);
                    atomicAdd(&hist[__float_as_uint(fabsf(a)) >> LQ_HIST_SHIFT], 1u);
                    bmax = fmaxf(bmax, b);
                }
            }
        }
    }
    if (hist && lane == 0 && bmax > 0.0f) atomicMax(bound_bits, __float_as_uint(bmax));
    if (__syncthreads_or(timed_out ? 1 : 0)) {
        set_err(err, DEV_ERR_TMA_TIMEOUT);
        // Give copies already issued a last bounded chance to land before the CTA's
        // shared memory is released.
        if (tid == 0)
            for (int k = max(0, my_count - gm.stages); k < my_count; ++k)
                (void)mbar_wait(&full[k % gm.stages], (uint32_t)((k / gm.stages) & 1));
        __syncthreads();
    }
}

// ------------------------------------------------------------------ exact ----
constexpr int RESCORE_THREADS = 256;  // 8 warps, one row per warp at a time

__global__ void __launch_bounds__(RESCORE_THREADS)
rescore_q4k_kernel(const uint8_t* __restrict__ W, int n_rows_total, int nsb, const float* __restrict__ xn,
                   const uint32_t* __restrict__ rows_idx, const int* __restrict__ n_rows_dev, int n_rows_host,
                   float* __restrict__ out, TokenWs ws, int top_k, int run_final, int* err, size_t ws_stride) {
    extern __shared__ __align__(128) uint8_t smem[];
    {
        const size_t off = ws_stride * blockIdx.y;
        ws = ws_at(ws, off);
        xn = tok_off(xn, off);
        rows_idx = tok_off(rows_idx, off);
        n_rows_dev = tok_off(n_rows_dev, off);
        out = tok_off(out, off);
    }
    float* sb_part_all = reinterpret_cast<float*>(smem);  // [8 warps][nsb]
    float* xs = sb_part_all + (RESCORE_THREADS / 32) * nsb; // [4*nsb chunks][68]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_rows = n_rows_dev ? min(*n_rows_dev, n_rows_total) : n_rows_host;
    const int row_bytes = nsb * 144;
    const int warps_total = gridDim.x * (RESCORE_THREADS / 32);
    if ((int)blockIdx.x * (RESCORE_THREADS / 32) < n_rows) {
        for (int i = threadIdx.x; i < nsb * 256; i += RESCORE_THREADS) xs[(i >> 6) * 68 + (i & 63)] = xn[i];
    }
    __syncthreads();
    for (int i = blockIdx.x * (RESCORE_THREADS / 32) + warp; i < n_rows; i += warps_total) {
        const uint32_t r = rows_idx ? rows_idx[i] : (uint32_t)i;
        const float v = exact_row_q4k(W + (size_t)r * row_bytes, xs, nsb, sb_part_all + warp * nsb, lane);
        if (lane == 0) out[i] = v;
    }
    if (run_final) {
        __shared__ int s_last;
        __shared__ SelectSmem<RESCORE_THREADS> sel_sm;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = (atomicAdd(&ws.sel->done_ctr, 1) == (int)gridDim.x - 1);
        __syncthreads();
        if (s_last) {
            __threadfence();
            final_pick_block<RESCORE_THREADS>(ws, err, sel_sm, xs, 4 * nsb * 68);
        }
    }
}

}  // namespace

int scan_q4k_smem_bytes(int hidden) {
    ScanGeom g;
    return scan_geom(hidden, g) ? g.smem_bytes : -1;
}

cudaError_t launch_scan_q4k(const Q4kMat& m, const XPrep& xp, float* scores, uint32_t* hist, uint32_t* bound_bits,
                            float c1, int* err, int sm_count, cudaStream_t st) {
    ScanGeom g;
    if (!scan_geom(m.cols, g)) return cudaErrorInvalidValue;
    if (m.rows == 0) return cudaSuccess;
    cudaError_t e = set_max_dyn_smem((const void*)scan_q4k_kernel, SCAN_SMEM_BUDGET + 4096);
    if (e != cudaSuccess) return e;
    const int n_tiles = (m.rows + g.R - 1) / g.R;
    const int grid = n_tiles < sm_count ? n_tiles : sm_count;
    scan_q4k_kernel<<<grid, SCAN_THREADS, g.smem_bytes, st>>>(m.w, m.rows, g, xp, scores, hist, bound_bits, c1, err);
    return cudaGetLastError();
}

cudaError_t launch_rescore_q4k(const Q4kMat& m, const float* xn, const uint32_t* rows_idx, const int* n_rows_dev,
                               int n_rows_host, float* out, TokenWs ws, int top_k, int run_final, int* err,
                               int sm_count, cudaStream_t st, int batch, size_t ws_stride) {
    if (m.cols <= 0 || m.cols % 256 != 0) return cudaErrorInvalidValue;
    const int nsb = m.cols / 256;
    int grid;
    // count unknown on the host: a fixed grid strides over the list (about 4 CTAs per SM in total)
    if (n_rows_dev) grid = batch > 1 ? (4 * sm_count / batch > 8 ? 4 * sm_count / batch : 8) : sm_count * 2;
    else {
        grid = (n_rows_host + 7) / 8;
        if (grid > sm_count * 8) grid = sm_count * 8;
        if (grid < 1) grid = 1;
    }
    const size_t smem = ((size_t)(RESCORE_THREADS / 32) * nsb + (size_t)4 * nsb * 68) * sizeof(float);
    cudaError_t e = set_max_dyn_smem((const void*)rescore_q4k_kernel, 96 * 1024);
    if (e != cudaSuccess) return e;
    rescore_q4k_kernel<<<dim3(grid, batch), RESCORE_THREADS, smem, st>>>(m.w, m.rows, nsb, xn, rows_idx, n_rows_dev,
                                                                        n_rows_host, out, ws, top_k, run_final, err,
                                                                        ws_stride);
    return cudaGetLastError();
}

}  // namespace lq
