// Fused persistent Q4_K walk for one token: every layer of a stack in ONE cooperative
// launch, one CTA per SM, four grid barriers per layer.
//
// Per layer each CTA
//   0. (team 0) RMS-normalises the residual and builds the 16-bit fixed-point copy of it
//      in shared memory (rms_norm_eps, crates/larql-compute/src/residual.rs:56-78);
//   1. scans its share of the gate rows (tiles of whole rows, TMA bulk copies issued by a
//      producer warp into a shared-memory ring), keeps the fast scores of ITS rows in
//      shared memory and adds their |score| keys to a global coarse histogram;
//      -- grid barrier --
//   2. reads the histogram, finds the bucket [t_lo, t_hi) of the K-th largest |score| and,
//      with B the bound on |fast - reference|, splits its rows into certainly-in
//      (> t_hi + 2B), band (>= t_lo - 2B) and out; re-scores its band rows in the
//      reference's exact f32 order and publishes them; gathers its certainly-in rows
//      (up dot, SiLU, down axpy — walk_ffn_sparse, crates/larql-inference/src/vindex/
//      walk_ffn/sparse.rs:218-289);
//      -- grid barrier --
//   3. picks, identically in every CTA, the K - n_in best band rows under (|score| desc,
//      row asc) (top_k_by_abs, crates/larql-vindex/src/index/compute/gate_knn/mod.rs:50-108)
//      and gathers the winners it owns; writes its partial out[H];
//      -- grid barrier --
//   4. sums a column slice of the partials in fixed order, adds the residual (run_ffn,
//      crates/larql-compute/src/forward/layer.rs:109-124) and writes the next residual.
//      -- grid barrier --
// A row is scanned, classified, re-scored and gathered by the CTA that streamed it, so no
// hit list travels between CTAs and the summation order is fixed: results are run-to-run
// identical.  Every wait (mbarrier, grid barrier) is bounded and reports through the error
// word instead of hanging.
#include "../../include/larql_cuda.h"
#include "q4k_exact.cuh"
#include "select.cuh"

namespace lq {

namespace {

constexpr int FW_CONSUMERS = 384;
constexpr int FW_THREADS = FW_CONSUMERS + 32;
constexpr int FW_NWARPS = FW_CONSUMERS / 32;
constexpr int FW_BAR_ALL = 0;        // all 544 threads
constexpr int FW_BAR_CONS = 9;       // the 512 consumers
constexpr int FW_MAX_STAGES = 8;
constexpr int FW_MAX_SLOTS = 32;
constexpr float FW_NOISE_FLOOR = 1e-10f;  // ACTIVATION_NOISE_FLOOR, walk_config.rs:64
constexpr int FW_PICK_CAP = 8192;    // band entries the final pick can stage in shared memory
constexpr int FW_RANK_CAP = 2048;    // up to this many band entries the pick ranks by counting

struct FusedGeom {
    int nsb, G, TS, P, Wt;      // super-blocks/row, cells/row, team size, teams, warps per team
    int row_bytes, R, Rt;       // rows per scan tile, rows per team per tile
    int tile_bytes, S;          // scan ring
    int slot_bytes, D;          // gather ring: one slot = up row + down row
    int max_slots;              // score slots per CTA (tiles per CTA * R)
    int off_xs, off_xa, off_xb, off_blk, off_wpart, off_scores, off_lists, off_red, off_ring;
    int ring_bytes, smem_bytes;
};

struct FusedLayer {
    const uint8_t* gate;
    const uint8_t* up;
    const uint8_t* down;
};

struct FusedArgs {
    const FusedLayer* layers;  // device array of n_layers entries, or nullptr: use `single`
    FusedLayer single;
    int n_layers, n_rows, top_k;
    uint32_t flags;
    float c1;
    const float* h_in;
    float* h_out;
    float* hbuf0;
    float* hbuf1;
    uint32_t* hist;        // [2][LQ_HIST_BINS]
    uint32_t* ctrs;        // see CTR_* below
    uint32_t* band_row;    // [n_rows]
    float* band_exact;     // [n_rows]
    uint32_t* pool_row;    // [grid][max_slots]: certainly-in rows a CTA hands over (beyond its fair share)
    float* pool_score;     // [grid][max_slots]
    uint32_t* pool_cnt;    // [grid]
    float* partials;       // [grid][H]
    uint32_t* hit_out;     // optional [top_k] selected rows of the LAST layer (unordered)
    uint32_t* count_out;   // optional: number of rows selected in the last layer
    lq_walk_stats* stats;  // optional, last layer
    unsigned long long* phase_ns;  // optional [16]: globaltimer stamps of CTA 0 in the last layer
    int* err;
};

enum { CTR_SYNC = 0, CTR_BOUND0 = 1, CTR_BOUND1 = 2, CTR_IN = 3, CTR_BAND = 4, CTR_HITS = 5, CTR_MAXBIN0 = 6,
       CTR_MAXBIN1 = 7, CTR_WORDS = 16 };

__host__ __device__ inline int fw_align(int v, int a) { return (v + a - 1) / a * a; }

__host__ inline bool fused_geom(int hidden, int n_rows, int grid_hint, FusedGeom& g) {
    if (hidden <= 0 || hidden % 256 != 0) return false;
    g.nsb = hidden / 256;
    g.G = 4 * g.nsb;
    g.TS = fw_align(g.G, 32);
    if (g.TS < 64) g.TS = 64;
    if (g.TS > FW_CONSUMERS) return false;
    g.P = FW_CONSUMERS / g.TS;
    if (g.P > 8) g.P = 8;
    g.Wt = g.TS / 32;
    g.row_bytes = g.nsb * 144;
    g.slot_bytes = 2 * g.row_bytes;
    int off = 1024;  // mbarriers
    g.off_xs = off;      off += fw_align(4 * g.nsb * 68 * 4, 128);
    g.off_xa = off;      off += fw_align(hidden, 128);
    g.off_xb = off;      off += fw_align(hidden, 128);
    g.off_blk = off;     off += fw_align(3 * (hidden / 32) * 4, 128);
    g.off_red = off;     off += 8192 + 1024;
    // rows per tile: about 36 KB, a multiple of P
    int r = (36 * 1024) / g.row_bytes / g.P * g.P;
    if (r < g.P) r = g.P;
    if (r > 8 * g.P) r = 8 * g.P;
    g.R = r;
    g.Rt = r / g.P;
    g.tile_bytes = g.R * g.row_bytes;
    g.off_wpart = off;   off += fw_align(2 * g.P * g.Rt * g.Wt * 4, 128);
    const int n_tiles = (n_rows + g.R - 1) / g.R;
    const int grid = grid_hint < n_tiles ? grid_hint : (n_tiles > 0 ? n_tiles : 1);
    g.max_slots = ((n_tiles + grid - 1) / grid) * g.R;
    g.off_scores = off;  off += fw_align(g.max_slots * 4, 128);
    g.off_lists = off;   off += fw_align(7 * g.max_slots * 4, 128);
    g.off_ring = off;
    const int budget = 224 * 1024;
    g.ring_bytes = (budget - off) / 128 * 128;
    if (g.ring_bytes < 2 * g.tile_bytes || g.ring_bytes < 2 * g.slot_bytes) return false;
    if (g.ring_bytes < FW_PICK_CAP * 8 + 24 * 1024) return false;
    if (g.ring_bytes < g.P * g.G * 65 * 4) return false;  // the merge stages one out[H] per team in the ring
    g.S = g.ring_bytes / g.tile_bytes;
    if (g.S > FW_MAX_STAGES) g.S = FW_MAX_STAGES;
    g.D = g.ring_bytes / g.slot_bytes;
    if (g.D > FW_MAX_SLOTS) g.D = FW_MAX_SLOTS;
    g.smem_bytes = off + g.ring_bytes;
    return true;
}

__device__ __forceinline__ unsigned long long gtimer() {
    return (unsigned long long)clock64();  // SM cycles (the accessor converts with the SM clock)
}
#define FW_STAMP(i)                                                                      \
    do {                                                                                 \
        if (a.phase_ns && l + 1 == a.n_layers && blockIdx.x == 0 && tid == 0) a.phase_ns[i] = gtimer(); \
    } while (0)

__device__ __forceinline__ void bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid barrier over all CTAs (consumer threads only).  `epoch` counts barriers so far.
// Bounded: gives up after about a second and records DEV_ERR_TMA_TIMEOUT.
__device__ __forceinline__ void grid_sync(uint32_t* ctr, uint32_t& epoch, int* err, bool& failed, int* s_flag) {
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    epoch += 1;
    if (threadIdx.x == 0 && !failed) {
        __threadfence();
        atomicAdd(ctr, 1u);
        const uint32_t target = epoch * gridDim.x;
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (ld_acquire_u32(ctr) < target) {
            // another CTA's failure (error word set) or a second of waiting ends the wait
            if (clock64() - t0 > (1ll << 31) || ((++spins & 63u) == 0 && *(volatile int*)err != 0)) {
                set_err(err, DEV_ERR_TMA_TIMEOUT);
                *s_flag = 1;
                break;
            }
        }
        __threadfence();
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    if (*s_flag) failed = true;
}

// One Q4_K cell (64 weights) against the thread's activation planes: fast value and bound.
struct CellX {
    uint32_t xa_lo[8], xb_lo[8], xa_hi[8], xb_hi[8];
    float st_lo, st_hi, su_lo, su_hi;
};

__device__ __forceinline__ float cell_dot(const uint8_t* cell, int g, const CellX& x, float ab_lo, float ab_hi,
                                          float c1, float& bound) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
    const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
    const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    int ia_lo = 0, ib_lo = 0, ia_hi = 0, ib_hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t lo = qw[j] & 0x0F0F0F0Fu, hi = qw[j] & 0xF0F0F0F0u;
        ia_lo = dp4a_us(lo, x.xa_lo[j], ia_lo);
        ib_lo = dp4a_uu(lo, x.xb_lo[j], ib_lo);
        ia_hi = dp4a_us(hi, x.xa_hi[j], ia_hi);
        ib_hi = dp4a_uu(hi, x.xb_hi[j], ib_hi);
    }
    const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
    uint32_t sc2, m2;
    q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
    const float sc_lo = (float)(sc2 & 0xff), sc_hi = (float)(sc2 >> 8);
    const float m_lo = (float)(m2 & 0xff), m_hi = (float)(m2 >> 8);
    const float dot_lo = x.st_lo * (float)(ia_lo * 256 + ib_lo);
    const float dot_hi = x.st_hi * (float)((ia_hi * 256 + ib_hi) >> 4);  // hi nibbles entered as 16*q
    if (c1 > 0.0f) {
        const float ad = fabsf(d), am = fabsf(dmin);
        const float qe = 15.0f * 32.0f * LQ_XQ_ERR_STEPS;
        bound = c1 * (ad * 15.0f * (sc_lo * ab_lo + sc_hi * ab_hi) + am * (m_lo * ab_lo + m_hi * ab_hi)) +
                ad * qe * (sc_lo * x.st_lo + sc_hi * x.st_hi);
    }
    return d * (sc_lo * dot_lo + sc_hi * dot_hi) - dmin * (m_lo * x.su_lo + m_hi * x.su_hi);
}

// The byte planes are stored word-major: word w (0..15, two 32-element blocks) of cell c sits
// at [w * G + c], so the lanes of a warp (consecutive cells) read consecutive words.
__device__ __forceinline__ void load_cellx(CellX& x, const uint32_t* xa, const uint32_t* xb, const float* blk, int nblk,
                                           int blk_lo, int G, int c) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        x.xa_lo[j] = xa[j * G + c];
        x.xb_lo[j] = xb[j * G + c];
        x.xa_hi[j] = xa[(8 + j) * G + c];
        x.xb_hi[j] = xb[(8 + j) * G + c];
    }
    x.st_lo = blk[blk_lo];
    x.st_hi = blk[blk_lo + 1];
    x.su_lo = blk[nblk + blk_lo];
    x.su_hi = blk[nblk + blk_lo + 1];
}

// Producer warp: issues every TMA copy of the CTA.  Scan tiles of a layer need nothing
// from the consumers; gather copies need the row lists, handed over at CTA barriers.
struct Rings {
    uint64_t* full;    // [S]
    uint64_t* empty;   // [S]   (arrival count: all consumers)
    uint64_t* gfull;   // [D]
    uint64_t* gempty;  // [D]
    uint8_t* ring;
};

__device__ __forceinline__ void producer_gather(const Rings& rg, const FusedGeom& gm, const FusedLayer& ly,
                                                const int* list, bool rows_direct, int n, uint32_t& g_it,
                                                int first_tile, int lane, bool& failed) {
    for (int i = 0; i < n; ++i) {
        const uint32_t gi = g_it + i;
        const int slot = gi % gm.D;
        if (gi >= (uint32_t)gm.D && !failed && !mbar_wait(&rg.gempty[slot], ((gi / gm.D) - 1) & 1)) failed = true;
        const int m = list[i];  // a score slot of this CTA, or (rows_direct) a global row
        const size_t row = rows_direct ? (size_t)(uint32_t)m
                                       : (size_t)(first_tile + (m / gm.R) * (int)gridDim.x) * gm.R + (m % gm.R);
        uint8_t* dst = rg.ring + (size_t)slot * gm.slot_bytes;
        if (lane == 0) mbar_expect_tx(&rg.gfull[slot], (uint32_t)gm.slot_bytes);
        __syncwarp();
        if (lane == 0) tma_bulk_g2s(dst, ly.up + row * gm.row_bytes, gm.row_bytes, &rg.gfull[slot]);
        if (lane == 1) tma_bulk_g2s(dst + gm.row_bytes, ly.down + row * gm.row_bytes, gm.row_bytes, &rg.gfull[slot]);
    }
    g_it += n;
}

// Consumers: gather the listed rows (score slots of this CTA).  Team t takes items
// t, t+P, ...; each item: up dot -> act -> down axpy into the thread's 64 accumulators.
__device__ __forceinline__ void consumer_gather(const Rings& rg, const FusedGeom& gm, const int* list, int n,
                                                const float* scores, uint32_t& g_it, const uint32_t* xa_s,
                                                const uint32_t* xb_s, const float* blk_s, float* wpart, int team, int c,
                                                bool active, float (&acc_lo)[32], float (&acc_hi)[32], float& corr_lo,
                                                float& corr_hi, bool& failed) {
    const int lane = threadIdx.x & 31, wt = (threadIdx.x % gm.TS) >> 5;
    const int s = c >> 2, g = c & 3, nblk = gm.nsb * 8;
    for (int i = team; i < n; i += gm.P) {
        const uint32_t gi = g_it + i;
        const int slot = gi % gm.D;
        if (!failed && !mbar_wait(&rg.gfull[slot], (gi / gm.D) & 1)) failed = true;
        const uint8_t* up_row = rg.ring + (size_t)slot * gm.slot_bytes;
        const uint8_t* down_row = up_row + gm.row_bytes;
        float val = 0.0f;
        if (active) {
            // activation planes straight from shared memory: the 64 accumulators stay in registers
            const uint8_t* cell = up_row + s * 144;
            const int blk_lo = s * 8 + 2 * g;
            const uint32_t* pa = xa_s + c;  // word-major planes: word w of this cell at [w * G + c]
            const uint32_t* pb = xb_s + c;
            const int G = gm.G;
            const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
            int ia_lo = 0, ib_lo = 0, ia_hi = 0, ib_hi = 0;
#pragma unroll
            for (int h4 = 0; h4 < 2; ++h4) {
                const uint4 q = *reinterpret_cast<const uint4*>(cell + 16 + g * 32 + 16 * h4);
                const uint32_t qw4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t lo = qw4[j] & 0x0F0F0F0Fu, hi = qw4[j] & 0xF0F0F0F0u;
                    ia_lo = dp4a_us(lo, pa[(4 * h4 + j) * G], ia_lo);
                    ib_lo = dp4a_uu(lo, pb[(4 * h4 + j) * G], ib_lo);
                    ia_hi = dp4a_us(hi, pa[(8 + 4 * h4 + j) * G], ia_hi);
                    ib_hi = dp4a_uu(hi, pb[(8 + 4 * h4 + j) * G], ib_hi);
                }
            }
            const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
            uint32_t sc2, m2;
            q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
            const float dot_lo = blk_s[blk_lo] * (float)(ia_lo * 256 + ib_lo);
            const float dot_hi = blk_s[blk_lo + 1] * (float)((ia_hi * 256 + ib_hi) >> 4);
            val = d * ((float)(sc2 & 0xff) * dot_lo + (float)(sc2 >> 8) * dot_hi) -
                  dmin * ((float)(m2 & 0xff) * blk_s[nblk + blk_lo] + (float)(m2 >> 8) * blk_s[nblk + blk_lo + 1]);
        }
        for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
        float* wp = wpart + (((i / gm.P) & 1) * gm.P + team) * gm.Wt;
        if (lane == 0) wp[wt] = val;
        bar_sync(1 + team, gm.TS);
        float upv = 0.0f;
        for (int w = 0; w < gm.Wt; ++w) upv += wp[w];
        const float gs = list ? scores[list[i]] : scores[i];  // list == nullptr: scores are per item
        const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
        float act = (gs * sig) * upv;
        if (!(fabsf(act) > FW_NOISE_FLOOR)) act = 0.0f;
        if (active && act != 0.0f) {
            const uint8_t* cell = down_row + s * 144;
            const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
            const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
            const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
            uint32_t sc2, m2;
            q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
            const float ad = act * d, am = act * dmin;
            // q enters as f = 1 + q/128 built by a byte permute; out += A*f, corrected by -A at the end
            const float A_lo = ad * (float)(sc2 & 0xff) * 128.0f, A_hi = ad * (float)(sc2 >> 8) * 128.0f;
            corr_lo += A_lo + am * (float)(m2 & 0xff);
            corr_hi += A_hi + am * (float)(m2 >> 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t lo = (qw[j] & 0x0F0F0F0Fu) | 0x80808080u;
                const uint32_t hi = ((qw[j] >> 4) & 0x0F0F0F0Fu) | 0x80808080u;
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {
                    const float fl = __uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7044u | (bb << 8)));
                    const float fh = __uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7044u | (bb << 8)));
                    acc_lo[4 * j + bb] = fmaf(A_lo, fl, acc_lo[4 * j + bb]);
                    acc_hi[4 * j + bb] = fmaf(A_hi, fh, acc_hi[4 * j + bb]);
                }
            }
        }
        mbar_arrive(&rg.gempty[slot]);
    }
    g_it += n;
}

__global__ void __launch_bounds__(FW_THREADS, 1) walk_fused_q4k_kernel(FusedGeom gm, FusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    Rings rg;
    rg.full = bars;
    rg.empty = bars + FW_MAX_STAGES;
    rg.gfull = bars + 2 * FW_MAX_STAGES;
    rg.gempty = bars + 2 * FW_MAX_STAGES + FW_MAX_SLOTS;
    rg.ring = smem + gm.off_ring;
    int* s_ctl = reinterpret_cast<int*>(smem + 1024 - 64);  // small control words (inside the barrier page)
    float* xs = reinterpret_cast<float*>(smem + gm.off_xs);
    uint32_t* xa_s = reinterpret_cast<uint32_t*>(smem + gm.off_xa);
    uint32_t* xb_s = reinterpret_cast<uint32_t*>(smem + gm.off_xb);
    float* blk_s = reinterpret_cast<float*>(smem + gm.off_blk);  // [3][H/32]: step, sum, abs
    float* red = reinterpret_cast<float*>(smem + gm.off_red);
    float* wpart = reinterpret_cast<float*>(smem + gm.off_wpart);
    float* my_scores = reinterpret_cast<float*>(smem + gm.off_scores);
    int* in_list = reinterpret_cast<int*>(smem + gm.off_lists);
    int* band_list = in_list + gm.max_slots;
    float* band_ex = reinterpret_cast<float*>(band_list + gm.max_slots);
    int* g2_rows = reinterpret_cast<int*>(band_ex + gm.max_slots);         // [2 * max_slots] global rows of the second gather
    float* g2_scores = reinterpret_cast<float*>(g2_rows + 2 * gm.max_slots);  // [2 * max_slots] their gate scores

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_producer = tid >= FW_CONSUMERS;
    const int hidden = gm.nsb * 256, nblk = gm.nsb * 8;
    const int R = gm.R, P = gm.P;
    const int n_tiles = (a.n_rows + R - 1) / R;
    const int first_tile = blockIdx.x;
    const int my_count = first_tile < n_tiles ? (n_tiles - first_tile + gridDim.x - 1) / gridDim.x : 0;
    const int n_slots = my_count * R;

    if (tid == 0) {
        s_ctl[6] = 0;
        for (int i = 0; i < gm.S; ++i) {
            mbar_init(&rg.full[i], 1);
            mbar_init(&rg.empty[i], FW_CONSUMERS);
        }
        for (int i = 0; i < gm.D; ++i) {
            mbar_init(&rg.gfull[i], 1);
            mbar_init(&rg.gempty[i], gm.TS);
        }
        fence_mbar_init();
    }
    __syncthreads();

    uint32_t scan_it = 0, g_it = 0;
    bool failed = false;

    if (is_producer) {
        // ------------------------------------------------------------ producer warp
        for (int l = 0; l < a.n_layers; ++l) {
            const FusedLayer ly = a.layers ? a.layers[l] : a.single;
            for (int k = 0; k < my_count; ++k) {
                const uint32_t it = scan_it + k;
                const int stg = it % gm.S;
                if (it >= (uint32_t)gm.S && !failed && !mbar_wait(&rg.empty[stg], ((it / gm.S) - 1) & 1)) failed = true;
                if (lane == 0) {
                    const int row0 = (first_tile + k * (int)gridDim.x) * R;
                    const uint32_t bytes = (uint32_t)min(R, a.n_rows - row0) * (uint32_t)gm.row_bytes;
                    mbar_expect_tx(&rg.full[stg], bytes);
                    tma_bulk_g2s(rg.ring + (size_t)stg * gm.tile_bytes, ly.gate + (size_t)row0 * gm.row_bytes, bytes,
                                 &rg.full[stg]);
                }
            }
            scan_it += my_count;
            bar_sync(FW_BAR_ALL, FW_THREADS);  // A: certainly-in list ready
            // the gather ring aliases the scan ring: wait until every scan tile has been consumed
            for (uint32_t it = scan_it > (uint32_t)gm.S ? scan_it - gm.S : 0; it < scan_it; ++it)
                if (!failed && !mbar_wait(&rg.empty[it % gm.S], (it / gm.S) & 1)) failed = true;
            producer_gather(rg, gm, ly, in_list, false,
                            min(s_ctl[0], (a.top_k + (int)gridDim.x - 1) / (int)gridDim.x + 2), g_it, first_tile, lane,
                            failed);
            bar_sync(FW_BAR_ALL, FW_THREADS);  // B: band winners ready (ring is idle: the pick staged in it)
            producer_gather(rg, gm, ly, g2_rows, true, s_ctl[2], g_it, first_tile, lane, failed);
            bar_sync(FW_BAR_ALL, FW_THREADS);  // C: every gather slot consumed -> next layer's tiles may land
        }
        if (failed) set_err(a.err, DEV_ERR_TMA_TIMEOUT);
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int team = tid / gm.TS, c = tid % gm.TS, wt = c >> 5;
    const bool in_team = team < P;
    const bool active = in_team && c < gm.G;
    const int s = c >> 2, g = c & 3;
    uint32_t epoch = 0;
    const float* h_cur = a.h_in;

    for (int l = 0; l < a.n_layers; ++l) {
        const FusedLayer ly = a.layers ? a.layers[l] : a.single;
        const int par = l & 1;
        uint32_t* hist = a.hist + (size_t)par * LQ_HIST_BINS;
        float* h_next = (l + 1 == a.n_layers) ? a.h_out : (par ? a.hbuf1 : a.hbuf0);

        FW_STAMP(0);
        // ---- 0. prepare the activation: one thread per 32-element block ---------------------
        {
            const int n_blk32 = 2 * gm.G;
            double sq = 0.0;
            for (int blk = tid; blk < n_blk32; blk += FW_CONSUMERS) {
                float* xdst = xs + (blk >> 1) * 68 + (blk & 1) * 32;
                const float4* src = reinterpret_cast<const float4*>(h_cur + (size_t)blk * 32);
                float4 t[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) t[j] = __ldcg(src + j);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    *reinterpret_cast<float4*>(xdst + 4 * j) = t[j];
                    sq += (double)t[j].x * (double)t[j].x + (double)t[j].y * (double)t[j].y;
                    sq += (double)t[j].z * (double)t[j].z + (double)t[j].w * (double)t[j].w;
                }
            }
            float rms = 1.0f;
            if (a.flags & LQ_WALK_RMSNORM) {
                double* dred = reinterpret_cast<double*>(red);
                for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (lane == 0) dred[warp] = sq;
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                double t = 0.0;
                for (int w = 0; w < FW_NWARPS; ++w) t += dred[w];
                rms = (float)sqrt(t / (double)hidden + 1e-6);
            }
            bool bad = false;
            for (int blk = tid; blk < n_blk32; blk += FW_CONSUMERS) {
                const int cc = blk >> 1, hb = blk & 1;
                float* xdst = xs + cc * 68 + hb * 32;
                float v[32];
                float amax = 0.0f, sum = 0.0f, asum = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 t = *reinterpret_cast<const float4*>(xdst + 4 * j);
                    v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (a.flags & LQ_WALK_RMSNORM) v[j] = __fdiv_rn(v[j], rms);
                    bad |= !isfinite(v[j]);
                    amax = fmaxf(amax, fabsf(v[j]));
                    sum += v[j];
                    asum += fabsf(v[j]);
                }
                const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
                blk_s[blk] = amax / 32767.0f;
                blk_s[nblk + blk] = sum;
                blk_s[2 * nblk + blk] = asum;
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    uint32_t wa = 0, wb = 0;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        int q = __float2int_rn(v[4 * j4 + b] * inv);
                        q = max(-32767, min(32767, q));
                        wa |= (uint32_t)((q >> 8) & 0xff) << (8 * b);
                        wb |= (uint32_t)(q & 0xff) << (8 * b);
                    }
                    xa_s[(hb * 8 + j4) * gm.G + cc] = wa;
                    xb_s[(hb * 8 + j4) * gm.G + cc] = wb;
                    *reinterpret_cast<float4*>(xdst + 4 * j4) =
                        make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
                }
            }
            if (bad) set_err(a.err, DEV_ERR_NAN_SCORE);
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);

        FW_STAMP(1);
        // ---- 1. scan this CTA's gate tiles --------------------------------------------
        {
            CellX x;
            float ab_lo = 0.0f, ab_hi = 0.0f, bmax = 0.0f;
            uint32_t kmax = 0;
            if (active) {
                load_cellx(x, xa_s, xb_s, blk_s, nblk, s * 8 + 2 * g, gm.G, c);
                ab_lo = blk_s[2 * nblk + s * 8 + 2 * g];
                ab_hi = blk_s[2 * nblk + s * 8 + 2 * g + 1];
            }
            for (int k = 0; k < my_count; ++k) {
                const uint32_t it = scan_it + k;
                const int stg = it % gm.S;
                if (!failed && !mbar_wait(&rg.full[stg], (it / gm.S) & 1)) failed = true;
                const int row0 = (first_tile + k * (int)gridDim.x) * R;
                const int rows_here = min(R, a.n_rows - row0);
                const uint8_t* tb = rg.ring + (size_t)stg * gm.tile_bytes;
                float* wp = wpart + (size_t)(k & 1) * P * gm.Rt * gm.Wt;
                if (in_team) {
                    for (int j = 0; j < gm.Rt; ++j) {
                        const int r = team + j * P;
                        float val = 0.0f;
                        if (active && r < rows_here) {
                            float b = 0.0f;
                            val = cell_dot(tb + (size_t)r * gm.row_bytes + s * 144, g, x, ab_lo, ab_hi, a.c1, b);
                            bmax = fmaxf(bmax, b);
                        }
                        for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
                        if (lane == 0) wp[(team * gm.Rt + j) * gm.Wt + wt] = val;
                    }
                }
                mbar_arrive(&rg.empty[stg]);
                if (in_team) {
                    bar_sync(1 + team, gm.TS);
                    if (c < gm.Rt) {
                        const int r = team + c * P;
                        float sc = 0.0f;
                        for (int w = 0; w < gm.Wt; ++w) sc += wp[(team * gm.Rt + c) * gm.Wt + w];
                        my_scores[k * R + r] = sc;
                        if (r < rows_here) {
                            if (sc != sc) set_err(a.err, DEV_ERR_NAN_SCORE);
                            const uint32_t bin = __float_as_uint(fabsf(sc)) >> LQ_HIST_SHIFT;
                            atomicAdd(&hist[bin], 1u);
                            kmax = max(kmax, bin);
                        }
                    }
                }
            }
            scan_it += my_count;
            // bound: sum over the team's cells of each thread's largest cell bound
            if (in_team) {
                for (int o = 16; o > 0; o >>= 1) bmax += __shfl_xor_sync(0xffffffffu, bmax, o);
                float* wb = red + team * gm.Wt;
                if (lane == 0) wb[wt] = bmax;
                bar_sync(1 + team, gm.TS);
                if (c == 0) {
                    float t = 0.0f;
                    for (int w = 0; w < gm.Wt; ++w) t += wb[w];
                    if (t > 0.0f) atomicMax(&a.ctrs[CTR_BOUND0 + par], __float_as_uint(t));
                }
                if (c < gm.Rt && kmax > 0u) atomicMax(&a.ctrs[CTR_MAXBIN0 + par], kmax);
            }
            if (tid == 0) {
                s_ctl[4] = 0;
                s_ctl[7] = 0;
            }
        }
        FW_STAMP(2);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[6]);
        FW_STAMP(3);

        // ---- 2. threshold bucket from the global histogram -----------------------------
        float hi, lo, B;
        {
            // Read the histogram from the highest occupied bin downwards, 1024 bins per round
            // (256 threads x 4 bins, thread 0 the highest), until the cumulative count reaches K.
            constexpr int HT = 256;
            const uint32_t bbits = __ldcg(&a.ctrs[CTR_BOUND0 + par]);
            const uint32_t maxbin = min(__ldcg(&a.ctrs[CTR_MAXBIN0 + par]), (uint32_t)LQ_HIST_BINS - 1u);
            const uint32_t K = (uint32_t)a.top_k;
            uint32_t* wsum = reinterpret_cast<uint32_t*>(red);
            uint32_t above_total = 0;
            for (int base_end = (int)(maxbin / 4u + 1u) * 4; base_end > 0; base_end -= 4 * HT) {
                const int b0 = base_end - 4 * (tid + 1);
                uint4 t4 = make_uint4(0u, 0u, 0u, 0u);
                if (tid < HT && b0 >= 0) t4 = __ldcg(reinterpret_cast<const uint4*>(hist + b0));
                const uint32_t own = t4.x + t4.y + t4.z + t4.w;
                uint32_t pre = own;  // inclusive prefix in thread order (higher bins first)
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t v = __shfl_up_sync(0xffffffffu, pre, o);
                    if (lane >= o) pre += v;
                }
                if (lane == 31) wsum[warp] = pre;
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                uint32_t lower = 0, chunk_total = 0;
                for (int w = 0; w < HT / 32; ++w) {
                    const uint32_t v = wsum[w];
                    if (w < warp) lower += v;
                    chunk_total += v;
                }
                const uint32_t incl = above_total + lower + pre, excl = incl - own;
                if (tid < HT && excl < K && K <= incl) {
                    uint32_t acc = excl;
                    int b = 3;
                    const uint32_t bins4[4] = {t4.x, t4.y, t4.z, t4.w};
                    for (; b > 0; --b) {
                        if (acc + bins4[b] >= K) break;
                        acc += bins4[b];
                    }
                    s_ctl[4] = b0 + b;
                    s_ctl[7] = 1;
                }
                above_total += chunk_total;
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                if (s_ctl[7]) break;
            }
            const uint32_t bstar = (uint32_t)s_ctl[4];
            B = __uint_as_float(bbits);
            const float t_lo = __uint_as_float(bstar << LQ_HIST_SHIFT);
            const uint32_t hb = (bstar + 1u) << LQ_HIST_SHIFT;
            const float t_hi = __uint_as_float(hb > 0x7F800000u ? 0x7F800000u : hb);
            const float two_b = __fmul_ru(2.0f, B);
            hi = __fadd_ru(t_hi, two_b);
            lo = __fadd_rd(t_lo, -two_b);
            if (l + 1 == a.n_layers && a.stats && blockIdx.x == 0 && tid == 0) {
                a.stats->tau = t_lo;
                a.stats->bound = B;
            }
        }

        // ---- classify own rows (ordered compaction over the score slots) ---------------
        {
            int* wcnt = reinterpret_cast<int*>(red) + 64;  // [2][16]
            const int chunk = (n_slots + FW_NWARPS - 1) / FW_NWARPS;
            const int chunk32 = (chunk + 31) / 32 * 32;
            const int beg = warp * chunk32, end = min(n_slots, beg + chunk32);
            auto cls = [&](int m) -> int {
                const int row = (first_tile + (m / R) * (int)gridDim.x) * R + (m % R);
                if (row >= a.n_rows) return 0;
                const float v = fabsf(my_scores[m]);
                return v > hi ? 1 : (v >= lo ? 2 : 0);
            };
            int ca = 0, cb = 0;
            for (int m0 = beg; m0 < end; m0 += 32) {
                const int m = m0 + lane;
                const int cc = m < end ? cls(m) : 0;
                ca += __popc(__ballot_sync(0xffffffffu, cc == 1));
                cb += __popc(__ballot_sync(0xffffffffu, cc == 2));
            }
            if (lane == 0) {
                wcnt[warp] = ca;
                wcnt[16 + warp] = cb;
            }
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
            int oa = 0, ob = 0, ta = 0, tb2 = 0;
            for (int w = 0; w < FW_NWARPS; ++w) {
                if (w < warp) {
                    oa += wcnt[w];
                    ob += wcnt[16 + w];
                }
                ta += wcnt[w];
                tb2 += wcnt[16 + w];
            }
            for (int m0 = beg; m0 < end; m0 += 32) {
                const int m = m0 + lane;
                const int cc = m < end ? cls(m) : 0;
                const uint32_t ba = __ballot_sync(0xffffffffu, cc == 1), bb = __ballot_sync(0xffffffffu, cc == 2);
                const uint32_t lt = (1u << lane) - 1u;
                if (cc == 1) in_list[oa + __popc(ba & lt)] = m;
                if (cc == 2) band_list[ob + __popc(bb & lt)] = m;
                oa += __popc(ba);
                ob += __popc(bb);
            }
            if (tid == 0) {
                s_ctl[0] = ta;   // certainly-in rows of this CTA
                s_ctl[1] = tb2;  // band rows of this CTA
            }
        }
        bar_sync(FW_BAR_ALL, FW_THREADS);  // A
        FW_STAMP(4);
        const int n_in_mine = s_ctl[0], n_band_mine = s_ctl[1];

        // ---- exact re-score of own band rows (one warp per row), publish them ----------
        for (int i = warp; i < n_band_mine; i += FW_NWARPS) {
            const int m = band_list[i];
            const size_t row = (size_t)(first_tile + (m / R) * (int)gridDim.x) * R + (m % R);
            // per-warp scratch for super-block partials lives in wpart (idle between scan and gather)
            const float v = exact_row_q4k(ly.gate + row * gm.row_bytes, xs, gm.nsb, red + 256 + warp * gm.nsb, lane);
            if (lane == 0) band_ex[i] = v;
        }
        if (tid == 0) {
            atomicAdd(&a.ctrs[CTR_IN], (uint32_t)n_in_mine);
            s_ctl[3] = n_band_mine ? (int)atomicAdd(&a.ctrs[CTR_BAND], (uint32_t)n_band_mine) : 0;
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        {
            const int base = s_ctl[3];
            for (int i = tid; i < n_band_mine; i += FW_CONSUMERS) {
                const int m = band_list[i];
                const float v = band_ex[i];
                if (v != v) set_err(a.err, DEV_ERR_NAN_SCORE);
                a.band_row[base + i] = (uint32_t)((first_tile + (m / R) * (int)gridDim.x) * R + (m % R));
                a.band_exact[base + i] = v;
            }
        }

        // A CTA gathers at most its fair share (+2) of certainly-in rows itself; the rest goes to a pool
        // that all CTAs share out after the next barrier, so one heavy CTA does not hold everybody up.
        const int n_fair = (a.top_k + (int)gridDim.x - 1) / (int)gridDim.x + 2;
        const int n_keep = min(n_in_mine, n_fair), n_over = n_in_mine - n_keep;
        {
            uint32_t* pr = a.pool_row + (size_t)blockIdx.x * gm.max_slots;
            float* ps = a.pool_score + (size_t)blockIdx.x * gm.max_slots;
            for (int i = tid; i < n_over; i += FW_CONSUMERS) {
                const int m = in_list[n_keep + i];
                pr[i] = (uint32_t)((first_tile + (m / R) * (int)gridDim.x) * R + (m % R));
                ps[i] = my_scores[m];
            }
            if (tid == 0) a.pool_cnt[blockIdx.x] = (uint32_t)n_over;
        }

        FW_STAMP(5);
        // ---- gather the certainly-in rows ---------------------------------------------
        float acc_lo[32], acc_hi[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc_lo[j] = acc_hi[j] = 0.0f;
        float corr_lo = 0.0f, corr_hi = 0.0f;
        if (in_team)
            consumer_gather(rg, gm, in_list, n_keep, my_scores, g_it, xa_s, xb_s, blk_s, wpart, team, c, active,
                            acc_lo, acc_hi, corr_lo, corr_hi, failed);
        else
            g_it += n_keep;
        FW_STAMP(6);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[6]);
        FW_STAMP(7);

        // ---- 3. final pick among all band rows, identically in every CTA ---------------
        {
            const int n_in_tot = (int)__ldcg(&a.ctrs[CTR_IN]);
            const int n_band_tot = min((int)__ldcg(&a.ctrs[CTR_BAND]), a.n_rows);
            const int need = a.top_k - n_in_tot;
            uint32_t tau_key = 0, row_cut = 0xffffffffu;
            bool take_all = need >= n_band_tot;
            // Small bands (the usual case): every CTA ranks its own band rows against all band
            // entries by counting; large bands fall back to a radix select of the threshold.
            const bool by_rank = !take_all && need > 0 && n_band_tot <= FW_RANK_CAP;
            int* win_s = reinterpret_cast<int*>(rg.ring + FW_PICK_CAP * 8);
            if (!take_all && need > 0) {
                // stage (|v| key, row) of every band entry in the idle ring
                uint32_t* keys = reinterpret_cast<uint32_t*>(rg.ring);
                uint32_t* rows = keys + FW_PICK_CAP;
                const bool staged = n_band_tot <= FW_PICK_CAP;
                if (staged) {
                    for (int i = tid; i < n_band_tot; i += FW_CONSUMERS) {
                        keys[i] = abs_key(__ldcg(&a.band_exact[i]));
                        rows[i] = __ldcg(&a.band_row[i]);
                    }
                    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                }
                if (by_rank) {
                    for (int i = warp; i < n_band_mine; i += FW_NWARPS) {
                        const int m = band_list[i];
                        const uint32_t key = abs_key(band_ex[i]);
                        const uint32_t row = (uint32_t)((first_tile + (m / R) * (int)gridDim.x) * R + (m % R));
                        int ahead = 0;  // entries that order before this one under (|v| desc, row asc)
                        for (int j = lane; j < n_band_tot; j += 32) {
                            const uint32_t kj = keys[j];
                            ahead += (kj > key || (kj == key && rows[j] < row)) ? 1 : 0;
                        }
                        for (int o = 16; o > 0; o >>= 1) ahead += __shfl_xor_sync(0xffffffffu, ahead, o);
                        if (lane == 0) win_s[i] = ahead < need ? 1 : 0;
                    }
                    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                } else {
                    SelectSmem<FW_CONSUMERS>& sm =
                        *reinterpret_cast<SelectSmem<FW_CONSUMERS>*>(rg.ring + FW_PICK_CAP * 8);
                    int cnt_gt, need_eq;
                    auto keyf = [&](int i) -> uint32_t { return staged ? keys[i] : abs_key(__ldcg(&a.band_exact[i])); };
                    block_kth_largest_keys<FW_CONSUMERS, FW_BAR_CONS>(keyf, n_band_tot, need, sm, tau_key, cnt_gt, need_eq);
                    // ties at the threshold: the need_eq lowest rows win
                    auto rowf = [&](int i) -> uint32_t {
                        if (keyf(i) != tau_key) return 0u;
                        return ~(staged ? rows[i] : __ldcg(&a.band_row[i]));
                    };
                    uint32_t cut_key;
                    int c2, n2;
                    block_kth_largest_keys<FW_CONSUMERS, FW_BAR_CONS>(rowf, n_band_tot, need_eq, sm, cut_key, c2, n2);
                    row_cut = ~cut_key;
                    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                }
            }
            // winners among this CTA's band rows, in slot order
            if (warp == 0) {
                int cnt = 0;
                for (int i0 = 0; i0 < n_band_mine; i0 += 32) {
                    const int i = i0 + lane;
                    bool win = false;
                    int m = 0;
                    if (i < n_band_mine && need > 0) {
                        m = band_list[i];
                        const uint32_t key = abs_key(band_ex[i]);
                        const uint32_t row = (uint32_t)((first_tile + (m / R) * (int)gridDim.x) * R + (m % R));
                        win = by_rank ? (win_s[i] != 0)
                                      : (take_all || key > tau_key || (key == tau_key && row <= row_cut));
                    }
                    const uint32_t bal = __ballot_sync(0xffffffffu, win);
                    if (win) {
                        const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
                        g2_rows[pos] = (first_tile + (m / R) * (int)gridDim.x) * R + (m % R);
                        g2_scores[pos] = band_ex[i];  // the gather uses the exact gate score
                    }
                    cnt += __popc(bal);
                }
                if (lane == 0) s_ctl[2] = cnt;
            }
            // this CTA's share of the pooled certainly-in rows: pool items j = cta, cta + grid, ... of the
            // per-CTA segments taken in CTA order (a fixed order: results stay run-to-run identical)
            {
                const int NC = (int)gridDim.x;
                int* prefix = reinterpret_cast<int*>(red) + 1280;  // [NC + 1]
                int* wtot = reinterpret_cast<int*>(red) + 1200;    // [FW_NWARPS]
                int inc = tid < NC ? (int)__ldcg(&a.pool_cnt[tid]) : 0;
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += v;
                }
                if (lane == 31) wtot[warp] = inc;
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                int lower = 0;
                for (int w = 0; w < warp; ++w) lower += wtot[w];
                if (tid < NC) prefix[tid + 1] = lower + inc;
                if (tid == 0) prefix[0] = 0;
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                const int total = prefix[NC], n_win = s_ctl[2];
                const int n_pool_mine = total > (int)blockIdx.x ? (total - (int)blockIdx.x + NC - 1) / NC : 0;
                for (int i = tid; i < n_pool_mine; i += FW_CONSUMERS) {
                    const int j = (int)blockIdx.x + i * NC;
                    int sa = 0, sb = NC;  // prefix[sa] <= j < prefix[sb]
                    while (sb - sa > 1) {
                        const int mid = (sa + sb) >> 1;
                        if (prefix[mid] <= j) sa = mid;
                        else sb = mid;
                    }
                    const size_t src = (size_t)sa * gm.max_slots + (size_t)(j - prefix[sa]);
                    g2_rows[n_win + i] = (int)__ldcg(&a.pool_row[src]);
                    g2_scores[n_win + i] = __ldcg(&a.pool_score[src]);
                }
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                if (tid == 0) s_ctl[2] = n_win + n_pool_mine;
            }
            if (l + 1 == a.n_layers && a.stats && blockIdx.x == 0 && tid == 0) {
                a.stats->n_certain = n_in_tot;
                a.stats->n_band = n_band_tot;
                a.stats->n_hits = min(a.top_k, a.n_rows);
                a.stats->need = need;
            }
            if (l + 1 == a.n_layers && a.count_out && blockIdx.x == 0 && tid == 0)
                *a.count_out = (uint32_t)min(a.top_k, a.n_rows);
        }
        // the pick staged plain stores in the ring; order them before the TMA writes that follow
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        bar_sync(FW_BAR_ALL, FW_THREADS);  // B
        FW_STAMP(8);
        const int n_g2 = s_ctl[2];
        if (in_team)
            consumer_gather(rg, gm, nullptr, n_g2, g2_scores, g_it, xa_s, xb_s, blk_s, wpart, team, c, active, acc_lo,
                            acc_hi, corr_lo, corr_hi, failed);
        else
            g_it += n_g2;
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // every team has finished reading its gather slots
        FW_STAMP(9);

        // optional: selected rows of the last layer (unordered)
        if (l + 1 == a.n_layers && a.hit_out) {
            if (tid == 0) s_ctl[5] = (int)atomicAdd(&a.ctrs[CTR_HITS], (uint32_t)(n_keep + n_g2));
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
            const int base = s_ctl[5];
            for (int i = tid; i < n_keep + n_g2; i += FW_CONSUMERS) {
                uint32_t row;
                if (i < n_keep) {
                    const int m = in_list[i];
                    row = (uint32_t)((first_tile + (m / R) * (int)gridDim.x) * R + (m % R));
                } else {
                    row = (uint32_t)g2_rows[i - n_keep];
                }
                if (base + i < a.top_k) a.hit_out[base + i] = row;
            }
        }

        // ---- partial out[H] of this CTA: the teams' accumulators, summed in team order ---------
        {
            // one region per team in the idle ring, 64-float chunks at a stride of 65
            float* out_r = reinterpret_cast<float*>(rg.ring);
            const int region = gm.G * 65;
            if (active) {
                float* o_lo = out_r + team * region + c * 65;
                float* o_hi = o_lo + 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    o_lo[j] = acc_lo[j] - corr_lo;
                    o_hi[j] = acc_hi[j] - corr_hi;
                }
            }
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
            float* dst = a.partials + (size_t)blockIdx.x * hidden;
            for (int i = tid; i < hidden; i += FW_CONSUMERS) {
                const int o = (i >> 6) * 65 + (i & 63);
                float v = out_r[o];
                for (int p = 1; p < P; ++p) v += out_r[p * region + o];
                dst[i] = v;
            }
        }
        // the merge used the ring with plain loads and stores; order them before the TMA writes of
        // the next layer's tiles
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        bar_sync(FW_BAR_ALL, FW_THREADS);  // C: the ring is free for the next layer's tiles
        // housekeeping for the layer after next (nobody reads these before two more grid barriers)
        for (int i = blockIdx.x * FW_CONSUMERS + tid; i < LQ_HIST_BINS; i += gridDim.x * FW_CONSUMERS) hist[i] = 0;
        if (blockIdx.x == 0 && tid == 0) {
            a.ctrs[CTR_BOUND0 + par] = 0;
            a.ctrs[CTR_MAXBIN0 + par] = 0;
        }
        FW_STAMP(10);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[6]);
        FW_STAMP(11);

        // ---- 4. finish: fixed-order sum of a column slice of the partials + residual ----
        {
            const int ncol4 = hidden / 4;
            const int per = (ncol4 + gridDim.x - 1) / gridDim.x;      // float4 columns per CTA
            const int col0 = blockIdx.x * per, ncol = max(0, min(per, ncol4 - col0));
            const int ygroups = max(1, min(FW_CONSUMERS / max(per, 1), 64));
            float4* red4 = reinterpret_cast<float4*>(red);            // [ygroups][per] (<= 512 entries)
            const int j = tid % per, y = tid / per;
            if (y < ygroups && j < ncol) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int p = y; p < (int)gridDim.x; p += ygroups) {
                    const float4 t = __ldcg(reinterpret_cast<const float4*>(a.partials + (size_t)p * hidden) + col0 + j);
                    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
                }
                red4[y * per + j] = acc;
            }
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
            if (tid < ncol) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int yy = 0; yy < ygroups; ++yy) {
                    const float4 v = red4[yy * per + tid];
                    t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
                }
                if (a.flags & LQ_WALK_RESIDUAL) {
                    const float4 hres = __ldcg(reinterpret_cast<const float4*>(h_cur) + col0 + tid);
                    t.x += hres.x; t.y += hres.y; t.z += hres.z; t.w += hres.w;
                }
                reinterpret_cast<float4*>(h_next)[col0 + tid] = t;
            }
            if (blockIdx.x == 0 && tid == 0) {
                a.ctrs[CTR_IN] = 0;
                a.ctrs[CTR_BAND] = 0;
            }
        }
        FW_STAMP(12);
        h_cur = h_next;
        if (l + 1 < a.n_layers) grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[6]);
    }
    if (failed) set_err(a.err, DEV_ERR_TMA_TIMEOUT);
}

}  // namespace

// Host side ------------------------------------------------------------------------
struct FusedPlan {
    FusedGeom geom;
    int grid;
};

bool fused_q4k_supported(int hidden, int n_rows, int top_k, int sm_count) {
    FusedGeom g;
    if (n_rows <= 0 || top_k <= 0 || top_k >= n_rows) return false;
    if (!fused_geom(hidden, n_rows, sm_count, g)) return false;
    const int per = (hidden / 4 + sm_count - 1) / sm_count;
    return per <= FW_CONSUMERS && g.max_slots <= 16384;
}

size_t fused_q4k_ws_bytes(int hidden, int n_rows, int sm_count) {
    FusedGeom g;
    size_t pool = 0;
    if (fused_geom(hidden, n_rows, sm_count, g)) pool = ((size_t)sm_count * g.max_slots * 4 + 255) / 256 * 256;
    return (size_t)2 * LQ_HIST_BINS * 4 + CTR_WORDS * 4 + (size_t)n_rows * 8 + 2 * pool + 4096 +
           (size_t)sm_count * hidden * 4 + (size_t)2 * hidden * 4 + 4096;
}

// ws: fused_q4k_ws_bytes() of zero-initialised device memory, 256-byte aligned.  layers_dev:
// n_layers x {gate, up, down} device pointers in device memory.
cudaError_t launch_walk_fused_q4k(const void* layers_dev, const uint8_t* const* single, int n_layers, int n_rows,
                                  int hidden, int top_k,
                                  uint32_t flags, float c1, const float* h_in, float* h_out, uint8_t* ws,
                                  uint32_t* hit_out, uint32_t* count_out, lq_walk_stats* stats_dev, int* err,
                                  int sm_count, cudaStream_t st) {
    FusedGeom g;
    if (!fused_geom(hidden, n_rows, sm_count, g)) return cudaErrorInvalidValue;
    const int n_tiles = (n_rows + g.R - 1) / g.R;
    const int grid = sm_count < n_tiles ? sm_count : n_tiles;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(walk_fused_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    FusedArgs a;
    a.layers = reinterpret_cast<const FusedLayer*>(layers_dev);
    a.single = single ? FusedLayer{single[0], single[1], single[2]} : FusedLayer{nullptr, nullptr, nullptr};
    a.n_layers = n_layers;
    a.n_rows = n_rows;
    a.top_k = top_k;
    a.flags = flags;
    a.c1 = c1;
    a.h_in = h_in;
    a.h_out = h_out;
    uint8_t* p = ws;
    a.hist = reinterpret_cast<uint32_t*>(p);        p += (size_t)2 * LQ_HIST_BINS * 4;
    a.ctrs = reinterpret_cast<uint32_t*>(p);        p += 256;
    a.band_row = reinterpret_cast<uint32_t*>(p);    p += ((size_t)n_rows * 4 + 255) / 256 * 256;
    a.band_exact = reinterpret_cast<float*>(p);     p += ((size_t)n_rows * 4 + 255) / 256 * 256;
    const size_t pool = ((size_t)sm_count * g.max_slots * 4 + 255) / 256 * 256;
    a.pool_row = reinterpret_cast<uint32_t*>(p);    p += pool;
    a.pool_score = reinterpret_cast<float*>(p);     p += pool;
    a.pool_cnt = reinterpret_cast<uint32_t*>(p);    p += 4096;
    a.hbuf0 = reinterpret_cast<float*>(p);          p += (size_t)hidden * 4;
    a.hbuf1 = reinterpret_cast<float*>(p);          p += (size_t)hidden * 4;
    a.partials = reinterpret_cast<float*>(p);
    a.hit_out = hit_out;
    a.count_out = count_out;
    a.stats = stats_dev;
    a.phase_ns = stats_dev ? reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(stats_dev) + 64) : nullptr;
    a.err = err;
    // the barrier counter and the per-launch counters start from zero (the histogram is kept
    // zero by the kernel itself; a failed launch is followed by a full clear on the host side)
    cudaError_t e = cudaMemsetAsync(a.ctrs, 0, 256, st);
    if (e != cudaSuccess) return e;
    void* args[] = {&g, &a};
    e = cudaLaunchCooperativeKernel((const void*)walk_fused_q4k_kernel, dim3(grid), dim3(FW_THREADS), args,
                                    (size_t)g.smem_bytes, st);
    return e;
}

}  // namespace lq
