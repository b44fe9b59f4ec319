// Fused persistent Q4_K walk for one token: every layer of a stack in ONE cooperative
// launch, one CTA per SM, four grid barriers per layer.
//
// Per layer each CTA
//   0. RMS-normalises the residual and builds the 16-bit fixed-point copy of it in shared
//      memory, all consumer threads in parallel (rms_norm_eps,
//      crates/larql-compute/src/residual.rs:56-78), together with the per-block constants of
//      the score error bound, which use the MEASURED fixed-point error of each block;
//   1. scans its share of the gate rows (tiles of whole rows, TMA bulk copies into a
//      shared-memory ring, issued by one thread a few tiles ahead), keeps the fast scores of
//      ITS rows in shared memory and adds their |score| keys to a global coarse histogram;
//      the first tiles of the NEXT layer's gate rows are prefetched into L2 (the weights do
//      not depend on the residual), so HBM keeps working through the phases below;
//      -- grid barrier A --
//   2. reads the histogram, finds the bucket [t_lo, t_hi) of the K-th largest |score| and,
//      with B the bound on |fast - reference|, splits its rows into certainly-in
//      (> t_hi + 2B), band (>= t_lo - 2B) and out; re-scores its band rows in the
//      reference's exact f32 order and publishes them;
//      -- grid barrier B --
//   3. picks, identically in every CTA, the K - n_in best band rows under (|score| desc,
//      row asc) (top_k_by_abs, crates/larql-vindex/src/index/compute/gate_knn/mod.rs:50-108);
//      gathers its certainly-in rows and the winners it owns (up dot, SiLU, down axpy —
//      walk_ffn_sparse, crates/larql-inference/src/vindex/walk_ffn/sparse.rs:218-289): every
//      thread fetches its own 48-byte pieces of the rows (down rows by cp.async into the idle
//      ring, up rows into registers), all up dots first, then all down rows; writes its
//      partial out[H];
//      -- grid barrier C --
//   4. sums a column slice of the partials in fixed order, adds the residual (run_ffn,
//      crates/larql-compute/src/forward/layer.rs:109-124) and writes the next residual.
//      -- grid barrier D --
// A row is scanned, classified, re-scored and gathered by the CTA that streamed it, so no
// hit list travels between CTAs and the summation order is fixed: results are run-to-run
// identical.  Every wait (mbarrier, grid barrier) is bounded and reports through the error
// word instead of hanging.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/larql_cuda.h"
#include "q4k_exact.cuh"
#include "select.cuh"

namespace lq {

namespace {

// No separate producer warp: the last warp to release a ring stage refills it.
// Tuning knobs (compile time).  16 warps at 128 registers per thread beat 12 warps at 168 registers, and
// one row per thread and pass beats two interleaved: every phase of this kernel is latency bound, so
// resident warps count most.
#ifndef FW_CFG_THREADS
#define FW_CFG_THREADS 512
#endif
constexpr int FW_CONSUMERS = FW_CFG_THREADS;
constexpr int FW_THREADS = FW_CONSUMERS;
constexpr int FW_NWARPS = FW_CONSUMERS / 32;
constexpr int FW_BAR_CONS = 0;       // the whole CTA
constexpr int FW_MAX_STAGES = 8;
constexpr int FW_MAX_GROWS = 64;     // rows one gather chunk stages in the ring
constexpr float FW_NOISE_FLOOR = 1e-10f;  // ACTIVATION_NOISE_FLOOR, walk_config.rs:64
constexpr int FW_PICK_CAP = 8192;    // band entries the final pick can stage in shared memory
constexpr int FW_RANK_CAP = 2048;    // up to this many band entries the pick ranks by counting
constexpr int FW_STAMPS = 13;
constexpr int FW_MAX_WORLD = 8;              // ranks of one feature-sharded walk
// The |score| keys of a layer crowd into a few hundred neighbouring histogram bins, i.e. a handful of cache
// lines, and every CTA adds its rows at the same moment: the histogram is kept as FW_HIST_COPIES copies
// (a warp adds to copy (CTA + warp) mod copies, readers sum the copies) so that those adds spread over
// that many times more lines.
constexpr int FW_HIST_COPIES = 8;
constexpr int FW_HIST_WORDS = FW_HIST_COPIES * LQ_HIST_BINS;

struct FusedGeom {
    int nsb, G, TS, P, Wt;      // super-blocks/row, cells/row, team size, teams, warps per team
    int row_bytes, R, Rt;       // rows per scan tile, rows per team per tile
    int tile_bytes, S;          // scan ring
    int D2;                     // rows of one gather chunk (down rows staged in the idle ring)
    int E;                      // ring slots that may be filled before the final pick (the pick stages a small band behind them)
    int off_pick;               // where in the ring the pick stages a band of up to FW_RANK_CAP entries
    int max_slots;              // score slots per CTA (tiles per CTA * R)
    int off_xs, off_xa, off_xb, off_blk, off_wpart, off_psum, off_scores, off_lists, off_red, off_ring;
    int ring_bytes, smem_bytes;
};

struct FusedLayer {
    const uint8_t* gate;
    const uint8_t* up;
    const uint8_t* down;
};

// Feature-sharded walk over the GPUs of one box: every rank runs this kernel on its own row range and the
// ranks meet in each other's memory.  area[r] is rank r's exchange area as mapped into this process
// (area[rank]: this GPU's own), all laid out alike, in 16-byte LINES {word0, epoch, word1, epoch}:
//   meta  [world]                      score bound bits | highest occupied histogram bin of a rank's rows
//   cnt   [world]                      certainly-in rows | band rows of a rank
//   hist  [world][LQ_HIST_BINS / 2]    a rank's histogram, two bins per line
//   band  [n_rows_global]              band entries {global row | exact score}, rank r's from line row_offset(r) on
//   xsum  [world][hidden / 2]          a rank's partial layer output, two floats per line
// A rank writes its own slot of each array into EVERY rank's area with one 16-byte store per line; a reader
// (always reading its own GPU's memory) takes a line once both epoch words carry the layer's epoch, which only
// ever grows, across launches too.  Each 8-byte half of such a store arrives whole, so data and epoch cannot be
// torn apart and no fence or separate flag is needed: an exchange costs one trip over NVLink.  A slot is
// rewritten only after every reader is done with it, because a rank cannot get a layer ahead without the
// others' lines of the layer in between.
struct FusedPeers {
    int world, rank, row_offset, n_rows_global;
    uint32_t xepoch0;  // epoch of the last layer of the previous launch on these areas
    uint32_t off_meta, off_cnt, off_hist, off_band, off_xsum;
    uint32_t pad[2];
    int seg_off[FW_MAX_WORLD];  // row_offset of every rank
    uint8_t* area[FW_MAX_WORLD];
};

struct FusedArgs {
    const FusedLayer* layers;  // device array of n_layers entries, or nullptr: use `single`
    FusedLayer single;
    int n_layers, n_rows, top_k;
    uint32_t flags;
    float c1;
    int pf_tiles;          // tiles of the next layer's gate share each CTA prefetches into L2 during the tail
    int pf_late;           // 1: start that prefetch only after the gather (0: right after the scan)
    int pf_dist;           // tiles the L2 prefetch runs ahead of the ring inside a layer's scan
    int stamp_cta;         // the CTA whose clock stamps are recorded
    const float* h_in;
    float* h_out;
    float* hbuf0;
    float* hbuf1;
    uint32_t* hist;        // [2][FW_HIST_COPIES][LQ_HIST_BINS]
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
    unsigned long long* phase_ns;  // optional [FW_STAMPS]: clock stamps of CTA 0 in the stamped layer
    int* err;
    FusedPeers px;         // world == 1: unused
};

enum { CTR_SYNC = 0, CTR_BOUND0 = 1, CTR_BOUND1 = 2, CTR_IN = 3, CTR_BAND = 4, CTR_HITS = 5, CTR_MAXBIN0 = 6,
       CTR_MAXBIN1 = 7, CTR_BDONE = 8, CTR_WORDS = 16 };

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
    int off = 1024;  // mbarriers
    g.off_xs = off;      off += fw_align(4 * g.nsb * 68 * 4, 128);
    g.off_xa = off;      off += fw_align(hidden, 128);
    g.off_xb = off;      off += fw_align(hidden, 128);
    g.off_blk = off;     off += fw_align(4 * (hidden / 32) * 4, 128);
    g.off_red = off;     off += 8192 + 1024;
    // rows per tile: about 36 KB, a multiple of P
    int r = (36 * 1024) / g.row_bytes / g.P * g.P;
    if (r < g.P) r = g.P;
    if (r > 8 * g.P) r = 8 * g.P;
    g.R = r;
    g.Rt = r / g.P;
    g.tile_bytes = g.R * g.row_bytes;
    g.off_psum = off;    off += fw_align(FW_MAX_GROWS * g.Wt * 4, 128) + fw_align(FW_MAX_GROWS * 4, 128);
    const int n_tiles = (n_rows + g.R - 1) / g.R;
    const int grid = grid_hint < n_tiles ? grid_hint : (n_tiles > 0 ? n_tiles : 1);
    g.max_slots = ((n_tiles + grid - 1) / grid) * g.R;
    g.off_scores = off;  off += fw_align(g.max_slots * 4, 128);
    g.off_wpart = off;   off += fw_align(g.max_slots * g.Wt * 4, 128);  // per slot: one partial score per warp of its team
    g.off_lists = off;   off += fw_align(7 * g.max_slots * 4, 128);
    g.off_ring = off;
    const int budget = 224 * 1024;
    g.ring_bytes = (budget - off) / 128 * 128;
    if (g.ring_bytes < 2 * g.tile_bytes || g.ring_bytes < 2 * g.row_bytes) return false;
    if (g.ring_bytes < FW_PICK_CAP * 8 + 24 * 1024) return false;
    if (g.ring_bytes < g.P * g.G * 65 * 4) return false;  // the merge stages one out[H] per team in the ring
    g.S = g.ring_bytes / g.tile_bytes;
    if (g.S > FW_MAX_STAGES) g.S = FW_MAX_STAGES;
    g.D2 = g.ring_bytes / g.row_bytes;
    if (g.D2 > FW_MAX_GROWS) g.D2 = FW_MAX_GROWS;
    const int pick_small = fw_align(FW_RANK_CAP * 8 + g.max_slots * 4, 128);
    g.off_pick = g.ring_bytes - pick_small;
    g.E = g.off_pick / g.row_bytes;
    if (g.E > g.D2) g.E = g.D2;
    g.smem_bytes = off + g.ring_bytes;
    return true;
}

__device__ __forceinline__ unsigned long long gtimer() {
    return (unsigned long long)clock64();  // SM cycles (the accessor converts with the SM clock)
}
__device__ __forceinline__ void bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// One exchange line: two data words, each beside the epoch it belongs to.
__device__ __forceinline__ void line_store(void* p, uint32_t w0, uint32_t w1, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(w0), "r"(epoch), "r"(w1), "r"(epoch)
                 : "memory");
}
__device__ __forceinline__ bool line_load(const void* p, uint32_t epoch, uint32_t& w0, uint32_t& w1) {
    uint32_t e0, e1;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(e0), "=r"(w1), "=r"(e1) : "l"(p)
                 : "memory");
    return e0 == epoch && e1 == epoch;
}
// Waits (bounded: about a second, or until another CTA has recorded an error) for a line of this epoch.
// On failure the words read as zero and DEV_ERR_TMA_TIMEOUT is recorded.
// (The spin is out of line: it is inlined at dozens of places otherwise, and the sharded kernel's code must stay
// inside the instruction cache like the one-GPU kernel's.)
__device__ __noinline__ void line_spin(const void* p, uint32_t epoch, uint32_t& w0, uint32_t& w1, int* err);
__device__ __forceinline__ void line_wait(const void* p, uint32_t epoch, uint32_t& w0, uint32_t& w1, int* err) {
    if (line_load(p, epoch, w0, w1)) return;
    line_spin(p, epoch, w0, w1, err);
}
__device__ __noinline__ void line_spin(const void* p, uint32_t epoch, uint32_t& w0, uint32_t& w1, int* err) {
    if (line_load(p, epoch, w0, w1)) return;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!line_load(p, epoch, w0, w1)) {
        if (((++spins & 63u) == 0) && (clock64() - t0 > (1ll << 31) || *(volatile int*)err != 0)) {
            set_err(err, DEV_ERR_TMA_TIMEOUT);
            w0 = w1 = 0u;
            return;
        }
    }
}
// The same line of every rank's slot (rank r's at base + r * rank_stride): all loads are issued before any
// is looked at, so the usual case costs one round trip to L2 whatever the number of ranks.
__device__ __forceinline__ void lines_wait_ranks(const uint4* base, size_t rank_stride, int world, uint32_t epoch,
                                                 uint32_t (&w0)[FW_MAX_WORLD], uint32_t (&w1)[FW_MAX_WORLD], int* err) {
    bool ok = true;
#pragma unroll
    for (int r = 0; r < FW_MAX_WORLD; ++r) {
        w0[r] = w1[r] = 0u;
        if (r < world) ok &= line_load(base + (size_t)r * rank_stride, epoch, w0[r], w1[r]);
    }
    if (ok) return;
#pragma unroll
    for (int r = 0; r < FW_MAX_WORLD; ++r)
        if (r < world) line_wait(base + (size_t)r * rank_stride, epoch, w0[r], w1[r], err);
}
// size a multiple of 16, address 16-byte aligned; this GPU's own memory
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Grid barriers over all CTAs, counting arrivals in a global word that
// starts at zero with the launch.  Bounded: a wait gives up after about a second, or as soon as
// another CTA has recorded an error, and records DEV_ERR_TMA_TIMEOUT.
__device__ __forceinline__ void grid_arrive(uint32_t* ctr, bool failed) {
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    if (threadIdx.x == 0 && !failed) {
        __threadfence();
        atomicAdd(ctr, 1u);
    }
}
__device__ __forceinline__ void grid_wait(const uint32_t* ctr, uint32_t target, int* err, bool& failed, int* s_flag) {
    if (threadIdx.x == 0 && !failed) {
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (ld_acquire_u32(ctr) < target) {
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
__device__ __forceinline__ void grid_sync(uint32_t* ctr, uint32_t& epoch, int* err, bool& failed, int* s_flag) {
    epoch += 1;
    grid_arrive(ctr, failed);
    grid_wait(ctr, epoch * gridDim.x, err, failed, s_flag);
}

// One Q4_K cell (64 weights) against the thread's activation planes: fast value and bound.
// Per 32-element block: st = fixed-point step, su = sum of x, bu / bv = bound constants (see the
// prepare phase): |fast - reference| of a row <= sum over its blocks of |d| sc bu + |dmin| m bv.
struct CellX {
    uint32_t xa_lo[8], xb_lo[8], xa_hi[8], xb_hi[8];
    float st_lo, st_hi, su_lo, su_hi, bu_lo, bu_hi, bv_lo, bv_hi;
};

__device__ __forceinline__ float cell_dot(const uint8_t* cell, int g, const CellX& x, float& bound) {
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
    bound = fabsf(d) * (sc_lo * x.bu_lo + sc_hi * x.bu_hi) + fabsf(dmin) * (m_lo * x.bv_lo + m_hi * x.bv_hi);
    return d * (sc_lo * dot_lo + sc_hi * dot_hi) - dmin * (m_lo * x.su_lo + m_hi * x.su_hi);
}

// The byte planes are stored word-major: word w (0..15, two 32-element blocks) of cell c sits
// at [w * G + c], so the lanes of a warp (consecutive cells) read consecutive words.
// blk: [4][nblk] = step, sum, bu, bv.
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
    x.bu_lo = blk[2 * nblk + blk_lo];
    x.bu_hi = blk[2 * nblk + blk_lo + 1];
    x.bv_lo = blk[3 * nblk + blk_lo];
    x.bv_hi = blk[3 * nblk + blk_lo + 1];
}

// One cell (registers) against the thread's activation planes: the fast value only.
__device__ __forceinline__ float cell_value(const uint4& hdr, const uint4& q0, const uint4& q1, int g, const CellX& x) {
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
    const float dot_lo = x.st_lo * (float)(ia_lo * 256 + ib_lo);
    const float dot_hi = x.st_hi * (float)((ia_hi * 256 + ib_hi) >> 4);
    return d * ((float)(sc2 & 0xff) * dot_lo + (float)(sc2 >> 8) * dot_hi) -
           dmin * ((float)(m2 & 0xff) * x.su_lo + (float)(m2 >> 8) * x.su_hi);
}

// One cell (registers) against the activation planes read from shared memory: the same value as
// cell_value(), for code that cannot afford to keep a CellX in registers.
__device__ __forceinline__ float cell_value_smem(const uint4& hdr, const uint4& q0, const uint4& q1, int g,
                                                 const uint32_t* xa, const uint32_t* xb, const float* blk, int nblk,
                                                 int blk_lo, int G, int c) {
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    int ia_lo = 0, ib_lo = 0, ia_hi = 0, ib_hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t lo = qw[j] & 0x0F0F0F0Fu, hi = qw[j] & 0xF0F0F0F0u;
        ia_lo = dp4a_us(lo, xa[j * G + c], ia_lo);
        ib_lo = dp4a_uu(lo, xb[j * G + c], ib_lo);
        ia_hi = dp4a_us(hi, xa[(8 + j) * G + c], ia_hi);
        ib_hi = dp4a_uu(hi, xb[(8 + j) * G + c], ib_hi);
    }
    const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
    uint32_t sc2, m2;
    q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
    const float dot_lo = blk[blk_lo] * (float)(ia_lo * 256 + ib_lo);
    const float dot_hi = blk[blk_lo + 1] * (float)((ia_hi * 256 + ib_hi) >> 4);
    return d * ((float)(sc2 & 0xff) * dot_lo + (float)(sc2 >> 8) * dot_hi) -
           dmin * ((float)(m2 & 0xff) * blk[nblk + blk_lo] + (float)(m2 >> 8) * blk[nblk + blk_lo + 1]);
}

// out += act * (one 64-weight cell of a down row), into the thread's 64 accumulators.  q enters as
// f = 1 + q/128 built by a byte permute: out += A*f, corrected by -A at the end (corr_*).
__device__ __forceinline__ void axpy_cell(const uint8_t* cell, int g, float act, float (&acc_lo)[32], float (&acc_hi)[32],
                                          float& corr_lo, float& corr_hi) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
    const uint4 d0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
    const uint4 d1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
    const uint32_t qw[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
    uint32_t sc2, m2;
    q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
    const float ad = act * d, am = act * dmin;
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

// Gather of one chunk of rows (global row numbers and gate scores in shared memory).
// Team t takes items t, t+P, ...; a thread owns one 64-weight cell of every row.
//   1. the chunk's up rows move into the idle ring (row i at i * row_bytes): one TMA bulk copy per row,
//      issued by thread i, all completing on one mbarrier;
//   2. up dots out of shared memory against the activation planes (held in registers), reduced per warp
//      into psum[i][warp of the team]; as soon as a team is done with a row's slot, one of its threads
//      starts the copy of the same feature's down row into it (a second mbarrier collects those);
//   3. thread i turns row i's partials into act_i = silu(gate_i) * up_i;
//   4. once the down rows have landed: axpy of each of the team's rows into the thread's 64 accumulators;
//   5. every thread leaves its accumulators in the ring (one region of G * 65 floats per team,
//      64-float chunks at a stride of 65) for the merge.
struct GatherArgs {
    const uint8_t* up;
    const uint8_t* down;
    const int* rows;
    const float* scores;
    uint8_t* ring;
    float* psum;       // [FW_MAX_GROWS][Wt]
    float* act;        // [FW_MAX_GROWS]
    uint64_t* bar;     // mbarrier of the down-row copies
    uint64_t* ubar;    // mbarrier of the up-row copies
    const uint32_t* xa_s;
    const uint32_t* xb_s;
    const float* blk_s;
    int nsb, G, TS, P, Wt, row_bytes;
};

__device__ __forceinline__ void gather_stage(const GatherArgs& ga, int base, int nn, uint32_t bar_parity, bool& failed) {
    const int tid = threadIdx.x, lane = tid & 31;
    const int team = tid / ga.TS, c = tid % ga.TS, wt = c >> 5;
    const bool in_team = team < ga.P;
    const bool active = in_team && c < ga.G;
    const int s = c >> 2, g = c & 3, nblk = ga.nsb * 8, P = ga.P;
    // 1. the chunk's up rows -> ring (row i at i * row_bytes), one bulk copy per row, issued by thread i
    if (tid == 0) {
        mbar_expect_tx(ga.ubar, (uint32_t)nn * (uint32_t)ga.row_bytes);
        mbar_expect_tx(ga.bar, (uint32_t)nn * (uint32_t)ga.row_bytes);  // the down rows follow slot by slot
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // the expectations are armed before any copy can complete
#pragma unroll 1
    for (int i = tid; i < nn; i += FW_CONSUMERS)
        tma_bulk_g2s(ga.ring + (size_t)i * ga.row_bytes, ga.up + (size_t)(uint32_t)ga.rows[base + i] * ga.row_bytes,
                     (uint32_t)ga.row_bytes, ga.ubar);
    // 2. up dots out of shared memory; a team takes rows team, team + P, ...; as soon as all of the team's
    //    threads have read a row, its slot takes the same feature's down row
    if (in_team) {
        CellX x;
        {
            const int cl = active ? c : 0;  // unconditional: see the scan
            load_cellx(x, ga.xa_s, ga.xb_s, ga.blk_s, nblk, (cl >> 2) * 8 + 2 * (cl & 3), ga.G, cl);
        }
        if (!failed && !mbar_wait(ga.ubar, bar_parity)) failed = true;
#pragma unroll 1
        for (int i = team; i < nn; i += P) {
            float val = 0.0f;
            if (active) {
                const uint8_t* cell = ga.ring + (size_t)i * ga.row_bytes + s * 144;
                const uint4 hd = *reinterpret_cast<const uint4*>(cell);
                const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
                const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
                val = cell_value(hd, q0, q1, g, x);
            }
            for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
            if (lane == 0) ga.psum[i * ga.Wt + wt] = val;
            bar_sync(1 + team, ga.TS);  // every thread of the team is done with the up row
            if (c == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // plain reads before the TMA write
                tma_bulk_g2s(ga.ring + (size_t)i * ga.row_bytes,
                             ga.down + (size_t)(uint32_t)ga.rows[base + i] * ga.row_bytes, (uint32_t)ga.row_bytes, ga.bar);
            }
        }
    } else if (!failed && !mbar_wait(ga.ubar, bar_parity)) {
        failed = true;  // (threads outside the teams pass the phase too)
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    // 3. activations
#pragma unroll 1
    for (int i = tid; i < nn; i += FW_CONSUMERS) {
        float upv = 0.0f;
#pragma unroll 1
        for (int w = 0; w < ga.Wt; ++w) upv += ga.psum[i * ga.Wt + w];
        const float gs = ga.scores[base + i];
        const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
        const float act = (gs * sig) * upv;
        ga.act[i] = fabsf(act) > FW_NOISE_FLOOR ? act : 0.0f;
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    if (!failed && !mbar_wait(ga.bar, bar_parity)) failed = true;
    // 4. down rows
    float acc_lo[32], acc_hi[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) acc_lo[j] = acc_hi[j] = 0.0f;
    float corr_lo = 0.0f, corr_hi = 0.0f;
    if (active) {
#pragma unroll 1
        for (int i = team; i < nn; i += P) {
            const float act = ga.act[i];
            if (act == 0.0f) continue;
            axpy_cell(ga.ring + (size_t)i * ga.row_bytes + s * 144, g, act, acc_lo, acc_hi, corr_lo, corr_hi);
        }
    }
    // 5. every team has finished reading the staged rows: the ring now takes the accumulators
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    if (active) {
        float* o_lo = reinterpret_cast<float*>(ga.ring) + team * (ga.G * 65) + c * 65;
        float* o_hi = o_lo + 32;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            o_lo[j] = acc_lo[j] - corr_lo;
            o_hi[j] = acc_hi[j] - corr_hi;
        }
    }
}

// ---- kernel state shared by the phases ---------------------------------------------------------
// The geometry, the launch arguments and a few derived counts sit in shared memory so that every
// phase can be its own out-of-line function: each gets a register allocation of its own (the scan
// loop and the gather both want most of the file) and nothing stays live across phases but what
// these structs hold.
struct Ctx {
    FusedGeom gm;
    FusedArgs a;
    int n_tiles, first_tile, my_count, n_slots, n_ahead, stamp_layer;
};

// control words (ints), in the last 64 bytes of the barrier page
enum { SC_N_IN = 0, SC_N_BAND = 1, SC_N_G2 = 2, SC_BAND_BASE = 3, SC_BSTAR = 4, SC_HIT_BASE = 5, SC_FAILED = 6,
       SC_FOUND = 7, SC_GATHER_USES = 9, SC_N_KEEP = 10, SC_N_EARLY = 11, SC_BAND_USES = 12 };

struct Smem {
    uint8_t* base;
    __device__ __forceinline__ Ctx& cx() const { return *reinterpret_cast<Ctx*>(base + 192); }
    __device__ __forceinline__ uint64_t* full() const { return reinterpret_cast<uint64_t*>(base); }
    __device__ __forceinline__ uint64_t* gbar() const { return reinterpret_cast<uint64_t*>(base) + 2 * FW_MAX_STAGES; }
    // mbarriers of a layer's first gather chunk, each completing exactly once per layer (phase parity = layer & 1):
    // up rows staged before the pick, their down rows, the up rows of the rows added by the pick, their down rows;
    // ebar(4): the band rows staged for the exact re-score (its phase parity is counted in SC_BAND_USES)
    __device__ __forceinline__ uint64_t* ebar(int i) const { return gbar() + 2 + i; }
    __device__ __forceinline__ int* ctl() const { return reinterpret_cast<int*>(base + 1024 - 64); }
    // warps that have finished reading each ring stage's current tile
    __device__ __forceinline__ int* released() const { return reinterpret_cast<int*>(base + 1024 - 128); }
    __device__ __forceinline__ float* xs() const { return reinterpret_cast<float*>(base + cx().gm.off_xs); }
    __device__ __forceinline__ uint32_t* xa() const { return reinterpret_cast<uint32_t*>(base + cx().gm.off_xa); }
    __device__ __forceinline__ uint32_t* xb() const { return reinterpret_cast<uint32_t*>(base + cx().gm.off_xb); }
    __device__ __forceinline__ float* blk() const { return reinterpret_cast<float*>(base + cx().gm.off_blk); }
    __device__ __forceinline__ float* red() const { return reinterpret_cast<float*>(base + cx().gm.off_red); }
    __device__ __forceinline__ float* wpart() const { return reinterpret_cast<float*>(base + cx().gm.off_wpart); }
    __device__ __forceinline__ float* psum() const { return reinterpret_cast<float*>(base + cx().gm.off_psum); }
    __device__ __forceinline__ float* scores() const { return reinterpret_cast<float*>(base + cx().gm.off_scores); }
    __device__ __forceinline__ int* in_list() const { return reinterpret_cast<int*>(base + cx().gm.off_lists); }
    __device__ __forceinline__ int* band_list() const { return in_list() + cx().gm.max_slots; }
    __device__ __forceinline__ float* band_ex() const { return reinterpret_cast<float*>(band_list() + cx().gm.max_slots); }
    // [2 * max_slots] global rows of the gather and their gate scores
    __device__ __forceinline__ int* g_rows() const { return reinterpret_cast<int*>(band_ex() + cx().gm.max_slots); }
    __device__ __forceinline__ float* g_scores() const { return reinterpret_cast<float*>(g_rows() + 2 * cx().gm.max_slots); }
    __device__ __forceinline__ uint8_t* ring() const { return base + cx().gm.off_ring; }
};
static_assert(FW_NWARPS <= 32, "per-warp scratch arrays hold 32 warps");
static_assert(192 + sizeof(Ctx) <= 1024 - 128, "context does not fit the barrier page");

#define FW_STAMP(i)                                                                                    \
    do {                                                                                               \
        if (a.phase_ns && l == cx.stamp_layer && (int)blockIdx.x == a.stamp_cta && threadIdx.x == 0) a.phase_ns[i] = gtimer(); \
    } while (0)

__device__ __forceinline__ FusedLayer layer_of(const FusedArgs& a, int l) { return a.layers ? a.layers[l] : a.single; }
// epoch of the exchange lines of layer l of this launch
__device__ __forceinline__ uint32_t x_epoch(const FusedArgs& a, int l) { return a.px.xepoch0 + (uint32_t)l + 1u; }
__device__ __forceinline__ int row_of_slot(const Ctx& cx, int m) {
    return (cx.first_tile + (m / cx.gm.R) * (int)gridDim.x) * cx.gm.R + (m % cx.gm.R);
}

// One thread issues the TMA copy of a gate tile: tile `it` (counted over all layers) goes to stage
// it % S.  The caller knows that every warp has finished with that stage's previous tile.
__device__ __forceinline__ void issue_tile(const Smem& sm, const FusedLayer& lyr, int k, uint32_t it) {
    const Ctx& cx = sm.cx();
    const int S = cx.gm.S, stg = it % S;
    const int row0 = (cx.first_tile + k * (int)gridDim.x) * cx.gm.R;
    const uint32_t bytes = (uint32_t)min(cx.gm.R, cx.a.n_rows - row0) * (uint32_t)cx.gm.row_bytes;
    mbar_expect_tx(&sm.full()[stg], bytes);
    tma_bulk_g2s(sm.ring() + (size_t)stg * cx.gm.tile_bytes, lyr.gate + (size_t)row0 * cx.gm.row_bytes, bytes,
                 &sm.full()[stg]);
}
// L2 prefetch of this CTA's tiles [from, upto) of a layer's gate rows (one thread).
__device__ __forceinline__ void prefetch_tiles(const Smem& sm, const FusedLayer& lyr, int from, int upto) {
    const Ctx& cx = sm.cx();
    for (int t = from; t < min(upto, cx.my_count); ++t) {
        const int row0 = (cx.first_tile + t * (int)gridDim.x) * cx.gm.R;
        const uint32_t bytes = (uint32_t)min(cx.gm.R, cx.a.n_rows - row0) * (uint32_t)cx.gm.row_bytes;
        l2_prefetch_bulk(lyr.gate + (size_t)row0 * cx.gm.row_bytes, bytes);
    }
}
// Tiles [0, S) of a layer go straight into the ring; how many more are in L2 when its scan starts:
// the tail of the previous layer prefetches them (the next layer's gate rows do not depend on this
// layer's result, and the selection, gather and reduction phases leave HBM idle); inside the scan the
// prefetch then stays pf_dist tiles ahead of the ring.
__device__ __forceinline__ int tiles_covered_at_scan_start(const Ctx& cx) {
    return max(cx.gm.S + max(cx.a.pf_dist, 0), cx.a.pf_tiles);
}
__device__ __forceinline__ void prefetch_next_gate(const Smem& sm, int l) {
    const Ctx& cx = sm.cx();
    if (threadIdx.x == 0 && l + 1 < cx.a.n_layers && (cx.a.pf_tiles > 0 || cx.a.pf_dist > 0))
        prefetch_tiles(sm, cx.a.layers[l + 1], cx.gm.S, tiles_covered_at_scan_start(cx));
}

// ---- 0. prepare the activation ----------------------------------------------------------------
__device__ __noinline__ void phase_prepare(int l, const float* h_cur) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom& gm = cx.gm;
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hidden = gm.nsb * 256, nblk = gm.nsb * 8;
    float* xs = sm.xs();
    uint32_t* xa_s = sm.xa();
    uint32_t* xb_s = sm.xb();
    float* blk_s = sm.blk();
    // pass 1: copy the residual into shared memory, sum of squares in f64
    double sq = 0.0;
    const float4* src = reinterpret_cast<const float4*>(h_cur);
    for (int i = tid; i < hidden / 4; i += FW_CONSUMERS) {
        const float4 t = __ldcg(src + i);
        *reinterpret_cast<float4*>(xs + ((4 * i) >> 6) * 68 + ((4 * i) & 63)) = t;
        sq += (double)t.x * (double)t.x + (double)t.y * (double)t.y;
        sq += (double)t.z * (double)t.z + (double)t.w * (double)t.w;
    }
    float rms = 1.0f;
    if (a.flags & LQ_WALK_RMSNORM) {
        double* dred = reinterpret_cast<double*>(sm.red());
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) dred[warp] = sq;
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        double t = 0.0;
#pragma unroll 1
        for (int w = 0; w < FW_NWARPS; ++w) t += dred[w];
        rms = (float)sqrt(t / (double)hidden + 1e-6);
    } else {
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    }
    // pass 2: four threads per 32-element block, 8 elements each.  With x_hat = step * q the
    // fixed-point copy, e = x - x_hat and a block's weights q_w in [0, 15]:
    //   |sum q_w e| = |sum (q_w - 7.5) e + 7.5 sum e| <= 7.5 (sum |e| + |sum e|),
    // so the block's contribution to |fast - reference| of a row is at most
    //   |d| sc (15 c1 sum|x| + 7.5 (sum|e| + |sum e|)) + |dmin| m c1 sum|x|  =: |d| sc bu + |dmin| m bv
    // (c1: rounding-count constant of the two evaluation orders).  e is measured, not assumed:
    // fmaf(-step, q, x) is exact up to one rounding of the result, covered by the margins below.
    bool bad = false;
    for (int u = tid; u < hidden / 8; u += FW_CONSUMERS) {
        const int blk = u >> 2, part = u & 3;
        const int cc = blk >> 1, hb = blk & 1;
        float* xdst = xs + cc * 68 + hb * 32 + part * 8;
        const float4 t0 = *reinterpret_cast<const float4*>(xdst);
        const float4 t1 = *reinterpret_cast<const float4*>(xdst + 4);
        float v[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
        float amax = 0.0f, sum = 0.0f, asum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (a.flags & LQ_WALK_RMSNORM) v[j] = __fdiv_rn(v[j], rms);
            bad |= !isfinite(v[j]);
            amax = fmaxf(amax, fabsf(v[j]));
            sum += v[j];
            asum += fabsf(v[j]);
        }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            asum += __shfl_xor_sync(0xffffffffu, asum, o);
        }
        const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
        const float step = amax / 32767.0f;
        float eabs = 0.0f, esum = 0.0f;
        uint32_t wa[2] = {0u, 0u}, wb[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int q = __float2int_rn(v[j] * inv);
            q = max(-32767, min(32767, q));
            const float e = fmaf(-step, (float)q, v[j]);
            eabs += fabsf(e);
            esum += e;
            wa[j >> 2] |= (uint32_t)((q >> 8) & 0xff) << (8 * (j & 3));
            wb[j >> 2] |= (uint32_t)(q & 0xff) << (8 * (j & 3));
        }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            eabs += __shfl_xor_sync(0xffffffffu, eabs, o);
            esum += __shfl_xor_sync(0xffffffffu, esum, o);
        }
        if (part == 0) {
            const float qe = 7.5f * (1.001f * (eabs + fabsf(esum)) + 4.8e-7f * asum);
            blk_s[blk] = step;
            blk_s[nblk + blk] = sum;
            blk_s[2 * nblk + blk] = 1.001f * (15.0f * a.c1 * asum + qe);
            blk_s[3 * nblk + blk] = 1.001f * a.c1 * asum;
        }
        xa_s[(hb * 8 + part * 2) * gm.G + cc] = wa[0];
        xa_s[(hb * 8 + part * 2 + 1) * gm.G + cc] = wa[1];
        xb_s[(hb * 8 + part * 2) * gm.G + cc] = wb[0];
        xb_s[(hb * 8 + part * 2 + 1) * gm.G + cc] = wb[1];
        *reinterpret_cast<float4*>(xdst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(xdst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (bad) set_err(a.err, DEV_ERR_NAN_SCORE);
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
}

// ---- 1. scan this CTA's gate tiles ---------------------------------------------------------------
__device__ __noinline__ void phase_scan(int l) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom gm = cx.gm;  // by value: the loop below must not re-read these after every barrier
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x, lane = tid & 31;
    const int team = tid / gm.TS, c = tid % gm.TS, wt = c >> 5;
    const int P = gm.P, R = gm.R, nblk = gm.nsb * 8;
    const bool in_team = team < P;
    const bool active = in_team && c < gm.G;
    const int s = c >> 2, g = c & 3;
    const int my_count = cx.my_count;
    const uint32_t scan_it = (uint32_t)l * (uint32_t)my_count;
    const FusedLayer ly = layer_of(a, l);
    uint32_t* hist = a.hist + (size_t)(l & 1) * FW_HIST_WORDS +
                     (size_t)((blockIdx.x + (tid >> 5)) % FW_HIST_COPIES) * LQ_HIST_BINS;
    float* my_scores = sm.scores();
    float* wpart = sm.wpart();
    uint64_t* full = sm.full();
    const uint8_t* ring = sm.ring();
    bool failed = false;

    CellX x;
    float bmax = 0.0f;
    uint32_t kmax = 0;
    {
        // loaded unconditionally (idle lanes take cell 0): a conditionally initialised struct ends up in local memory
        const int cl = active ? c : 0;
        load_cellx(x, sm.xa(), sm.xb(), sm.blk(), nblk, (cl >> 2) * 8 + 2 * (cl & 3), gm.G, cl);
    }
    int* released = sm.released();
    const int covered = tiles_covered_at_scan_start(cx);
    if (l == 0 && tid == 0 && a.pf_dist > 0) prefetch_tiles(sm, ly, gm.S, covered);  // later layers: done in the previous tail
#pragma unroll 1
    for (int k = 0; k < my_count; ++k) {
        const uint32_t it = scan_it + k;
        const int stg = it % gm.S;
        if (!failed && !mbar_wait(&full[stg], (it / gm.S) & 1)) failed = true;
        const int row0 = (cx.first_tile + k * (int)gridDim.x) * R;
        const int rows_here = min(R, a.n_rows - row0);
        const uint8_t* tb = ring + (size_t)stg * gm.tile_bytes + (active ? s : 0) * 144;  // idle lanes stay inside the row
        float* wp = wpart + (size_t)k * R * gm.Wt;  // [row of the tile][warp of the team]
        if (in_team) {
            // rows past the end of a ragged last tile are computed on whatever the stage holds and discarded
#pragma unroll 1
            for (int j = 0; j < gm.Rt; ++j) {
                const int r0 = team + j * P;
                const bool ok0 = active && r0 < rows_here;
                float b0;
                float v0 = cell_dot(tb + (size_t)(ok0 ? r0 : 0) * gm.row_bytes, g, x, b0);
                v0 = ok0 ? v0 : 0.0f;
                bmax = fmaxf(bmax, ok0 ? b0 : 0.0f);
                for (int o = 16; o > 0; o >>= 1) v0 += __shfl_xor_sync(0xffffffffu, v0, o);
                if (lane == 0) wp[r0 * gm.Wt + wt] = v0;
            }
        }
        // This warp has read the tile: the reduction above consumed every lane's loads.  The last warp to
        // say so refills the stage with the tile S further on (nobody waits for a stage to drain) and keeps
        // the L2 prefetch running ahead of the ring.
        __syncwarp();
        if (lane == 0 && atomicAdd(&released[stg], 1) == FW_NWARPS - 1) {
            released[stg] = 0;
            if (k + gm.S < my_count) issue_tile(sm, ly, k + gm.S, it + gm.S);
            const int t = k + gm.S + a.pf_dist;
            if (a.pf_dist > 0 && t >= covered) prefetch_tiles(sm, ly, t, t + 1);
        }
    }
    // every warp's partials are in place: scores of this CTA's rows, histogram, largest occupied bin
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
#pragma unroll 1
    for (int m = tid; m < cx.n_slots; m += FW_CONSUMERS) {
        float sc = 0.0f;
#pragma unroll 1
        for (int w = 0; w < gm.Wt; ++w) sc += wpart[m * gm.Wt + w];
        my_scores[m] = sc;
        if (row_of_slot(cx, m) < a.n_rows) {
            if (sc != sc) set_err(a.err, DEV_ERR_NAN_SCORE);
            const uint32_t bin = __float_as_uint(fabsf(sc)) >> LQ_HIST_SHIFT;
            atomicAdd(&hist[bin], 1u);
            kmax = max(kmax, bin);
        }
    }
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    if (!a.pf_late) prefetch_next_gate(sm, l);
    // bound: sum over the team's cells of each thread's largest cell bound; one atomic per CTA for the bound and
    // one for the largest occupied bin (they all go to two words that every CTA of the grid is updating)
    {
        for (int o = 16; o > 0; o >>= 1) bmax += __shfl_xor_sync(0xffffffffu, bmax, o);
        float* wb = sm.red();                                       // [warp] bound partials
        uint32_t* wk = reinterpret_cast<uint32_t*>(sm.red()) + 32;  // [warp] largest bins
        if (lane == 0) {
            wb[tid >> 5] = in_team ? bmax : 0.0f;
            wk[tid >> 5] = kmax;
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        if (tid < 32) {
            // lane t: the bound of team t (its warps' partials in warp order) and the largest bin of warp t
            float best = 0.0f;
            if (lane < P) {
#pragma unroll 1
                for (int w = 0; w < gm.Wt; ++w) best += wb[lane * gm.Wt + w];
            }
            uint32_t kb = lane < FW_NWARPS ? wk[lane] : 0u;
            for (int o = 16; o > 0; o >>= 1) {
                best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
                kb = max(kb, __shfl_xor_sync(0xffffffffu, kb, o));
            }
            best *= 1.0001f;  // the sums above round to nearest
            if (lane == 0) {
                if (best > 0.0f) atomicMax(&a.ctrs[CTR_BOUND0 + (l & 1)], __float_as_uint(best));
                if (kb > 0u) atomicMax(&a.ctrs[CTR_MAXBIN0 + (l & 1)], kb);
            }
        }
    }
    if (tid == 0) {
        sm.ctl()[SC_BSTAR] = 0;
        sm.ctl()[SC_FOUND] = 0;
    }
    if (failed) sm.ctl()[SC_FAILED] = 1;
}

// ---- 1b. sharded walk: this rank's histogram, bound and highest bin go to every rank -------------
// After a barrier over this GPU's CTAs the local histogram is complete; every CTA sends a slice of it,
// as lines, into slot `rank` of every rank's area (all bins, so a reader never meets a stale line).
__device__ __noinline__ void phase_xhist(int l) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const FusedArgs& a = sm.cx().a;
    const FusedPeers& px = a.px;
    const int tid = threadIdx.x, par = l & 1;
    const uint32_t ep = x_epoch(a, l);
    const uint2* hist2 = reinterpret_cast<const uint2*>(a.hist + (size_t)par * FW_HIST_WORDS);
    constexpr int N2 = LQ_HIST_BINS / 2;
    const int per = (N2 + gridDim.x - 1) / gridDim.x, c0 = blockIdx.x * per, n = max(0, min(per, N2 - c0));
#pragma unroll 1
    for (int i = tid; i < n * px.world; i += FW_CONSUMERS) {
        const int p = i / n, j = i - p * n;
        uint2 v = make_uint2(0u, 0u);
#pragma unroll
        for (int hc = 0; hc < FW_HIST_COPIES; ++hc) {
            const uint2 t = __ldcg(hist2 + (size_t)hc * N2 + c0 + j);
            v.x += t.x;
            v.y += t.y;
        }
        line_store(reinterpret_cast<uint4*>(px.area[p] + px.off_hist) + (size_t)px.rank * N2 + c0 + j, v.x, v.y, ep);
    }
    if (blockIdx.x == 0 && tid < px.world)
        line_store(reinterpret_cast<uint4*>(px.area[tid] + px.off_meta) + px.rank, __ldcg(&a.ctrs[CTR_BOUND0 + par]),
                   __ldcg(&a.ctrs[CTR_MAXBIN0 + par]), ep);
}

// ---- 2. threshold bucket, classification, exact re-score and publication of the band ------------
template <bool X>
__device__ __noinline__ void phase_select(int l) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom& gm = cx.gm;
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int par = l & 1;
    const uint32_t* hist = a.hist + (size_t)par * FW_HIST_WORDS;
    int* s_ctl = sm.ctl();
    float* red = sm.red();
    float* my_scores = sm.scores();
    int* in_list = sm.in_list();
    int* band_list = sm.band_list();
    float* band_ex = sm.band_ex();
    int* g2_rows = sm.g_rows();
    float* g2_scores = sm.g_scores();
    const int n_slots = cx.n_slots;

    float hi, lo;
    {
        // Read the histogram from the highest occupied bin downwards, 1024 bins per round
        // (256 threads x 4 bins, thread 0 the highest), until the cumulative count reaches K.
        constexpr int HT = 256;
        uint32_t bbits, maxbin;
        if (X) {
            // positive floats order like their bits: the largest bound of any rank, the highest bin of any rank
            const uint4* meta = reinterpret_cast<const uint4*>(a.px.area[a.px.rank] + a.px.off_meta);
            uint32_t wb[FW_MAX_WORLD], wm[FW_MAX_WORLD];
            lines_wait_ranks(meta, 1, a.px.world, x_epoch(a, l), wb, wm, a.err);
            bbits = 0u;
            maxbin = 0u;
#pragma unroll
            for (int r = 0; r < FW_MAX_WORLD; ++r) {  // (absent ranks read as zero)
                bbits = max(bbits, wb[r]);
                maxbin = max(maxbin, wm[r]);
            }
        } else {
            bbits = __ldcg(&a.ctrs[CTR_BOUND0 + par]);
            maxbin = __ldcg(&a.ctrs[CTR_MAXBIN0 + par]);
        }
        maxbin = min(maxbin, (uint32_t)LQ_HIST_BINS - 1u);
        const uint32_t K = (uint32_t)a.top_k;
        uint32_t* wsum = reinterpret_cast<uint32_t*>(red);
        uint32_t above_total = 0;
#pragma unroll 1
        for (int base_end = (int)(maxbin / 4u + 1u) * 4; base_end > 0; base_end -= 4 * HT) {
            const int b0 = base_end - 4 * (tid + 1);
            uint4 t4 = make_uint4(0u, 0u, 0u, 0u);
            if (tid < HT && b0 >= 0) {
                if (X) {
                    // every rank's four bins: two lines each, taken as they arrive
                    const uint4* hl = reinterpret_cast<const uint4*>(a.px.area[a.px.rank] + a.px.off_hist);
                    const uint32_t ep = x_epoch(a, l);
                    uint32_t w0[FW_MAX_WORLD], w1[FW_MAX_WORLD], w2[FW_MAX_WORLD], w3[FW_MAX_WORLD];
                    lines_wait_ranks(hl + b0 / 2, LQ_HIST_BINS / 2, a.px.world, ep, w0, w1, a.err);
                    lines_wait_ranks(hl + b0 / 2 + 1, LQ_HIST_BINS / 2, a.px.world, ep, w2, w3, a.err);
#pragma unroll
                    for (int r = 0; r < FW_MAX_WORLD; ++r) {
                        t4.x += w0[r]; t4.y += w1[r]; t4.z += w2[r]; t4.w += w3[r];
                    }
                } else {
#pragma unroll
                    for (int hc = 0; hc < FW_HIST_COPIES; ++hc) {
                        const uint4 t = __ldcg(reinterpret_cast<const uint4*>(hist + (size_t)hc * LQ_HIST_BINS + b0));
                        t4.x += t.x; t4.y += t.y; t4.z += t.z; t4.w += t.w;
                    }
                }
            }
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
                s_ctl[SC_BSTAR] = b0 + b;
                s_ctl[SC_FOUND] = 1;
            }
            above_total += chunk_total;
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
            if (s_ctl[SC_FOUND]) break;
        }
        const uint32_t bstar = (uint32_t)s_ctl[SC_BSTAR];
        const float B = __uint_as_float(bbits);
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
    // A CTA gathers at most n_fair rows of its own: its band rows (all of them may win) and certainly-in
    // rows up to the fair share + 1.  The rest of its certainly-in rows goes to a pool that all CTAs share
    // out after barrier B (filling the least loaded CTAs first), so one heavy CTA does not hold everybody up
    // and a CTA's list fits the ring in one piece.
    int n_fair;
    {
        int* wcnt = reinterpret_cast<int*>(red) + 64;  // [2][32]
        const int chunk = (n_slots + FW_NWARPS - 1) / FW_NWARPS;
        const int chunk32 = (chunk + 31) / 32 * 32;
        const int beg = warp * chunk32, end = min(n_slots, beg + chunk32);
        auto cls = [&](int m) -> int {
            if (row_of_slot(cx, m) >= a.n_rows) return 0;
            const float v = fabsf(my_scores[m]);
            return v > hi ? 1 : (v >= lo ? 2 : 0);
        };
        int ca = 0, cb = 0;
#pragma unroll 1
        for (int m0 = beg; m0 < end; m0 += 32) {
            const int m = m0 + lane;
            const int cc = m < end ? cls(m) : 0;
            ca += __popc(__ballot_sync(0xffffffffu, cc == 1));
            cb += __popc(__ballot_sync(0xffffffffu, cc == 2));
        }
        if (lane == 0) {
            wcnt[warp] = ca;
            wcnt[32 + warp] = cb;
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        int oa = 0, ob = 0, ta = 0, tb2 = 0;
#pragma unroll 1
        for (int w = 0; w < FW_NWARPS; ++w) {
            if (w < warp) {
                oa += wcnt[w];
                ob += wcnt[32 + w];
            }
            ta += wcnt[w];
            tb2 += wcnt[32 + w];
        }
        const int n_ctas = (int)gridDim.x * (X ? a.px.world : 1);
        n_fair = max(0, (a.top_k + n_ctas - 1) / n_ctas + 1 - tb2);
#pragma unroll 1
        for (int m0 = beg; m0 < end; m0 += 32) {
            const int m = m0 + lane;
            const int cc = m < end ? cls(m) : 0;
            const uint32_t ba = __ballot_sync(0xffffffffu, cc == 1), bb = __ballot_sync(0xffffffffu, cc == 2);
            const uint32_t lt = (1u << lane) - 1u;
            if (cc == 1) {
                const int pos = oa + __popc(ba & lt);
                in_list[pos] = m;
                if (pos < n_fair) {  // this CTA's own gather: global row and gate score
                    g2_rows[pos] = row_of_slot(cx, m);
                    g2_scores[pos] = my_scores[m];
                }
            }
            if (cc == 2) band_list[ob + __popc(bb & lt)] = m;
            oa += __popc(ba);
            ob += __popc(bb);
        }
        if (tid == 0) {
            s_ctl[SC_N_IN] = ta;     // certainly-in rows of this CTA
            s_ctl[SC_N_BAND] = tb2;  // band rows of this CTA
            s_ctl[SC_N_KEEP] = min(ta, n_fair);
            // The rows this CTA will gather whatever the pick decides (its own certainly-in rows up to the fair
            // share) do not wait for the pick: their up rows start moving into the idle ring now, the up dots
            // run while the grid barrier collects, and their down rows land while the pick runs.
            const int n_early = min(min(ta, n_fair), gm.E);
            s_ctl[SC_N_EARLY] = n_early;
            mbar_expect_tx(sm.ebar(0), (uint32_t)n_early * (uint32_t)gm.row_bytes);
            mbar_expect_tx(sm.ebar(1), (uint32_t)n_early * (uint32_t)gm.row_bytes);
        }
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    FW_STAMP(4);
    const int n_in_mine = s_ctl[SC_N_IN], n_band_mine = s_ctl[SC_N_BAND];
    // The band rows of the gate matrix are staged for the exact re-score in the slots behind the early rows,
    // and asked for FIRST: the re-score is on the critical path, the early rows have until the pick is over.
    const int n_early_sel = s_ctl[SC_N_EARLY];
    const int band_cap = max(1, gm.E - n_early_sel);  // band rows staged per round
    uint32_t band_uses = (uint32_t)s_ctl[SC_BAND_USES];
    {
        const FusedLayer ly = layer_of(a, l);
        const int nb0 = min(n_band_mine, band_cap);
        if (tid == 0 && nb0 > 0) mbar_expect_tx(sm.ebar(4), (uint32_t)nb0 * (uint32_t)gm.row_bytes);
        // (armed by thread 0, in program order, before it issues the first copy; copies of other warps may only
        // complete later than that: see the barrier below)
        if (nb0 > 32) bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        else __syncwarp();
#pragma unroll 1
        for (int i = tid; i < nb0; i += FW_CONSUMERS)
            tma_bulk_g2s(sm.ring() + (size_t)(n_early_sel + i) * gm.row_bytes,
                         ly.gate + (size_t)row_of_slot(cx, band_list[i]) * gm.row_bytes, (uint32_t)gm.row_bytes, sm.ebar(4));
#pragma unroll 1
        for (int i = tid; i < n_early_sel; i += FW_CONSUMERS)
            tma_bulk_g2s(sm.ring() + (size_t)i * gm.row_bytes, ly.up + (size_t)(uint32_t)g2_rows[i] * gm.row_bytes,
                         (uint32_t)gm.row_bytes, sm.ebar(0));
    }
    // ---- exact re-score of own band rows (one warp per row), publish them ----------
    // (this CTA's place in the band arrays is asked for first: the answer travels while the rows are re-scored)
    int band_base_t0 = 0;
    if (tid == 0) {
        atomicAdd(&a.ctrs[CTR_IN], (uint32_t)n_in_mine);
        band_base_t0 = n_band_mine ? (int)atomicAdd(&a.ctrs[CTR_BAND], (uint32_t)n_band_mine) : 0;
    }
    {
        const FusedLayer ly = layer_of(a, l);
        const float* xs = sm.xs();
        const uint8_t* stage = sm.ring() + (size_t)n_early_sel * gm.row_bytes;
#pragma unroll 1
        for (int r0 = 0; r0 < n_band_mine; r0 += band_cap) {
            const int nb = min(band_cap, n_band_mine - r0);
            if (r0 > 0) {
                // (a CTA with more band rows than free slots: further rounds through the same slots)
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                if (tid == 0) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_expect_tx(sm.ebar(4), (uint32_t)nb * (uint32_t)gm.row_bytes);
#pragma unroll 1
                    for (int i = 0; i < nb; ++i)
                        tma_bulk_g2s(sm.ring() + (size_t)(n_early_sel + i) * gm.row_bytes,
                                     ly.gate + (size_t)row_of_slot(cx, band_list[r0 + i]) * gm.row_bytes,
                                     (uint32_t)gm.row_bytes, sm.ebar(4));
                }
            }
            if (!mbar_wait(sm.ebar(4), band_uses & 1u)) s_ctl[SC_FAILED] = 1;
            band_uses += 1;
            // A CTA has a few band rows and sixteen warps: up to four warps share a row (each takes every wpr-th pass
            // of eight super-blocks; the partials of a row are summed in super-block order afterwards).
            const int passes = (gm.nsb + 7) / 8;
            const int wpr = (4 * nb <= FW_NWARPS && passes >= 4) ? 4 : ((2 * nb <= FW_NWARPS && passes >= 2) ? 2 : 1);
            const int groups = FW_NWARPS / wpr;  // rows in flight
#pragma unroll 1
            for (int i0 = 0; i0 < nb; i0 += groups) {
                const int i = i0 + warp / wpr;
                if (i < nb)
                    exact_row_q4k_passes<true>(stage + (size_t)i * gm.row_bytes, xs, gm.nsb, red + 256 + (warp / wpr) * gm.nsb,
                                               lane, warp % wpr, wpr);
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);
                if (i < nb && warp % wpr == 0 && lane == 0) {
                    const float* part = red + 256 + (warp / wpr) * gm.nsb;
                    float total = 0.0f;
#pragma unroll 1
                    for (int sb = 0; sb < gm.nsb; ++sb) total = __fadd_rn(total, part[sb]);
                    band_ex[r0 + i] = total;
                }
                bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // the partial arrays are free for the next rows
            }
        }
    }
    if (tid == 0) {
        s_ctl[SC_BAND_BASE] = band_base_t0;
        s_ctl[SC_BAND_USES] = (int)band_uses;
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    {
        const int base = s_ctl[SC_BAND_BASE];
#pragma unroll 1
        for (int i = tid; i < n_band_mine; i += FW_CONSUMERS) {
            const float v = band_ex[i];
            if (v != v) set_err(a.err, DEV_ERR_NAN_SCORE);
            if (X) {
                // global row number; this rank's entries start at entry row_offset of every rank's arrays
                const uint32_t row = (uint32_t)(row_of_slot(cx, band_list[i]) + a.px.row_offset);
                const size_t at = (size_t)a.px.row_offset + base + i;
                for (int p = 0; p < a.px.world; ++p)
                    line_store(reinterpret_cast<uint4*>(a.px.area[p] + a.px.off_band) + at, row, __float_as_uint(v),
                               x_epoch(a, l));
            } else {
                a.band_row[base + i] = (uint32_t)row_of_slot(cx, band_list[i]);
                a.band_exact[base + i] = v;
            }
        }
    }
    const int n_keep = min(n_in_mine, n_fair), n_over = n_in_mine - n_keep;
    {
        uint32_t* pr = a.pool_row + (size_t)blockIdx.x * gm.max_slots;
        float* ps = a.pool_score + (size_t)blockIdx.x * gm.max_slots;
#pragma unroll 1
        for (int i = tid; i < n_over; i += FW_CONSUMERS) {
            const int m = in_list[n_keep + i];
            pr[i] = (uint32_t)row_of_slot(cx, m);
            ps[i] = my_scores[m];
        }
        if (tid == 0) {
            a.pool_cnt[blockIdx.x] = (uint32_t)n_over;
            a.pool_cnt[512 + blockIdx.x] = (uint32_t)(n_keep + n_band_mine);  // upper bound of this CTA's load so far
        }
    }
    if (X) {
        // The last CTA of this rank to get here sends the rank's counts to every rank (its own too): whoever
        // holds a rank's counts knows that all of that rank's CTAs have published their band and pool rows.
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        if (tid == 0) {
            __threadfence();
            const uint32_t done = atomicAdd(&a.ctrs[CTR_BDONE], 1u) + 1u;
            if (done == (uint32_t)(l + 1) * gridDim.x) {
                __threadfence();
                const uint32_t n_in = __ldcg(&a.ctrs[CTR_IN]), n_band = __ldcg(&a.ctrs[CTR_BAND]);
                for (int p = 0; p < a.px.world; ++p)
                    line_store(reinterpret_cast<uint4*>(a.px.area[p] + a.px.off_cnt) + a.px.rank, n_in, n_band,
                               x_epoch(a, l));
            }
        }
    }
}

// ---- 2b. up dots of the rows staged before the pick; their down rows take the slots ----------------
// Runs between the arrival at grid barrier B and the wait for it.  Team t takes rows t, t + P, ...; as soon as
// a team is done with a row's slot, the same feature's down row starts moving into it.
__device__ __noinline__ void phase_early(int l) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom& gm = cx.gm;
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x, lane = tid & 31;
    const int team = tid / gm.TS, c = tid % gm.TS, wt = c >> 5;
    const bool in_team = team < gm.P;
    const bool active = in_team && c < gm.G;
    const int s = c >> 2, g = c & 3, nblk = gm.nsb * 8;
    int* s_ctl = sm.ctl();
    const int n_early = s_ctl[SC_N_EARLY];
    const uint32_t par = (uint32_t)l & 1u;
    float* psum = sm.psum();
    float* act_s = psum + FW_MAX_GROWS * gm.Wt;
    const int* rows = sm.g_rows();
    const float* scores = sm.g_scores();
    uint8_t* ring = sm.ring();
    const uint8_t* down = layer_of(a, l).down;
    bool failed = false;
    if (in_team) {
        CellX x;
        {
            const int cl = active ? c : 0;  // unconditional: see the scan
            load_cellx(x, sm.xa(), sm.xb(), sm.blk(), nblk, (cl >> 2) * 8 + 2 * (cl & 3), gm.G, cl);
        }
        if (!mbar_wait(sm.ebar(0), par)) failed = true;
#pragma unroll 1
        for (int i = team; i < n_early; i += gm.P) {
            float val = 0.0f;
            if (active) {
                const uint8_t* cell = ring + (size_t)i * gm.row_bytes + s * 144;
                const uint4 hd = *reinterpret_cast<const uint4*>(cell);
                const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
                const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
                val = cell_value(hd, q0, q1, g, x);
            }
            for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
            if (lane == 0) psum[i * gm.Wt + wt] = val;
            bar_sync(1 + team, gm.TS);  // every thread of the team is done with the up row
            if (c == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // plain reads before the TMA write
                tma_bulk_g2s(ring + (size_t)i * gm.row_bytes, down + (size_t)(uint32_t)rows[i] * gm.row_bytes,
                             (uint32_t)gm.row_bytes, sm.ebar(1));
            }
        }
    } else if (!mbar_wait(sm.ebar(0), par)) {
        failed = true;  // (threads outside the teams pass the phase too)
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
#pragma unroll 1
    for (int i = tid; i < n_early; i += FW_CONSUMERS) {
        float upv = 0.0f;
#pragma unroll 1
        for (int w = 0; w < gm.Wt; ++w) upv += psum[i * gm.Wt + w];
        const float gs = scores[i];
        const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
        const float act = (gs * sig) * upv;
        act_s[i] = fabsf(act) > FW_NOISE_FLOOR ? act : 0.0f;
    }
    if (failed) s_ctl[SC_FAILED] = 1;
}

// The pick's rare path, kept out of line so that the usual path stays short: a band of more than
// FW_RANK_CAP entries.  Radix select of the threshold key among all band entries, then of the row cut among
// the entries that tie with it (the lowest rows win).  Up to FW_PICK_CAP entries are staged at the start of the
// ring by the caller; beyond that every read goes back to the band arrays.
template <bool X>
__device__ __noinline__ void pick_big_band(int l, int n_band_tot, int need, const int* seg_pre, uint32_t& tau_key,
                                           uint32_t& row_cut) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const FusedArgs& a = sm.cx().a;
    uint8_t* ring = sm.ring();
    const uint32_t* keys = reinterpret_cast<const uint32_t*>(ring);
    const uint32_t* rows = keys + FW_PICK_CAP;
    const bool staged = n_band_tot <= FW_PICK_CAP;
    const uint32_t* band_row_g = a.band_row;
    const float* band_exact_g = a.band_exact;
    const uint4* band_lines = X ? reinterpret_cast<const uint4*>(a.px.area[a.px.rank] + a.px.off_band) : nullptr;
    auto band_at = [&](int i) -> int {  // where entry i of all band entries sits in the band arrays
        if (!X) return i;
        int pre = 0, off = a.px.seg_off[0];
#pragma unroll 1
        for (int q = 1; q < a.px.world; ++q) {
            if (i >= seg_pre[q]) {
                pre = seg_pre[q];
                off = a.px.seg_off[q];
            }
        }
        return off + (i - pre);
    };
    SelectSmem<FW_CONSUMERS>& ssm = *reinterpret_cast<SelectSmem<FW_CONSUMERS>*>(ring + FW_PICK_CAP * 8);
    int cnt_gt, need_eq;
    // (a band too large to stage: every read waits for its line again, which costs nothing once it is there)
    auto entry = [&](int i, uint32_t& row) -> uint32_t {
        if (X) {
            uint32_t ex;
            line_wait(band_lines + band_at(i), x_epoch(a, l), row, ex, a.err);
            return abs_key(__uint_as_float(ex));
        }
        row = __ldcg(&band_row_g[i]);
        return abs_key(__ldcg(&band_exact_g[i]));
    };
    auto keyf = [&](int i) -> uint32_t {
        uint32_t row;
        return staged ? keys[i] : entry(i, row);
    };
    block_kth_largest_keys<FW_CONSUMERS, FW_BAR_CONS>(keyf, n_band_tot, need, ssm, tau_key, cnt_gt, need_eq);
    // ties at the threshold: the need_eq lowest rows win
    const uint32_t tau = tau_key;
    auto rowf = [&](int i) -> uint32_t {
        uint32_t row = 0u;
        const uint32_t key = staged ? keys[i] : entry(i, row);
        if (key != tau) return 0u;
        return ~(staged ? rows[i] : row);
    };
    uint32_t cut_key;
    int c2, n2;
    block_kth_largest_keys<FW_CONSUMERS, FW_BAR_CONS>(rowf, n_band_tot, need_eq, ssm, cut_key, c2, n2);
    row_cut = ~cut_key;
}

// ---- 3. final pick among all band rows, identically in every CTA ---------------------------------
template <bool X>
__device__ __noinline__ void phase_pick(int l) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom& gm = cx.gm;
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int* s_ctl = sm.ctl();
    float* red = sm.red();
    const int* band_list = sm.band_list();
    const float* band_ex = sm.band_ex();
    int* g2_rows = sm.g_rows();
    float* g2_scores = sm.g_scores();
    uint8_t* ring = sm.ring();
    const int n_band_mine = s_ctl[SC_N_BAND], n_keep = s_ctl[SC_N_KEEP];

    // X: the band entries of rank r sit at [seg_off[r], seg_off[r] + its count) of this GPU's copy of the
    // band arrays; entry i of the concatenation is found through the running counts seg_pre[].
    int n_in_tot, n_band_tot;
    int seg_pre[FW_MAX_WORLD + 1];
    const uint32_t* band_row_g = a.band_row;
    const float* band_exact_g = a.band_exact;
    const uint4* band_lines = nullptr;
    if (X) {
        // every rank's counts, as they arrive; this GPU's own say that its band and pool rows are all published
        const uint4* cnt = reinterpret_cast<const uint4*>(a.px.area[a.px.rank] + a.px.off_cnt);
        uint32_t c_in[FW_MAX_WORLD], c_band[FW_MAX_WORLD];
        lines_wait_ranks(cnt, 1, a.px.world, x_epoch(a, l), c_in, c_band, a.err);
        n_in_tot = 0;
        seg_pre[0] = 0;
#pragma unroll
        for (int r = 0; r < FW_MAX_WORLD; ++r) {
            n_in_tot += (int)c_in[r];
            seg_pre[r + 1] = seg_pre[r] + (int)c_band[r];
        }
        __threadfence();  // the pool rows and counts below were written before the counts were sent
        n_band_tot = min(seg_pre[FW_MAX_WORLD], a.px.n_rows_global);
        band_lines = reinterpret_cast<const uint4*>(a.px.area[a.px.rank] + a.px.off_band);
    } else {
        n_in_tot = (int)__ldcg(&a.ctrs[CTR_IN]);
        n_band_tot = min((int)__ldcg(&a.ctrs[CTR_BAND]), a.n_rows);
    }
    auto band_at = [&](int i) -> int {  // where entry i of all band entries sits in the band arrays
        if (!X) return i;
        int pre = 0, off = a.px.seg_off[0];
#pragma unroll
        for (int q = 1; q < FW_MAX_WORLD; ++q) {
            const bool in = q < a.px.world && i >= seg_pre[q];
            pre = in ? seg_pre[q] : pre;
            off = in ? a.px.seg_off[q] : off;
        }
        return off + (i - pre);
    };
    const int row_add = X ? a.px.row_offset : 0;  // own rows as global row numbers
    const int need = a.top_k - n_in_tot;
    uint32_t tau_key = 0, row_cut = 0xffffffffu;
    bool take_all = need >= n_band_tot;
    // Small bands (the usual case): every CTA ranks its own band rows against all band
    // entries by counting; large bands fall back to a radix select of the threshold.
    const bool by_rank = !take_all && need > 0 && n_band_tot <= FW_RANK_CAP;
    // A band of up to FW_RANK_CAP entries (the usual case) is staged at the end of the ring, behind the slots
    // that were filled before the pick; a larger one needs the ring from its start: the rows staged early
    // are then given up (their copies are waited for first) and the gather fetches them again.
    uint32_t* keys = reinterpret_cast<uint32_t*>(by_rank ? ring + gm.off_pick : ring);
    uint32_t* rows = keys + (by_rank ? FW_RANK_CAP : FW_PICK_CAP);
    int* win_s = by_rank ? reinterpret_cast<int*>(rows + FW_RANK_CAP) : reinterpret_cast<int*>(ring + FW_PICK_CAP * 8);
    if (!take_all && need > 0 && !by_rank) {
        if (!mbar_wait(sm.ebar(1), (uint32_t)l & 1u)) s_ctl[SC_FAILED] = 1;
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        if (tid == 0) s_ctl[SC_N_EARLY] = 0;
    }
    int* ired = reinterpret_cast<int*>(red);
    int* scal = ired + 1240;     // my first pool item, my share
    int* prefix = ired + 1280;   // [NC + 1] pool segments (start of every CTA's rows in the pool)
    constexpr int STAGERS = FW_CONSUMERS - 32;  // the last warp shares out the pool meanwhile
    if (warp == FW_NWARPS - 1) {
        // This CTA's share of the pooled certainly-in rows.  Every CTA computes the same assignment from the
        // published counts: CTA c has load e_c (own rows + band rows) and the pool is poured over the CTAs
        // like water, the least loaded first, up to a common level L; a CTA below the level takes L - e_c
        // pool rows (one fewer for the last few, so that the shares add up to the pool), as a contiguous
        // range of the pool in CTA order.  A fixed rule: results stay run-to-run identical.  One warp,
        // lane j holding CTAs j*cpl .. j*cpl + cpl - 1.
        const int NC = (int)gridDim.x, cpl = (NC + 31) / 32;
        auto wsum = [](int v) {
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            return v;
        };
        auto wscan_excl = [&](int v) {  // exclusive prefix over the lanes
            int inc = v;
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            return inc - v;
        };
        int ov[8], ev[8];
        int lane_over = 0, lane_e = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane * cpl + i;
            const bool valid = i < cpl && c < NC;
            ov[i] = valid ? (int)__ldcg(&a.pool_cnt[c]) : 0;
            ev[i] = valid ? (int)__ldcg(&a.pool_cnt[512 + c]) : 0x3fffffff;
            lane_over += ov[i];
            lane_e += valid ? ev[i] : 0;
        }
        const int total = wsum(lane_over), sum_e = wsum(lane_e);
        {
            int run = wscan_excl(lane_over);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = lane * cpl + i;
                if (i < cpl && c < NC) prefix[c] = run;
                run += ov[i];
            }
            if (lane == 0) prefix[NC] = total;
        }
        auto fill_at = [&](int level) {  // sum over CTAs of max(0, level - e_c)
            int f = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) f += max(0, level - ev[i]);
            return wsum(f);
        };
        // the level is the smallest L with fill(L) >= total; ceil((sum e + total) / NC) is an upper bound
        int level = total > 0 ? (sum_e + total + NC - 1) / NC : 0;
        while (level > 0 && fill_at(level - 1) >= total) level -= 1;
        const int excess = fill_at(level) - total;
        int lane_below = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) lane_below += ev[i] < level ? 1 : 0;
        const int n_below = wsum(lane_below);
        int rank = wscan_excl(lane_below);
        int share[8], lane_share = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool below = ev[i] < level;
            share[i] = below ? level - ev[i] - (rank >= n_below - excess ? 1 : 0) : 0;
            rank += below ? 1 : 0;
            lane_share += share[i];
        }
        int first = wscan_excl(lane_share);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < cpl && lane * cpl + i == (int)blockIdx.x) {
                scal[0] = first;
                scal[1] = share[i];
            }
            first += share[i];
        }
    }
    // This CTA's share of the pool is fetched into registers as soon as the share is known (after the barrier that
    // ends the staging below) and stored once the winners are counted: its round trip to global memory runs
    // beside the ranking.
    bool pool_early = false;
    uint32_t pool_r = 0u;
    float pool_s = 0.0f;
    auto pool_src = [&](int j) -> size_t {
        const int NC = (int)gridDim.x;
        int sa = 0, sb = NC;  // prefix[sa] <= j < prefix[sb]
        while (sb - sa > 1) {
            const int mid = (sa + sb) >> 1;
            if (prefix[mid] <= j) sa = mid;
            else sb = mid;
        }
        return (size_t)sa * gm.max_slots + (size_t)(j - prefix[sa]);
    };
    if (!take_all && need > 0) {
        // stage (|v| key, row) of every band entry in the idle ring
        const bool staged = n_band_tot <= FW_PICK_CAP;
        if (staged) {
            if (tid < STAGERS)
#pragma unroll 1
                for (int i = tid; i < n_band_tot; i += STAGERS) {
                    if (X) {
                        uint32_t row, ex;
                        line_wait(band_lines + band_at(i), x_epoch(a, l), row, ex, a.err);
                        keys[i] = abs_key(__uint_as_float(ex));
                        rows[i] = row;
                    } else {
                        keys[i] = abs_key(__ldcg(&band_exact_g[i]));
                        rows[i] = __ldcg(&band_row_g[i]);
                    }
                }
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
            if (scal[1] <= FW_CONSUMERS) {  // (the last warp's results are in place after the barrier)
                pool_early = true;
                if (tid < scal[1]) {
                    const size_t src = pool_src(scal[0] + tid);
                    pool_r = __ldcg(&a.pool_row[src]);
                    pool_s = __ldcg(&a.pool_score[src]);
                }
            }
        }
        if (by_rank) {
#pragma unroll 1
            for (int i = warp; i < n_band_mine; i += FW_NWARPS) {
                const uint32_t key = abs_key(band_ex[i]);
                const uint32_t row = (uint32_t)(row_of_slot(cx, band_list[i]) + row_add);
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
            pick_big_band<X>(l, n_band_tot, need, seg_pre, tau_key, row_cut);
            bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        }
    }
    // winners among this CTA's band rows, in slot order, after the CTA's own certainly-in rows
    if (warp == 0) {
        int cnt = 0;
#pragma unroll 1
        for (int i0 = 0; i0 < n_band_mine; i0 += 32) {
            const int i = i0 + lane;
            bool win = false;
            uint32_t row = 0;
            if (i < n_band_mine && need > 0) {
                const uint32_t key = abs_key(band_ex[i]);
                row = (uint32_t)(row_of_slot(cx, band_list[i]) + row_add);
                win = by_rank ? (win_s[i] != 0) : (take_all || key > tau_key || (key == tau_key && row <= row_cut));
            }
            const uint32_t bal = __ballot_sync(0xffffffffu, win);
            if (win) {
                const int pos = n_keep + cnt + __popc(bal & ((1u << lane) - 1u));
                g2_rows[pos] = (int)row - row_add;  // the gather addresses this rank's own rows
                g2_scores[pos] = band_ex[i];        // the gather uses the exact gate score
            }
            cnt += __popc(bal);
        }
        if (lane == 0) s_ctl[SC_N_G2] = n_keep + cnt;
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // winners and the pool assignment are in place
    {
        const int n_win = s_ctl[SC_N_G2];  // own rows and winners so far
        const int my_first = scal[0], n_pool_mine = scal[1];
        if (pool_early) {
            if (tid < n_pool_mine) {
                g2_rows[n_win + tid] = (int)pool_r;
                g2_scores[n_win + tid] = pool_s;
            }
        } else {
#pragma unroll 1
            for (int i = tid; i < n_pool_mine; i += FW_CONSUMERS) {
                const size_t src = pool_src(my_first + i);
                g2_rows[n_win + i] = (int)__ldcg(&a.pool_row[src]);
                g2_scores[n_win + i] = __ldcg(&a.pool_score[src]);
            }
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // (every thread has read the counts above)
        if (tid == 0) s_ctl[SC_N_G2] = n_win + n_pool_mine;
    }
    if (l + 1 == a.n_layers && a.stats && blockIdx.x == 0 && tid == 0) {
        a.stats->n_certain = n_in_tot;
        a.stats->n_band = n_band_tot;
        a.stats->n_hits = min(a.top_k, X ? a.px.n_rows_global : a.n_rows);
        a.stats->need = need;
    }
    if (!X && l + 1 == a.n_layers && a.count_out && blockIdx.x == 0 && tid == 0)
        *a.count_out = (uint32_t)min(a.top_k, a.n_rows);
    // the pick staged plain stores in the ring; order them before the TMA writes of the gather
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
}

// The teams' accumulators, staged in the ring (one region per team, 64-float chunks at a stride of 65), are
// summed in team order into this CTA's partial out[H] (first: stored; later chunks: added).
__device__ __forceinline__ void merge_partials(bool first) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const FusedGeom& gm = sm.cx().gm;
    const int tid = threadIdx.x, hidden = gm.nsb * 256, P = gm.P;
    const float* out_r = reinterpret_cast<const float*>(sm.ring());
    const int region = gm.G * 65;
    float* dst = sm.cx().a.partials + (size_t)blockIdx.x * hidden;
    // four outputs per trip, their loads issued together (the teams' values are added in team order either way)
    for (int i0 = tid; i0 < hidden; i0 += 4 * FW_CONSUMERS) {
        float v[4];
        int o[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = min(i0 + u * FW_CONSUMERS, hidden - 1);
            o[u] = (i >> 6) * 65 + (i & 63);
            v[u] = out_r[o[u]];
        }
        for (int p = 1; p < P; ++p) {
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] += out_r[p * region + o[u]];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * FW_CONSUMERS;
            if (i < hidden) dst[i] = first ? v[u] : dst[i] + v[u];
        }
    }
    // the merge used the ring with plain loads and stores; order them before the next TMA writes
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // the staging area is free again
}

// The gather's rare path, kept out of line: a CTA with more rows than the ring stages at once takes the rest
// chunk by chunk (up rows staged, dotted, down rows into the same slots, added), each chunk merged into the partial.
__device__ __noinline__ void gather_more_chunks(int l, int n0, int n_g2) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const FusedGeom& gm = sm.cx().gm;
    int* s_ctl = sm.ctl();
    const FusedLayer ly = layer_of(sm.cx().a, l);
    uint32_t gather_uses = (uint32_t)s_ctl[SC_GATHER_USES];
    bool failed = false;
#pragma unroll 1
    for (int base = n0; base < n_g2; base += gm.D2) {
        GatherArgs ga;
        ga.up = ly.up; ga.down = ly.down; ga.rows = sm.g_rows(); ga.scores = sm.g_scores(); ga.ring = sm.ring();
        ga.psum = sm.psum(); ga.act = sm.psum() + FW_MAX_GROWS * gm.Wt; ga.bar = sm.gbar(); ga.ubar = sm.gbar() + 1;
        ga.xa_s = sm.xa(); ga.xb_s = sm.xb(); ga.blk_s = sm.blk();
        ga.nsb = gm.nsb; ga.G = gm.G; ga.TS = gm.TS; ga.P = gm.P; ga.Wt = gm.Wt; ga.row_bytes = gm.row_bytes;
        gather_stage(ga, base, min(gm.D2, n_g2 - base), gather_uses & 1u, failed);  // leaves the accumulators staged in the ring
        gather_uses += 1;
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        merge_partials(false);
    }
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    if (threadIdx.x == 0) s_ctl[SC_GATHER_USES] = (int)gather_uses;
    if (failed) s_ctl[SC_FAILED] = 1;
}

// ---- gather: own certainly-in rows (up to the fair share), band winners, pool share; merge ------
__device__ __noinline__ void phase_gather(int l) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom& gm = cx.gm;
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x;
    const int P = gm.P;
    int* s_ctl = sm.ctl();
    const int n_g2 = s_ctl[SC_N_G2];
    bool failed = false;
    const FusedLayer ly = layer_of(a, l);
    // First chunk: rows [0, n_early) were staged before the pick (up dots done, activations in place, down rows
    // on their way into the same slots); rows [n_early, n0) are what the pick added (band winners, pool share).
    // Their up rows go to slots n_early.. and, where the ring has room, their down rows to slots n0.. at once;
    // while those copies travel the early rows are added into the accumulators.
    const int n0 = min(n_g2, gm.D2);
    {
        const int lane = tid & 31;
        const int team = tid / gm.TS, c = tid % gm.TS, wt = c >> 5;
        const bool in_team = team < P;
        const bool active = in_team && c < gm.G;
        const int s = c >> 2, g = c & 3, nblk = gm.nsb * 8, rb = gm.row_bytes;
        const uint32_t par = (uint32_t)l & 1u;
        const int n_early = min(s_ctl[SC_N_EARLY], n0);
        const int n_x = n0 - n_early;
        const bool both = n0 + n_x <= gm.D2;
        const int* rows = sm.g_rows();
        const float* scores = sm.g_scores();
        uint8_t* ring = sm.ring();
        float* psum = sm.psum();
        float* act_s = psum + FW_MAX_GROWS * gm.Wt;
        if (tid == 0) {
            mbar_expect_tx(sm.ebar(2), (uint32_t)n_x * (uint32_t)rb);
            mbar_expect_tx(sm.ebar(3), (uint32_t)n_x * (uint32_t)rb);
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // the expectations are armed before any copy can complete
#pragma unroll 1
        for (int i = tid; i < n_x; i += FW_CONSUMERS) {
            const size_t src = (size_t)(uint32_t)rows[n_early + i] * rb;
            tma_bulk_g2s(ring + (size_t)(n_early + i) * rb, ly.up + src, (uint32_t)rb, sm.ebar(2));
            if (both) tma_bulk_g2s(ring + (size_t)(n0 + i) * rb, ly.down + src, (uint32_t)rb, sm.ebar(3));
        }
        float acc_lo[32], acc_hi[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc_lo[j] = acc_hi[j] = 0.0f;
        float corr_lo = 0.0f, corr_hi = 0.0f;
        // the early rows' down rows
        if (!failed && !mbar_wait(sm.ebar(1), par)) failed = true;
        if (active) {
#pragma unroll 1
            for (int i = team; i < n_early; i += P) {
                const float act = act_s[i];
                if (act == 0.0f) continue;
                axpy_cell(ring + (size_t)i * rb + s * 144, g, act, acc_lo, acc_hi, corr_lo, corr_hi);
            }
        }
        // the added rows: up dots against the planes in shared memory (the accumulators hold the registers)
        if (!failed && !mbar_wait(sm.ebar(2), par)) failed = true;
        if (in_team) {
            const int cl = active ? c : 0;
#pragma unroll 1
            for (int i = team; i < n0; i += P) {
                if (i < n_early) continue;
                float val = 0.0f;
                if (active) {
                    const uint8_t* cell = ring + (size_t)i * rb + s * 144;
                    const uint4 hd = *reinterpret_cast<const uint4*>(cell);
                    const uint4 q0 = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
                    const uint4 q1 = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
                    val = cell_value_smem(hd, q0, q1, g, sm.xa(), sm.xb(), sm.blk(), nblk, (cl >> 2) * 8 + 2 * (cl & 3),
                                          gm.G, cl);
                }
                for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
                if (lane == 0) psum[i * gm.Wt + wt] = val;
                if (!both) {
                    bar_sync(1 + team, gm.TS);  // every thread of the team is done with the up row
                    if (c == 0) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // plain reads before the TMA write
                        tma_bulk_g2s(ring + (size_t)i * rb, ly.down + (size_t)(uint32_t)rows[i] * rb, (uint32_t)rb, sm.ebar(3));
                    }
                }
            }
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
#pragma unroll 1
        for (int i = n_early + tid; i < n0; i += FW_CONSUMERS) {
            float upv = 0.0f;
#pragma unroll 1
            for (int w = 0; w < gm.Wt; ++w) upv += psum[i * gm.Wt + w];
            const float gs = scores[i];
            const float sig = __fdiv_rn(1.0f, 1.0f + expf(-gs));
            const float act = (gs * sig) * upv;
            act_s[i] = fabsf(act) > FW_NOISE_FLOOR ? act : 0.0f;
        }
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        if (!failed && !mbar_wait(sm.ebar(3), par)) failed = true;
        if (active) {
#pragma unroll 1
            for (int i = team; i < n0; i += P) {
                if (i < n_early) continue;
                const float act = act_s[i];
                if (act == 0.0f) continue;
                const int slot = both ? n0 + (i - n_early) : i;
                axpy_cell(ring + (size_t)slot * rb + s * 144, g, act, acc_lo, acc_hi, corr_lo, corr_hi);
            }
        }
        // every team has finished reading the staged rows: the ring now takes the accumulators
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        if (active) {
            float* o_lo = reinterpret_cast<float*>(ring) + team * (gm.G * 65) + c * 65;
            float* o_hi = o_lo + 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                o_lo[j] = acc_lo[j] - corr_lo;
                o_hi[j] = acc_hi[j] - corr_hi;
            }
        }
    }
    if (a.pf_late) prefetch_next_gate(sm, l);
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);
    FW_STAMP(8);
    merge_partials(true);
    if (n0 < n_g2) gather_more_chunks(l, n0, n_g2);
    if (failed) s_ctl[SC_FAILED] = 1;

    // optional: selected rows of the last layer (unordered)
    if (l + 1 == a.n_layers && a.hit_out) {
        if (tid == 0) s_ctl[SC_HIT_BASE] = (int)atomicAdd(&a.ctrs[CTR_HITS], (uint32_t)n_g2);
        bar_sync(FW_BAR_CONS, FW_CONSUMERS);
        const int base = s_ctl[SC_HIT_BASE];
        const int* g2_rows = sm.g_rows();
#pragma unroll 1
        for (int i = tid; i < n_g2; i += FW_CONSUMERS)
            if (base + i < a.top_k) a.hit_out[base + i] = (uint32_t)g2_rows[i];  // (a sharded walk: this rank's own row numbers)
    }
    // the ring is free: the next layer's first tiles may land
    if (tid < cx.n_ahead && l + 1 < a.n_layers) {  // (thread k issues tile k: every stage has its own barrier)
        const FusedLayer nx = a.layers[l + 1];
        const uint32_t it0 = (uint32_t)(l + 1) * (uint32_t)cx.my_count;
        issue_tile(sm, nx, tid, it0 + tid);
    }
    // housekeeping for the layer after next (nobody reads these before two more grid barriers)
    uint4* hist4 = reinterpret_cast<uint4*>(a.hist + (size_t)(l & 1) * FW_HIST_WORDS);
    for (int i = blockIdx.x * FW_CONSUMERS + tid; i < FW_HIST_WORDS / 4; i += gridDim.x * FW_CONSUMERS)
        hist4[i] = make_uint4(0u, 0u, 0u, 0u);
    if (blockIdx.x == 0 && tid == 0) {
        a.ctrs[CTR_BOUND0 + (l & 1)] = 0;
        a.ctrs[CTR_MAXBIN0 + (l & 1)] = 0;
    }
}

// ---- 4. finish: fixed-order sum of a column slice of the partials + residual --------------------
// X: the slice sum first goes into slot `rank` of every rank's xsum, and the slots are added up in rank order.
template <bool X>
__device__ __noinline__ void phase_finish(const float* h_cur, float* h_next, uint32_t ep) {
    extern __shared__ __align__(128) uint8_t smem[];  // the kernel's dynamic shared memory
    const Smem sm{smem};
    const Ctx& cx = sm.cx();
    const FusedGeom& gm = cx.gm;
    const FusedArgs& a = cx.a;
    const int tid = threadIdx.x;
    const int hidden = gm.nsb * 256;
    const int ncol4 = hidden / 4;
    const int per = (ncol4 + gridDim.x - 1) / gridDim.x;      // float4 columns per CTA
    const int col0 = blockIdx.x * per, ncol = max(0, min(per, ncol4 - col0));
    const int ygroups = max(1, min(FW_CONSUMERS / max(per, 1), 64));
    float4* red4 = reinterpret_cast<float4*>(sm.red());       // [ygroups][per] (<= 512 entries)
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
        if (X) {
            // this rank's sums of the slice go to every rank; the slice of the layer's output is every rank's
            // sums added up in rank order (the same on every rank), taken as they arrive
            const size_t at = 2 * (size_t)(col0 + tid);
            for (int p = 0; p < a.px.world; ++p) {
                uint4* xl = reinterpret_cast<uint4*>(a.px.area[p] + a.px.off_xsum) + (size_t)a.px.rank * (hidden / 2) + at;
                line_store(xl, __float_as_uint(t.x), __float_as_uint(t.y), ep);
                line_store(xl + 1, __float_as_uint(t.z), __float_as_uint(t.w), ep);
            }
            const uint4* xsum = reinterpret_cast<const uint4*>(a.px.area[a.px.rank] + a.px.off_xsum) + at;
            t = make_float4(0.f, 0.f, 0.f, 0.f);
            uint32_t w0[FW_MAX_WORLD], w1[FW_MAX_WORLD], w2[FW_MAX_WORLD], w3[FW_MAX_WORLD];
            lines_wait_ranks(xsum, (size_t)(hidden / 2), a.px.world, ep, w0, w1, a.err);
            lines_wait_ranks(xsum + 1, (size_t)(hidden / 2), a.px.world, ep, w2, w3, a.err);
#pragma unroll
            for (int r = 0; r < FW_MAX_WORLD; ++r)
                if (r < a.px.world) {
                    t.x += __uint_as_float(w0[r]); t.y += __uint_as_float(w1[r]);
                    t.z += __uint_as_float(w2[r]); t.w += __uint_as_float(w3[r]);
                }
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
    bar_sync(FW_BAR_CONS, FW_CONSUMERS);  // red is reused by the next phase
}

// Parameters -> shared memory, barriers, the first tiles of layer 0.
__device__ __forceinline__ void fused_setup(const FusedGeom& gm_in, const FusedArgs& a_in) {
    extern __shared__ __align__(128) uint8_t smem[];
    const Smem sm{smem};
    const int tid = threadIdx.x;
    Ctx& cxw = sm.cx();
    const uint32_t* gsrc = reinterpret_cast<const uint32_t*>(&gm_in);
    const uint32_t* asrc = reinterpret_cast<const uint32_t*>(&a_in);
    uint32_t* gdst = reinterpret_cast<uint32_t*>(&cxw.gm);
    uint32_t* adst = reinterpret_cast<uint32_t*>(&cxw.a);
#pragma unroll 1
    for (int i = tid; i < (int)(sizeof(FusedGeom) / 4); i += FW_THREADS) gdst[i] = gsrc[i];
#pragma unroll 1
    for (int i = tid; i < (int)(sizeof(FusedArgs) / 4); i += FW_THREADS) adst[i] = asrc[i];
    if (tid == 0) {
        const int R = gm_in.R;
        cxw.n_tiles = (a_in.n_rows + R - 1) / R;
        cxw.first_tile = blockIdx.x;
        cxw.my_count =
            (int)blockIdx.x < cxw.n_tiles ? (cxw.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
        cxw.n_slots = cxw.my_count * R;
        cxw.n_ahead = min(gm_in.S, cxw.my_count);  // tiles issued before a layer's scan starts (a full ring)
        cxw.stamp_layer = a_in.n_layers >= 2 ? a_in.n_layers - 2 : 0;
        int* s_ctl = sm.ctl();
        for (int i = 0; i < 16; ++i) s_ctl[i] = 0;
#pragma unroll 1
        for (int i = 0; i < gm_in.S; ++i) {
            mbar_init(&sm.full()[i], 1);
            sm.released()[i] = 0;
        }
        mbar_init(sm.gbar(), 1);
        mbar_init(sm.gbar() + 1, 1);
        for (int i = 0; i < 5; ++i) mbar_init(sm.ebar(i), 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (tid == 0) {
        const Ctx& cx = sm.cx();
        const FusedLayer l0 = layer_of(cx.a, 0);
#pragma unroll 1
        for (int k = 0; k < cx.n_ahead; ++k) issue_tile(sm, l0, k, (uint32_t)k);
    }
}

__global__ void __launch_bounds__(FW_THREADS, 1)
walk_fused_q4k_kernel(const __grid_constant__ FusedGeom gm_in, const __grid_constant__ FusedArgs a_in) {
    extern __shared__ __align__(128) uint8_t smem[];
    const Smem sm{smem};
    fused_setup(gm_in, a_in);
    const Ctx& cx = sm.cx();
    const FusedArgs& a = cx.a;
    int* s_ctl = sm.ctl();
    uint32_t epoch = 0;
    bool failed = false;
    const float* h_cur = a.h_in;
    const int n_layers = a.n_layers;
    for (int l = 0; l < n_layers; ++l) {
        float* h_next = (l + 1 == n_layers) ? a.h_out : ((l & 1) ? a.hbuf1 : a.hbuf0);
        FW_STAMP(0);
        phase_prepare(l, h_cur);
        FW_STAMP(1);
        phase_scan(l);
        FW_STAMP(2);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[SC_FAILED]);  // A: histogram complete
        FW_STAMP(3);
        phase_select<false>(l);
        FW_STAMP(5);
        // B: band and pool rows published.  Between arriving and waiting, the up dots of the rows staged early.
        epoch += 1;
        grid_arrive(&a.ctrs[CTR_SYNC], failed);
        phase_early(l);
        grid_wait(&a.ctrs[CTR_SYNC], epoch * gridDim.x, a.err, failed, &s_ctl[SC_FAILED]);
        FW_STAMP(6);
        phase_pick<false>(l);
        FW_STAMP(7);
        phase_gather(l);
        FW_STAMP(9);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[SC_FAILED]);  // C: partials written
        FW_STAMP(10);
        phase_finish<false>(h_cur, h_next, 0u);
        FW_STAMP(11);
        h_cur = h_next;
        if (l + 1 < n_layers) grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[SC_FAILED]);  // D: next residual
        FW_STAMP(12);
    }
    if (failed || s_ctl[SC_FAILED]) set_err(a.err, DEV_ERR_TMA_TIMEOUT);
}

// The same walk on one rank of a feature-sharded stack: this GPU's rows of every layer, the selection made
// over all ranks' rows.  Per layer:
//   scan own rows; barrier over this GPU's CTAs (its histogram is complete); histogram slices to every rank;
//   threshold from every rank's histogram (lines taken as they arrive) and classification; own band rows to
//   every rank, and once all of this GPU's CTAs have done so, its counts;
//   final pick over every rank's band rows (the same on every CTA of every rank), gather of own rows;
//   barrier over this GPU's CTAs; slice sums of the partials to every rank; every rank's sums of the slice,
//   as they arrive, plus the residual make the slice of the next residual; barrier over this GPU's CTAs.
// Three barriers per layer, all local; the ranks wait for each other only where they read each other's lines.
__global__ void __launch_bounds__(FW_THREADS, 1)
walk_fused_q4k_sharded_kernel(const __grid_constant__ FusedGeom gm_in, const __grid_constant__ FusedArgs a_in) {
    extern __shared__ __align__(128) uint8_t smem[];
    const Smem sm{smem};
    fused_setup(gm_in, a_in);
    const Ctx& cx = sm.cx();
    const FusedArgs& a = cx.a;
    int* s_ctl = sm.ctl();
    uint32_t epoch = 0;
    bool failed = false;
    const float* h_cur = a.h_in;
    const int n_layers = a.n_layers;
    for (int l = 0; l < n_layers; ++l) {
        float* h_next = (l + 1 == n_layers) ? a.h_out : ((l & 1) ? a.hbuf1 : a.hbuf0);
        FW_STAMP(0);
        phase_prepare(l, h_cur);
        FW_STAMP(1);
        phase_scan(l);
        FW_STAMP(2);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[SC_FAILED]);  // A: this GPU's histogram complete
        phase_xhist(l);
        FW_STAMP(3);
        phase_select<true>(l);
        FW_STAMP(5);
        phase_early(l);
        FW_STAMP(6);
        phase_pick<true>(l);
        FW_STAMP(7);
        phase_gather(l);
        FW_STAMP(9);
        grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[SC_FAILED]);  // C: this GPU's partials written
        FW_STAMP(10);
        phase_finish<true>(h_cur, h_next, x_epoch(a, l));
        FW_STAMP(11);
        h_cur = h_next;
        if (l + 1 < n_layers) grid_sync(&a.ctrs[CTR_SYNC], epoch, a.err, failed, &s_ctl[SC_FAILED]);  // D: next residual
        FW_STAMP(12);
    }
    if (a.count_out && blockIdx.x == 0 && threadIdx.x == 0) *a.count_out = __ldcg(&a.ctrs[CTR_HITS]);
    if (failed || s_ctl[SC_FAILED]) set_err(a.err, DEV_ERR_TMA_TIMEOUT);
}

}  // namespace

// Host side ------------------------------------------------------------------------
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
    return (size_t)2 * FW_HIST_WORDS * 4 + 256 + (size_t)n_rows * 8 + 512 + 2 * pool + 4096 +
           (size_t)sm_count * hidden * 4 + (size_t)2 * hidden * 4 + 4096;
}

int fused_q4k_stamp_count() { return FW_STAMPS; }

// The leading part of the workspace that a failed launch may leave dirty: histograms and counters.
size_t fused_q4k_ws_dirty_bytes() { return (size_t)2 * FW_HIST_WORDS * 4 + 256; }

namespace {

struct XLayout {
    uint32_t off_meta, off_cnt, off_hist, off_band, off_xsum;
    size_t bytes;
};
XLayout x_layout(int hidden, int n_rows_global, int world) {  // everything in 16-byte lines
    XLayout x;
    size_t o = 0;
    x.off_meta = (uint32_t)o;  o += 256;
    x.off_cnt = (uint32_t)o;   o += 256;
    o = 1024;
    x.off_hist = (uint32_t)o;  o += (size_t)world * (LQ_HIST_BINS / 2) * 16;
    x.off_band = (uint32_t)o;  o += ((size_t)n_rows_global * 16 + 255) / 256 * 256;
    x.off_xsum = (uint32_t)o;  o += (size_t)world * (hidden / 2) * 16;
    x.bytes = (o + 255) / 256 * 256;
    return x;
}

cudaError_t fill_args(FusedArgs& a, const FusedGeom& g, const void* layers_dev, const uint8_t* const* single,
                      int n_layers, int n_rows, int hidden, int top_k, uint32_t flags, float c1, const float* h_in,
                      float* h_out, uint8_t* ws, uint32_t* hit_out, uint32_t* count_out, lq_walk_stats* stats_dev,
                      int* err, int sm_count, cudaStream_t st) {
    a.layers = reinterpret_cast<const FusedLayer*>(layers_dev);
    a.single = single ? FusedLayer{single[0], single[1], single[2]} : FusedLayer{nullptr, nullptr, nullptr};
    a.n_layers = n_layers;
    a.n_rows = n_rows;
    a.top_k = top_k;
    a.flags = flags;
    a.c1 = c1;
    // L2 prefetch of gate tiles ahead of the ring (within a layer: LARQL_B200_FUSED_PFD tiles; across layers,
    // during the previous layer's tail: LARQL_B200_FUSED_PF tiles).  Off by default: measured on B200 the scan
    // waits for data only a tenth of its time, and the prefetch traffic slows the gather by more than it saves.
    static const int pf_env = [] { const char* v = getenv("LARQL_B200_FUSED_PF"); return v ? atoi(v) : -1; }();
    static const int pf_late_env = [] { const char* v = getenv("LARQL_B200_FUSED_PF_LATE"); return v ? atoi(v) : 1; }();
    static const int pf_dist_env = [] { const char* v = getenv("LARQL_B200_FUSED_PFD"); return v ? atoi(v) : 0; }();
    a.pf_dist = pf_dist_env;
    a.pf_tiles = (a.layers && n_layers > 1 && pf_env > 0) ? pf_env : 0;
    a.pf_late = pf_late_env ? 1 : 0;
    {
        const char* v = stats_dev ? getenv("LARQL_B200_FUSED_STAMP_CTA") : nullptr;  // (read per stamped launch: a diagnostic)
        a.stamp_cta = v ? atoi(v) : 0;
    }
    a.h_in = h_in;
    a.h_out = h_out;
    uint8_t* p = ws;
    a.hist = reinterpret_cast<uint32_t*>(p);        p += (size_t)2 * FW_HIST_WORDS * 4;
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
    memset(&a.px, 0, sizeof a.px);
    a.px.world = 1;
    // the barrier counters and the per-launch counters start from zero (the histogram is kept
    // zero by the kernel itself; a failed launch is followed by a full clear on the host side)
    return cudaMemsetAsync(a.ctrs, 0, 256, st);
}

}  // namespace

size_t fused_q4k_xarea_bytes(int hidden, int n_rows_global, int world) {
    return x_layout(hidden, n_rows_global, world).bytes;
}

bool fused_q4k_sharded_supported(int hidden, int n_rows_local, int n_rows_global, int top_k, int world, int sm_count) {
    FusedGeom g;
    if (world < 1 || world > FW_MAX_WORLD || n_rows_local <= 0 || top_k <= 0 || top_k >= n_rows_global) return false;
    if (!fused_geom(hidden, n_rows_local, sm_count, g)) return false;
    const int per = (hidden / 4 + sm_count - 1) / sm_count;
    // every CTA of every rank takes part in every barrier: a rank needs at least one tile per CTA
    const int n_tiles = (n_rows_local + g.R - 1) / g.R;
    return per <= FW_CONSUMERS && g.max_slots <= 16384 && n_tiles >= sm_count;
}

// One rank's launch of a sharded walk.  areas[r]: rank r's exchange area (fused_q4k_xarea_bytes(), zeroed
// once when it was created) as mapped into this process; row_offsets[r]: first global row of rank r;
// xepoch0: how many layers earlier launches on these areas have walked (the exchange lines' epoch).
cudaError_t launch_walk_fused_q4k_sharded(const void* layers_dev, int n_layers, int n_rows_local, int n_rows_global,
                                          int hidden, int top_k, uint32_t flags, float c1, const float* h_in,
                                          float* h_out, uint8_t* ws, uint32_t* hit_out, uint32_t* count_out,
                                          lq_walk_stats* stats_dev, int* err, int sm_count, int world, int rank,
                                          uint8_t* const* areas, const int* row_offsets, uint32_t xepoch0,
                                          cudaStream_t st) {
    FusedGeom g;
    if (!fused_q4k_sharded_supported(hidden, n_rows_local, n_rows_global, top_k, world, sm_count))
        return cudaErrorInvalidValue;
    fused_geom(hidden, n_rows_local, sm_count, g);
    cudaError_t e = set_max_dyn_smem((const void*)walk_fused_q4k_sharded_kernel, 227 * 1024);
    if (e != cudaSuccess) return e;
    FusedArgs a;
    e = fill_args(a, g, layers_dev, nullptr, n_layers, n_rows_local, hidden, top_k, flags, c1, h_in, h_out, ws, hit_out,
                  count_out, stats_dev, err, sm_count, st);
    if (e != cudaSuccess) return e;
    const XLayout x = x_layout(hidden, n_rows_global, world);
    a.px.world = world;
    a.px.rank = rank;
    a.px.row_offset = row_offsets[rank];
    a.px.n_rows_global = n_rows_global;
    a.px.xepoch0 = xepoch0;
    a.px.off_meta = x.off_meta;
    a.px.off_cnt = x.off_cnt;
    a.px.off_hist = x.off_hist;
    a.px.off_band = x.off_band;
    a.px.off_xsum = x.off_xsum;
    for (int r = 0; r < world; ++r) {
        a.px.seg_off[r] = row_offsets[r];
        a.px.area[r] = areas[r];
    }
    void* args[] = {&g, &a};
    return cudaLaunchCooperativeKernel((const void*)walk_fused_q4k_sharded_kernel, dim3(sm_count), dim3(FW_THREADS), args,
                                       (size_t)g.smem_bytes, st);
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
    cudaError_t e = set_max_dyn_smem((const void*)walk_fused_q4k_kernel, 227 * 1024);
    if (e != cudaSuccess) return e;
    FusedArgs a;
    e = fill_args(a, g, layers_dev, single, n_layers, n_rows, hidden, top_k, flags, c1, h_in, h_out, ws, hit_out,
                  count_out, stats_dev, err, sm_count, st);
    if (e != cudaSuccess) return e;
    void* args[] = {&g, &a};
    return cudaLaunchCooperativeKernel((const void*)walk_fused_q4k_kernel, dim3(grid), dim3(FW_THREADS), args,
                                       (size_t)g.smem_bytes, st);
}

}  // namespace lq
