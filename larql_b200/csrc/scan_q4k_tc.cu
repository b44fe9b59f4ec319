// Batched Q4_K gate scan on the fifth-generation tensor cores: tcgen05.mma kind::i8, accumulators in
// tensor memory.  Fast scores of every gate row for up to 32 tokens per launch (more tokens: more
// launches), with the |score| histogram and the rigorous bound on |fast - reference| that the exact
// top-K machinery needs (the same contract as the mma.sync scan in scan_q4k_mma.cu).
//
// scores[tok][row] = sum_k W[row][k] x[tok][k] is a contraction, but a Q4_K row carries a 6-bit scale and a
// 6-bit minimum per 32 weights and the activation a fixed-point step, so integer products of different
// sub-blocks cannot simply be added up.  The scales are folded into the integer operands:
//   * weights: w' = sc * q (sc the sub-block's scale, q the nibble), split as sc = 8 sh + sl into two byte
//     planes Ph = sh * q and Pl = sl * q (each <= 105, so one 32-bit multiply scales four packed nibbles),
//     expanded from the 144-byte super-blocks into shared memory;
//   * activation: 16-bit fixed point with ONE step per 256-element super-block and token,
//     x ~ step (256 a + b), a in s8, b in u8; and the eight block sums sum(x_j) of a super-block likewise,
//     sum(x_j) ~ step2 (256 a'_j + b'_j), as one more K slice whose weight bytes are the minima m_j
//     (prepared per token by prep_sb_planes_kernel).
// One super-block of one row and token is then
//     d step (2048 Ph.a + 8 Ph.b + 256 Pl.a + Pl.b) - dmin step2 (256 m.a' + m.b')
// with six exact s32 sums: 34 MMAs (8 sub-blocks x 4 plane pairs + 2, M = 128 rows, N = tokens, K = 32)
// and ONE epilogue per super-block (tcgen05.ld of the six values, a handful of multiply-adds).
// The integer dots are exact, so the bound is the fixed-point and rounding bound of the batch-1 scan with
// the super-block steps in place of the block step.  Reference arithmetic the scores approximate:
// q4k_matmul_into, crates/larql-compute/src/cpu/ops/q4_common/matmul.rs:20-139.
//
// A CTA owns 128 rows and walks the hidden dimension one super-block at a time, two stages deep:
//   warps 4-11  bring the raw super-blocks (cp.async, the next one in flight while this one is used) and the
//               tokens' operand tiles (L2 hits) in, and expand the nibbles into the two weight planes and the
//               minima, laid out as tcgen05 K-major operand tiles;
//   warp 12     waits for a stage, issues its 34 MMAs and commits them to an mbarrier;
//   warps 0-3   (one thread per row = one TMEM lane) read the accumulators back and keep the f32 scores of
//               their row for every token in registers.
// Every wait is bounded and reports through the error word; TMEM is freed on every path.
#include "../../include/larql_cuda.h"
#include "kernels.h"

namespace lq {

namespace {

constexpr int TC_ROWS = 128;                 // rows per CTA = TMEM lanes
constexpr int TC_EPI_WARPS = 4, TC_LOAD_WARPS = 8;
constexpr int TC_THREADS = (TC_EPI_WARPS + TC_LOAD_WARPS + 1) * 32;
constexpr int TC_LOADERS = TC_LOAD_WARPS * 32;
constexpr int TC_A_TILE = TC_ROWS * 32;      // one (plane, sub-block) weight tile
constexpr int TC_A_BYTES = 17 * TC_A_TILE;   // both planes of a super-block's 8 sub-blocks + the tile of the minima
constexpr int TC_RAW_BYTES = TC_ROWS * 144;  // one raw super-block of the CTA's rows
constexpr int TC_REC_FLOATS = 4;             // step, step2, U, V
constexpr int TC_HDR_RING = 4;               // row headers and token records live four super-blocks
constexpr int TC_TMEM_COLS = 512;            // two buffers of six accumulators x up to 32 tokens
constexpr int TC_SB_TILES = 18;              // token tiles per super-block: 2 planes x 8 sub-blocks + 2 of the sums

// Operand tiles are K-major, no swizzle: 8 rows x 16 bytes make one contiguous 128-byte core matrix; the two
// 16-byte K chunks of a row group sit 128 bytes apart (leading byte offset) and row groups 256 bytes apart
// (stride byte offset).
__host__ __device__ inline uint32_t tile_off(int row, int k) {
    return (uint32_t)(((row >> 3) * 2 + (k >> 4)) * 128 + (row & 7) * 16 + (k & 15));
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(256u >> 4) << 32) |
           (1ull << 46);
}
// kind::i8 instruction descriptor: s32 accumulators, unsigned A, B signed or unsigned, both K-major.
__host__ __device__ inline uint32_t instr_desc(int n, bool b_signed) {
    return (2u << 4) | (0u << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);
}

// Bounded spin on an mbarrier phase (about a second).  The handshakes of this kernel are a few hundred
// nanoseconds apart, so the waiters poll instead of parking.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((it & 1023u) == 0 && clock64() - t0 > (1ll << 31)) return false;
    }
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void named_bar(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Token tiles: with three slots the next super-block's tiles are requested before this one is expanded; 32
// tokens leave room for two, and the request follows the expansion.
__host__ __device__ constexpr int tc_b_ring(int nt) { return nt <= 16 ? 3 : 2; }

struct TcSmem {
    uint64_t full[2];       // stage filled and expanded (one arrival: a loader thread)
    uint64_t mma_done[2];   // the stage's MMAs have completed (tcgen05.commit)
    uint64_t tmem_free[2];  // the epilogue has read the accumulator buffer (128 arrivals)
    uint32_t tmem_base;
    int failed;
};

// Per token and super-block: the fixed-point planes as B operand tiles, the block sums as two more tiles,
// and the record {step, step2, U, V}: U = 63 (15 c1 sum|x| + 15 * 256 err step) and
// V = 63 (c1 sum|x| + 8 err step2) bound a row's |fast - reference| for this super-block by |d| U + |dmin| V
// (63: the largest 6-bit scale or minimum; err: LQ_XQ_ERR_STEPS of a step per fixed-point value).
// Tile t of super-block sb sits at (sb * 18 + t) * nt * 32: t = p * 8 + j for plane p of sub-block j, 16 + p
// for plane p of the block sums (bytes 0..7 of a row; the rest zero).
__global__ void __launch_bounds__(256) prep_sb_planes_kernel(TokenWs ws0, size_t ws_stride, int batch, int nt, int nsb,
                                                             float c1, uint8_t* __restrict__ btiles,
                                                             float* __restrict__ rec) {
    __shared__ float red[8], red2[8], red3[8];
    const int sb = blockIdx.x, tok = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float v = 0.0f;
    if (tok < batch) v = ws_at(ws0, ws_stride * tok).xn[sb * 256 + tid];
    float amax = fabsf(v);
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // warp w holds block w of the super-block (32 consecutive elements)
    float sum = v, asum = fabsf(v);
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        asum += __shfl_xor_sync(0xffffffffu, asum, o);
    }
    if (lane == 0) {
        red[warp] = amax;
        red2[warp] = sum;
        red3[warp] = asum;
    }
    __syncthreads();
    float am = 0.0f, as = 0.0f, sm2 = 0.0f;
    for (int w = 0; w < 8; ++w) {
        am = fmaxf(am, red[w]);
        as += red3[w];
        sm2 = fmaxf(sm2, fabsf(red2[w]));
    }
    const float inv = am > 0.0f ? 32767.0f / am : 0.0f, step = am / 32767.0f;
    const float inv2 = sm2 > 0.0f ? 32767.0f / sm2 : 0.0f, step2 = sm2 / 32767.0f;
    int q = __float2int_rn(v * inv);
    q = max(-32767, min(32767, q));
    const int j = tid >> 5, k = tid & 31;
    const size_t tile = (size_t)nt * 32, base = (size_t)sb * TC_SB_TILES * tile;
    btiles[base + (size_t)j * tile + tile_off(tok, k)] = (uint8_t)((q >> 8) & 0xff);
    btiles[base + (size_t)(8 + j) * tile + tile_off(tok, k)] = (uint8_t)(q & 0xff);
    if (tid < 32) {  // the two tiles of the block sums: byte k of the row is block k's sum, k < 8
        int q2 = 0;
        if (tid < 8) {
            q2 = __float2int_rn(red2[tid] * inv2);
            q2 = max(-32767, min(32767, q2));
        }
        btiles[base + (size_t)16 * tile + tile_off(tok, tid)] = (uint8_t)((q2 >> 8) & 0xff);
        btiles[base + (size_t)17 * tile + tile_off(tok, tid)] = (uint8_t)(q2 & 0xff);
    }
    if (tid < TC_REC_FLOATS) {
        float r = 0.0f;
        if (tid == 0) r = step;
        else if (tid == 1) r = step2;
        else if (tid == 2) r = 63.0f * (15.0f * c1 * as + 15.0f * 256.0f * LQ_XQ_ERR_STEPS * step);
        else r = 63.0f * (c1 * as + 8.0f * LQ_XQ_ERR_STEPS * step2);
        rec[((size_t)sb * nt + tok) * TC_REC_FLOATS + tid] = tok < batch ? r : 0.0f;
    }
}

template <int NT>
__global__ void __launch_bounds__(TC_THREADS, 1)
scan_q4k_tc_kernel(const uint8_t* __restrict__ W, int n_rows, int nsb, const uint8_t* __restrict__ btiles,
                   const float* __restrict__ rec, TokenWs ws0, size_t ws_stride, int batch, int want_hist, int* err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int B_BYTES = TC_SB_TILES * NT * 32;              // token tiles of one super-block
    constexpr int TC_B_RING = tc_b_ring(NT);
    constexpr int REC_BYTES = NT * TC_REC_FLOATS * 4;
    TcSmem& cs = *reinterpret_cast<TcSmem*>(smem);
    uint8_t* raw_ring = smem + 1024;                            // [2] raw super-blocks of the CTA's rows
    uint8_t* a_stage = raw_ring + 2 * TC_RAW_BYTES;             // [2] expanded weight planes of a super-block
    uint8_t* b_ring = a_stage + 2 * TC_A_BYTES;                 // [TC_B_RING] token tiles of a super-block
    uint8_t* hdr_ring = b_ring + TC_B_RING * B_BYTES;           // [TC_HDR_RING][128] d | dmin of the rows
    uint8_t* rec_ring = hdr_ring + TC_HDR_RING * TC_ROWS * 4;   // [TC_HDR_RING][NT] records
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_base = blockIdx.x * TC_ROWS;
    const size_t row_bytes = (size_t)nsb * 144;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&cs.full[i], 1);
            mbar_init(&cs.mma_done[i], 1);
            mbar_init(&cs.tmem_free[i], TC_EPI_WARPS * 32);
        }
        cs.failed = 0;
        fence_mbar_init();
    }
    if (warp == TC_EPI_WARPS + TC_LOAD_WARPS) {  // the MMA warp owns the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&cs.tmem_base)),
                     "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = cs.tmem_base;

    if (warp < TC_EPI_WARPS) {
        // ---- epilogue: thread = row = TMEM lane; once per super-block --------------------------------
        const int r = tid;  // 0..127
        const int row = row_base + r;
        float acc[NT], bnd[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = bnd[t] = 0.0f;
        bool failed = false;
        for (int s = 0; s < nsb; ++s) {
            const int tb = s & 1;
            if (!failed && !tc_wait(&cs.mma_done[tb], (uint32_t)(s >> 1) & 1u)) failed = true;
            if (failed) break;
            tc_fence_after();
            const uint32_t hdr = *reinterpret_cast<const uint32_t*>(hdr_ring + ((s % TC_HDR_RING) * TC_ROWS + r) * 4);
            const float4* rc = reinterpret_cast<const float4*>(rec_ring + (s % TC_HDR_RING) * REC_BYTES);
            const float d = f16_bits_to_f32(hdr), dmin = f16_bits_to_f32(hdr >> 16);
            const float ad = fabsf(d), adm = fabsf(dmin);
            const uint32_t tbase = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(tb * 6 * NT);
#pragma unroll
            for (int c = 0; c < NT / 16; ++c) {
                uint32_t xha[16], xhb[16], xla[16], xlb[16], y1[16], y0[16];
                tmem_ld16(tbase + c * 16, xha);
                tmem_ld16(tbase + NT + c * 16, xhb);
                tmem_ld16(tbase + 2 * NT + c * 16, xla);
                tmem_ld16(tbase + 3 * NT + c * 16, xlb);
                tmem_ld16(tbase + 4 * NT + c * 16, y1);
                tmem_ld16(tbase + 5 * NT + c * 16, y0);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int t = c * 16 + i;
                    const float4 q = rc[t];  // step, step2, U, V
                    const float main_i = fmaf((float)(int)xha[i], 2048.0f,
                                              fmaf((float)(int)xla[i], 256.0f, fmaf((float)(int)xhb[i], 8.0f, (float)(int)xlb[i])));
                    const float min_i = fmaf((float)(int)y1[i], 256.0f, (float)(int)y0[i]);
                    acc[t] += d * (q.x * main_i) - dmin * (q.y * min_i);
                    bnd[t] = fmaf(ad, q.z, fmaf(adm, q.w, bnd[t]));
                }
            }
            tc_fence_before();
            mbar_arrive(&cs.tmem_free[tb]);
        }
        if (failed) cs.failed = 1;
        // scores, histogram, largest bound of the warp's rows per token
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            float b = 0.0f;
            if (t < batch && row < n_rows && !failed) {
                const TokenWs w = ws_at(ws0, ws_stride * t);
                const float sc = acc[t];
                w.scores[row] = sc;
                if (want_hist) {
                    if (sc != sc) set_err(err, DEV_ERR_NAN_SCORE);
                    atomicAdd(&w.hist[__float_as_uint(fabsf(sc)) >> LQ_HIST_SHIFT], 1u);
                }
                b = bnd[t];
            }
            if (want_hist) {
                for (int o = 16; o > 0; o >>= 1) b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
                if (lane == 0 && t < batch && b > 0.0f)
                    atomicMax(&ws_at(ws0, ws_stride * t).sel->bound_bits, __float_as_uint(b));
            }
        }
    } else if (warp < TC_EPI_WARPS + TC_LOAD_WARPS) {
        // ---- loaders ----------------------------------------------------------------------------
        // cp.async groups are counted per thread and complete in order, so the two kinds of load are issued by
        // different threads: the first four warps only ever have raw super-blocks in flight (the next one is
        // requested before this one is expanded), the other four the token tiles of the next super-block.
        const int lt = tid - TC_EPI_WARPS * 32;  // 0..255
        bool failed = false;
        const bool raw_loader = lt < TC_LOADERS / 2;
        auto load_raw = [&](int s) {  // one commit group per super-block, empty past the end
            if (s < nsb) {
                uint8_t* raw = raw_ring + (size_t)(s & 1) * TC_RAW_BYTES;
                for (int i = lt; i < TC_ROWS * 9; i += TC_LOADERS / 2) {
                    const int r = i / 9, ch = i - r * 9;
                    const int row = min(row_base + r, n_rows - 1);
                    cp16(raw + r * 144 + ch * 16, W + (size_t)row * row_bytes + (size_t)s * 144 + ch * 16);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto load_tok = [&](int s) {  // token tiles and records of super-block s
            if (s < nsb) {
                const int l2 = lt - TC_LOADERS / 2;
                uint8_t* b_pl = b_ring + (size_t)(s % TC_B_RING) * B_BYTES;
                const uint8_t* src = btiles + (size_t)s * B_BYTES;
                for (int i = l2; i < B_BYTES / 16; i += TC_LOADERS / 2) cp16(b_pl + i * 16, src + (size_t)i * 16);
                for (int i = l2; i < REC_BYTES / 16; i += TC_LOADERS / 2)
                    cp16(rec_ring + (s % TC_HDR_RING) * REC_BYTES + i * 16,
                         reinterpret_cast<const uint8_t*>(rec) + (size_t)s * REC_BYTES + i * 16);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (raw_loader) load_raw(0);
        else load_tok(0);
        for (int s = 0; s < nsb; ++s) {
            const int st = s & 1;
            if (raw_loader) {
                load_raw(s + 1);  // the other raw slot held super-block s - 1, which this group has finished expanding
                asm volatile("cp.async.wait_group 1;" ::: "memory");  // super-block s has landed
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");  // the tiles of super-block s have landed
            }
            // the MMAs of super-block s - 2 read the weight planes of stage st, which the expansion overwrites
            if (s >= 2 && !failed && !tc_wait(&cs.mma_done[st], (uint32_t)((s - 2) >> 1) & 1u)) failed = true;
            if (failed) break;
            if (TC_B_RING == 3 && !raw_loader) load_tok(s + 1);  // its slot held the tiles of s - 2
            named_bar(1, TC_LOADERS);
            const uint8_t* raw = raw_ring + (size_t)st * TC_RAW_BYTES;
            uint8_t* a_pl = a_stage + (size_t)st * TC_A_BYTES;
            // unit = (row, pair g): 32 bytes of nibbles -> sub-blocks 2g (low nibbles) and 2g + 1 (high); a
            // quarter-warp (8 consecutive rows) stores one whole 128-byte core matrix at a time
            for (int u = lt; u < TC_ROWS * 4; u += TC_LOADERS) {
                const int r = u & (TC_ROWS - 1), g = u >> 7;
                const uint8_t* cell = raw + r * 144;
                const uint4 hdr = *reinterpret_cast<const uint4*>(cell);
                uint32_t sc2, m2;
                q4k_pair_scales(hdr.y, hdr.z, hdr.w, g, sc2, m2);
                if (g == 0) {
                    // d | dmin for the epilogue, and the tile of the row's eight minima (bytes 0..7 of the K slice)
                    *reinterpret_cast<uint32_t*>(hdr_ring + ((s % TC_HDR_RING) * TC_ROWS + r) * 4) = hdr.x;
                    uint32_t mw0 = m2 & 0xffffu, mw1, scx, mx;
                    q4k_pair_scales(hdr.y, hdr.z, hdr.w, 1, scx, mx);
                    mw0 |= (mx & 0xffffu) << 16;
                    q4k_pair_scales(hdr.y, hdr.z, hdr.w, 2, scx, mx);
                    mw1 = mx & 0xffffu;
                    q4k_pair_scales(hdr.y, hdr.z, hdr.w, 3, scx, mx);
                    mw1 |= (mx & 0xffffu) << 16;
                    uint8_t* t_m = a_pl + (size_t)16 * TC_A_TILE;
                    *reinterpret_cast<uint4*>(t_m + tile_off(r, 0)) = make_uint4(mw0, mw1, 0u, 0u);
                    *reinterpret_cast<uint4*>(t_m + tile_off(r, 16)) = make_uint4(0u, 0u, 0u, 0u);
                }
                const uint4 qa = *reinterpret_cast<const uint4*>(cell + 16 + g * 32);
                const uint4 qb = *reinterpret_cast<const uint4*>(cell + 32 + g * 32);
                const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                for (int hn = 0; hn < 2; ++hn) {
                    const int j = 2 * g + hn;
                    const uint32_t sc = hn ? (sc2 >> 8) : (sc2 & 0xff);
                    const uint32_t sh = sc >> 3, sl = sc & 7u;  // sc = 8 sh + sl: sh q, sl q <= 105 stay inside their bytes
                    uint32_t lo_w[8], hi_w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t nib = (hn ? (qw[i] >> 4) : qw[i]) & 0x0F0F0F0Fu;
                        hi_w[i] = nib * sh;
                        lo_w[i] = nib * sl;
                    }
                    uint8_t* t_hi = a_pl + (size_t)j * TC_A_TILE;
                    uint8_t* t_lo = a_pl + (size_t)(8 + j) * TC_A_TILE;
#pragma unroll
                    for (int kc = 0; kc < 2; ++kc) {
                        *reinterpret_cast<uint4*>(t_hi + tile_off(r, kc * 16)) =
                            make_uint4(hi_w[4 * kc], hi_w[4 * kc + 1], hi_w[4 * kc + 2], hi_w[4 * kc + 3]);
                        *reinterpret_cast<uint4*>(t_lo + tile_off(r, kc * 16)) =
                            make_uint4(lo_w[4 * kc], lo_w[4 * kc + 1], lo_w[4 * kc + 2], lo_w[4 * kc + 3]);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // plain stores -> the tensor core's reads
            named_bar(1, TC_LOADERS);
            if (lt == 0) mbar_arrive(&cs.full[st]);
            // the token tiles of super-block s + 1 go where those of s - 1 were: the MMAs that read them were
            // issued a whole super-block ago
            if (TC_B_RING == 2 && !raw_loader) {
                if (s >= 1 && !failed && !tc_wait(&cs.mma_done[st ^ 1], (uint32_t)((s - 1) >> 1) & 1u)) failed = true;
                if (failed) break;
                load_tok(s + 1);
            }
        }
        if (failed) cs.failed = 1;
    } else {
        // ---- MMA warp ---------------------------------------------------------------------------
        bool failed = false;
        const uint32_t idesc_s = instr_desc(NT, true), idesc_u = instr_desc(NT, false);
        for (int s = 0; s < nsb; ++s) {
            const int st = s & 1;
            if (!failed && !tc_wait(&cs.full[st], (uint32_t)(s >> 1) & 1u)) failed = true;
            if (s >= 2 && !failed && !tc_wait(&cs.tmem_free[st], (uint32_t)((s - 2) >> 1) & 1u)) failed = true;
            if (failed) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_addr = smem_u32(a_stage + (size_t)st * TC_A_BYTES);
                const uint32_t b_addr = smem_u32(b_ring + (size_t)(s % TC_B_RING) * B_BYTES);
                const uint32_t dha = tmem + (uint32_t)(st * 6 * NT), dhb = dha + NT, dla = dha + 2 * NT, dlb = dha + 3 * NT;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint64_t ph = smem_desc(a_addr + j * TC_A_TILE);
                    const uint64_t pl = smem_desc(a_addr + (8 + j) * TC_A_TILE);
                    const uint64_t xa = smem_desc(b_addr + j * NT * 32);
                    const uint64_t xb = smem_desc(b_addr + (8 + j) * NT * 32);
                    const uint32_t acc = j > 0 ? 1u : 0u;  // the super-block's first MMA overwrites
                    umma_i8(dha, ph, xa, idesc_s, acc);
                    umma_i8(dhb, ph, xb, idesc_u, acc);
                    umma_i8(dla, pl, xa, idesc_s, acc);
                    umma_i8(dlb, pl, xb, idesc_u, acc);
                }
                // minima x block sums
                const uint64_t mt = smem_desc(a_addr + 16 * TC_A_TILE);
                umma_i8(dha + 4 * NT, mt, smem_desc(b_addr + 16 * NT * 32), idesc_s, 0u);
                umma_i8(dha + 5 * NT, mt, smem_desc(b_addr + 17 * NT * 32), idesc_u, 0u);
                umma_commit(&cs.mma_done[st]);
            }
            __syncwarp();
        }
        if (failed) cs.failed = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_EPI_WARPS + TC_LOAD_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
    }
    if (tid == 0 && cs.failed) set_err(err, DEV_ERR_TMA_TIMEOUT);
}

template <int NT>
size_t tc_smem_bytes() {
    return 1024 + (size_t)2 * TC_RAW_BYTES + (size_t)2 * TC_A_BYTES + (size_t)tc_b_ring(NT) * TC_SB_TILES * NT * 32 +
           (size_t)TC_HDR_RING * TC_ROWS * 4 + (size_t)TC_HDR_RING * NT * TC_REC_FLOATS * 4;
}

}  // namespace

size_t scan_q4k_tc_scratch_bytes(int cols) {
    const size_t nsb = (size_t)cols / 256;
    return nsb * TC_SB_TILES * 32 * 32 + nsb * 32 * TC_REC_FLOATS * 4 + 1024;
}

// scratch: scan_q4k_tc_scratch_bytes(cols) of device memory, 256-byte aligned.  batch <= 32.
cudaError_t launch_scan_q4k_tc(const Q4kMat& m, TokenWs ws0, size_t ws_stride, int batch, int want_hist, float c1,
                               uint8_t* scratch, int* err, cudaStream_t st) {
    if (m.cols <= 0 || m.cols % 256 != 0 || batch < 1 || batch > 32) return cudaErrorInvalidValue;
    if (m.rows == 0) return cudaSuccess;
    const int nsb = m.cols / 256, nt = batch <= 16 ? 16 : 32;
    uint8_t* btiles = scratch;
    float* rec = reinterpret_cast<float*>(scratch + (((size_t)nsb * TC_SB_TILES * nt * 32 + 255) / 256 * 256));
    prep_sb_planes_kernel<<<dim3(nsb, nt), 256, 0, st>>>(ws0, ws_stride, batch, nt, nsb, c1, btiles, rec);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int grid = (m.rows + TC_ROWS - 1) / TC_ROWS;
    if (nt == 16) {
        if ((e = set_max_dyn_smem((const void*)scan_q4k_tc_kernel<16>, 227 * 1024)) != cudaSuccess) return e;
        scan_q4k_tc_kernel<16><<<grid, TC_THREADS, tc_smem_bytes<16>(), st>>>(m.w, m.rows, nsb, btiles, rec, ws0, ws_stride,
                                                                              batch, want_hist, err);
    } else {
        if ((e = set_max_dyn_smem((const void*)scan_q4k_tc_kernel<32>, 227 * 1024)) != cudaSuccess) return e;
        scan_q4k_tc_kernel<32><<<grid, TC_THREADS, tc_smem_bytes<32>(), st>>>(m.w, m.rows, nsb, btiles, rec, ws0, ws_stride,
                                                                              batch, want_hist, err);
    }
    return cudaGetLastError();
}

}  // namespace lq
