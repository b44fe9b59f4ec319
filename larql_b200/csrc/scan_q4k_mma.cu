// Batched Q4_K gate scan on the tensor cores: fast scores of every gate row for up to 64 tokens
// per launch.
//
// At batch >= 2 the scan is a contraction: scores[token][row] = sum_k W[row][k] x[token][k].  The
// 4-bit weights and the tokens' 16-bit fixed-point activation planes (x ~ step (256 a + b), a in
// s8, b in u8 per 32-element block; the same planes the batch-1 scan uses) are multiplied with
// integer MMAs, one 32-element sub-block per instruction, so the integer dots are exact; the
// sub-block scale d*sc, the block step and the -dmin*m*sum(x) term of the sum_x form
// (crates/larql-compute/src/cpu/ops/q4_common/matvec_f32.rs:107-164, the reference batch-1 row;
// the batched reference, q4k_matmul_into in .../q4_common/matmul.rs:20-139, associates
// differently and is covered by the same bound) are applied in f32 in the epilogue of each MMA.
// Every token gets what the batch-1 scan leaves: scores, the coarse |score| histogram and a
// rigorous bound on |fast - reference|, so the exact top-K machinery that follows is shared.
//
// Layout of the work: a CTA owns 64 rows (four m16 blocks) and walks the hidden dimension one
// 256-element super-block at a time, double-buffered with cp.async: 64 x 144 B of weights and,
// per token, the two 256-byte planes plus the blocks' step / sum / |sum|.  Warp w takes m16 block
// (w & 3) and the 8-token groups congruent to (w >> 2) mod 2.
#include "../../include/larql_cuda.h"
#include "kernels.h"

namespace lq {

namespace {

constexpr int MS_THREADS = 256;
constexpr int MS_ROWS = 64;           // rows per CTA
constexpr int MS_MAX_TOK = 64;        // tokens per launch
constexpr int MS_TOK_WORDS = 132;     // two 64-word planes + 4 words of padding (bank spread)
constexpr int MS_REC_FLOATS = 32;     // step[8], sum[8], abs[8], U, V, padding
constexpr int MS_TOK_BYTES = MS_TOK_WORDS * 4 + MS_REC_FLOATS * 4;
constexpr int MS_W_BYTES = MS_ROWS * 144;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8u8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NTG: 8-token groups per warp (1, 2 or 4): batch <= 16, 32, 64.
template <int NTG>
__global__ void __launch_bounds__(MS_THREADS, 1)
scan_q4k_mma_kernel(const uint8_t* __restrict__ W, int n_rows, int nsb, TokenWs ws0, size_t ws_stride, int batch,
                    int want_hist, float c1, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int mb = warp & 3, tgp = warp >> 2;  // m16 block, token-group parity
    const int row_bytes = nsb * 144;
    const int row_base = blockIdx.x * MS_ROWS;
    const int tok_pad = NTG * 16;  // tokens staged (multiple of 8 groups x 2 parities)
    const int stage_bytes = MS_W_BYTES + tok_pad * MS_TOK_BYTES;
    const float qe = 15.0f * 32.0f * LQ_XQ_ERR_STEPS;

    auto stage_w = [&](int st) -> uint8_t* { return smem + (size_t)st * stage_bytes; };
    auto stage_tok = [&](int st, int tok) -> uint8_t* {
        return smem + (size_t)st * stage_bytes + MS_W_BYTES + (size_t)tok * MS_TOK_BYTES;
    };
    // zero the planes of padding tokens once (both stages): their MMAs run but nothing is written
    for (int st = 0; st < 2; ++st)
        for (int tok = batch; tok < tok_pad; ++tok)
            for (int i = tid; i < MS_TOK_BYTES / 4; i += MS_THREADS) reinterpret_cast<uint32_t*>(stage_tok(st, tok))[i] = 0u;

    auto load_stage = [&](int st, int s) {
        // weights: 64 rows x 9 chunks of 16 B
        for (int i = tid; i < MS_ROWS * 9; i += MS_THREADS) {
            const int r = i / 9, ch = i % 9;
            const int row = min(row_base + r, n_rows - 1);
            cp_async16(stage_w(st) + r * 144 + ch * 16, W + (size_t)row * row_bytes + (size_t)s * 144 + ch * 16);
        }
        // tokens: planes a and b (16 chunks each), step / sum / abs (2 chunks each)
        for (int i = tid; i < batch * 38; i += MS_THREADS) {
            const int tok = i / 38, ch = i % 38;
            const TokenWs w = ws_at(ws0, ws_stride * tok);
            uint8_t* dst = stage_tok(st, tok);
            if (ch < 16) cp_async16(dst + ch * 16, reinterpret_cast<const uint8_t*>(w.xa + s * 64) + ch * 16);
            else if (ch < 32) cp_async16(dst + 256 + (ch - 16) * 16, reinterpret_cast<const uint8_t*>(w.xb + s * 64) + (ch - 16) * 16);
            else {
                const int k = (ch - 32) >> 1, h = (ch - 32) & 1;
                const float* src = (k == 0 ? w.bscale : (k == 1 ? w.bsum : w.babs)) + s * 8 + h * 4;
                cp_async16(dst + MS_TOK_WORDS * 4 + k * 32 + h * 16, src);
            }
        }
        cp_async_commit();
    };

    float acc[NTG][4], bnd[NTG][4];
#pragma unroll
    for (int i = 0; i < NTG; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = bnd[i][j] = 0.0f;

    load_stage(0, 0);
    for (int s = 0; s < nsb; ++s) {
        const int st = s & 1;
        if (s + 1 < nsb) {
            load_stage(st ^ 1, s + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // per token: U = 63 sum_sb (c1 15 |x|_sb + qe step_sb), V = 63 c1 sum_sb |x|_sb  (bound terms)
        if (tid < batch) {
            float* rec = reinterpret_cast<float*>(stage_tok(st, tid) + MS_TOK_WORDS * 4);
            float u = 0.0f, v = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                u += c1 * 15.0f * rec[16 + j] + qe * rec[j];
                v += rec[16 + j];
            }
            rec[24] = 63.0f * u;
            rec[25] = 63.0f * c1 * v;
        }
        __syncthreads();

        const uint8_t* wr0 = stage_w(st) + (mb * 16 + g) * 144;
        const uint8_t* wr1 = wr0 + 8 * 144;
        const uint4 h0 = *reinterpret_cast<const uint4*>(wr0);
        const uint4 h1 = *reinterpret_cast<const uint4*>(wr1);
        const float d0 = f16_bits_to_f32(h0.x), dm0 = f16_bits_to_f32(h0.x >> 16);
        const float d1 = f16_bits_to_f32(h1.x), dm1 = f16_bits_to_f32(h1.x >> 16);
        // bound terms of this super-block
#pragma unroll
        for (int i = 0; i < NTG; ++i) {
            const int tok0 = (tgp + 2 * i) * 8 + 2 * t;
            const float* r0 = reinterpret_cast<const float*>(stage_tok(st, tok0) + MS_TOK_WORDS * 4);
            const float* r1 = reinterpret_cast<const float*>(stage_tok(st, tok0 + 1) + MS_TOK_WORDS * 4);
            bnd[i][0] += fabsf(d0) * r0[24] + fabsf(dm0) * r0[25];
            bnd[i][1] += fabsf(d0) * r1[24] + fabsf(dm0) * r1[25];
            bnd[i][2] += fabsf(d1) * r0[24] + fabsf(dm1) * r0[25];
            bnd[i][3] += fabsf(d1) * r1[24] + fabsf(dm1) * r1[25];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // cell q: sub-blocks 2q (low nibbles) and 2q+1 (high nibbles)
            const uint32_t w00 = *reinterpret_cast<const uint32_t*>(wr0 + 16 + q * 32 + 4 * t);
            const uint32_t w01 = *reinterpret_cast<const uint32_t*>(wr0 + 16 + q * 32 + 16 + 4 * t);
            const uint32_t w10 = *reinterpret_cast<const uint32_t*>(wr1 + 16 + q * 32 + 4 * t);
            const uint32_t w11 = *reinterpret_cast<const uint32_t*>(wr1 + 16 + q * 32 + 16 + 4 * t);
            uint32_t sc2a, m2a, sc2b, m2b;
            q4k_pair_scales(h0.y, h0.z, h0.w, q, sc2a, m2a);
            q4k_pair_scales(h1.y, h1.z, h1.w, q, sc2b, m2b);
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                const int j = 2 * q + hi;
                uint32_t a[4];
                if (hi == 0) {
                    a[0] = w00 & 0x0F0F0F0Fu; a[1] = w10 & 0x0F0F0F0Fu; a[2] = w01 & 0x0F0F0F0Fu; a[3] = w11 & 0x0F0F0F0Fu;
                } else {
                    a[0] = (w00 >> 4) & 0x0F0F0F0Fu; a[1] = (w10 >> 4) & 0x0F0F0F0Fu;
                    a[2] = (w01 >> 4) & 0x0F0F0F0Fu; a[3] = (w11 >> 4) & 0x0F0F0F0Fu;
                }
                const float dsc0 = d0 * (float)((sc2a >> (8 * hi)) & 0xff), dmm0 = dm0 * (float)((m2a >> (8 * hi)) & 0xff);
                const float dsc1 = d1 * (float)((sc2b >> (8 * hi)) & 0xff), dmm1 = dm1 * (float)((m2b >> (8 * hi)) & 0xff);
#pragma unroll
                for (int i = 0; i < NTG; ++i) {
                    const int tg = tgp + 2 * i;
                    const uint32_t* pl = reinterpret_cast<const uint32_t*>(stage_tok(st, tg * 8 + g));
                    const uint32_t ba0 = pl[j * 8 + t], ba1 = pl[j * 8 + 4 + t];
                    const uint32_t bb0 = pl[64 + j * 8 + t], bb1 = pl[64 + j * 8 + 4 + t];
                    int ca[4] = {0, 0, 0, 0}, cb[4] = {0, 0, 0, 0};
                    mma_u8s8(ca, a, ba0, ba1);
                    mma_u8u8(cb, a, bb0, bb1);
                    const int tok0 = tg * 8 + 2 * t;
                    const float* r0 = reinterpret_cast<const float*>(stage_tok(st, tok0) + MS_TOK_WORDS * 4);
                    const float* r1 = reinterpret_cast<const float*>(stage_tok(st, tok0 + 1) + MS_TOK_WORDS * 4);
                    const float st0 = r0[j], su0 = r0[8 + j], st1 = r1[j], su1 = r1[8 + j];
                    const float v00 = st0 * (float)(ca[0] * 256 + cb[0]), v01 = st1 * (float)(ca[1] * 256 + cb[1]);
                    const float v10 = st0 * (float)(ca[2] * 256 + cb[2]), v11 = st1 * (float)(ca[3] * 256 + cb[3]);
                    acc[i][0] += dsc0 * v00 - dmm0 * su0;
                    acc[i][1] += dsc0 * v01 - dmm0 * su1;
                    acc[i][2] += dsc1 * v10 - dmm1 * su0;
                    acc[i][3] += dsc1 * v11 - dmm1 * su1;
                }
            }
        }
        __syncthreads();  // every warp is done with stage st before it is refilled
    }

    // scores, histogram, bound
#pragma unroll
    for (int i = 0; i < NTG; ++i) {
        const int tok0 = (tgp + 2 * i) * 8 + 2 * t;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int tok = tok0 + (e & 1), row = row_base + mb * 16 + g + 8 * (e >> 1);
            float b = bnd[i][e];
            if (tok >= batch || row >= n_rows) b = 0.0f;
            else {
                const TokenWs w = ws_at(ws0, ws_stride * tok);
                const float sc = acc[i][e];
                w.scores[row] = sc;
                if (want_hist) {
                    if (sc != sc) set_err(err, DEV_ERR_NAN_SCORE);
                    atomicAdd(&w.hist[__float_as_uint(fabsf(sc)) >> LQ_HIST_SHIFT], 1u);
                }
            }
            bnd[i][e] = b;
        }
        if (want_hist) {
            // largest bound over this warp's 16 rows, per token
            float b0 = fmaxf(bnd[i][0], bnd[i][2]), b1 = fmaxf(bnd[i][1], bnd[i][3]);
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                b0 = fmaxf(b0, __shfl_xor_sync(0xffffffffu, b0, o));
                b1 = fmaxf(b1, __shfl_xor_sync(0xffffffffu, b1, o));
            }
            if (g == 0) {
                if (tok0 < batch && b0 > 0.0f) atomicMax(&ws_at(ws0, ws_stride * tok0).sel->bound_bits, __float_as_uint(b0));
                if (tok0 + 1 < batch && b1 > 0.0f)
                    atomicMax(&ws_at(ws0, ws_stride * (tok0 + 1)).sel->bound_bits, __float_as_uint(b1));
            }
        }
    }
}

}  // namespace

cudaError_t launch_scan_q4k_mma(const Q4kMat& m, TokenWs ws0, size_t ws_stride, int batch, int want_hist, float c1,
                                int* err, int sm_count, cudaStream_t st) {
    (void)sm_count;
    if (m.cols <= 0 || m.cols % 256 != 0 || batch < 1 || batch > MS_MAX_TOK) return cudaErrorInvalidValue;
    if (m.rows == 0) return cudaSuccess;
    const int nsb = m.cols / 256;
    const int grid = (m.rows + MS_ROWS - 1) / MS_ROWS;
    const int ntg = batch <= 16 ? 1 : (batch <= 32 ? 2 : 4);
    const size_t smem = (size_t)2 * (MS_W_BYTES + (size_t)ntg * 16 * MS_TOK_BYTES);
    {
        cudaError_t e;
        if ((e = set_max_dyn_smem((const void*)scan_q4k_mma_kernel<1>, 200 * 1024)) ||
            (e = set_max_dyn_smem((const void*)scan_q4k_mma_kernel<2>, 200 * 1024)) ||
            (e = set_max_dyn_smem((const void*)scan_q4k_mma_kernel<4>, 200 * 1024)))
            return e;
    }
    if (ntg == 1)
        scan_q4k_mma_kernel<1><<<grid, MS_THREADS, smem, st>>>(m.w, m.rows, nsb, ws0, ws_stride, batch, want_hist, c1, err);
    else if (ntg == 2)
        scan_q4k_mma_kernel<2><<<grid, MS_THREADS, smem, st>>>(m.w, m.rows, nsb, ws0, ws_stride, batch, want_hist, c1, err);
    else
        scan_q4k_mma_kernel<4><<<grid, MS_THREADS, smem, st>>>(m.w, m.rows, nsb, ws0, ws_stride, batch, want_hist, c1, err);
    return cudaGetLastError();
}

}  // namespace lq
