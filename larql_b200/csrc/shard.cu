// Feature-sharded walk across the GPUs of one box: device-side pieces between the collectives.
//
// Every rank holds a contiguous range of feature rows of gate / up / down.  Per layer:
//   1. local scan -> local scores, local coarse histogram, local error bound;
//      all-reduce(sum) of [histogram | one bound slot per rank]            (collective 1)
//   2. every rank derives the SAME band thresholds from the global histogram, classifies its
//      rows, re-scores its band rows exactly, packs {n_in, n_band, rows, exact scores};
//      all-gather of the packs                                              (collective 2)
//   3. every rank runs the SAME final pick over all band rows (|score| desc, global row asc),
//      gathers the rows it owns (certain + its winners) into a partial out[H];
//      all-reduce(sum) of out[H]                                            (collective 3)
// The selected set is the unsharded reference's bit for bit (same proof as the single-GPU
// classification: the histogram and the bound are global).  The reference has no feature
// sharding (it shards layers / experts over HTTP, docs/ffn/distributed.md:14-40).
#include "select.cuh"

namespace lq {

namespace {

// bound slots after the histogram: slot r holds rank r's bound bits (others zero before the
// all-reduce), so a SUM all-reduce carries a MAX.
__global__ void shard_bound_max_kernel(const uint32_t* slots, int world, uint32_t* bound_bits) {
    if (threadIdx.x == 0) {
        uint32_t m = 0;
        for (int r = 0; r < world; ++r) m = max(m, slots[r]);
        *bound_bits = m;
    }
}

__global__ void shard_pack_kernel(TokenWs ws, uint32_t row_offset, int cap, int32_t* pack, int* err) {
    const int n_in = ws.sel->n_in;
    int n_band = ws.sel->n_band;
    const bool overflow = n_band > cap;
    if (overflow) {
        // more band rows than a pack holds: published as n_band = -1, so that every rank sees it after
        // the all-gather and fails the token (a truncated band would give a silently wrong top-K)
        if (threadIdx.x == 0 && blockIdx.x == 0) set_err(err, DEV_ERR_INTERNAL);
        n_band = 0;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        pack[0] = n_in;
        pack[1] = overflow ? -1 : n_band;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_band; i += gridDim.x * blockDim.x) {
        pack[2 + i] = (int32_t)(ws.band_idx[i] + row_offset);
        pack[2 + cap + i] = __float_as_int(ws.band_exact[i]);
        if (ws.band_exact[i] != ws.band_exact[i]) set_err(err, DEV_ERR_NAN_SCORE);
    }
}

constexpr int PICK_T = 512;
constexpr int MAX_WORLD = 16;

// Final pick over the gathered packs; appends this rank's winners to its hit list.
__global__ void __launch_bounds__(PICK_T) shard_pick_kernel(const int32_t* __restrict__ packs, int world, int rank,
                                                           int cap, int top_k, uint32_t row_offset, TokenWs ws,
                                                           int* err) {
    __shared__ SelectSmem<PICK_T> sm;
    __shared__ int s_off[MAX_WORLD + 1];
    __shared__ int s_nin;
    const int stride = 2 + 2 * cap;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        int off = 0, nin = 0;
        for (int r = 0; r < world; ++r) {
            s_off[r] = off;
            const int nb = packs[(size_t)r * stride + 1];
            if (nb < 0) set_err(err, DEV_ERR_INTERNAL);  // that rank's band did not fit its pack
            off += max(0, min(nb, cap));
            nin += packs[(size_t)r * stride];
        }
        s_off[world] = off;
        s_nin = nin;
    }
    __syncthreads();
    const int total = s_off[world], need = top_k - s_nin;
    const int n_in_local = ws.sel->n_in;
    const int n_band_local = min(ws.sel->n_band, cap);
    auto seg = [&](int i, int& r, int& j) {
        r = 0;
        while (r + 1 < world && i >= s_off[r + 1]) ++r;
        j = i - s_off[r];
    };
    auto keyf = [&](int i) -> uint32_t {
        int r, j;
        seg(i, r, j);
        return abs_key(__int_as_float(packs[(size_t)r * stride + 2 + cap + j]));
    };
    uint32_t tau_key = 0, row_cut = 0xffffffffu;
    const bool take_all = need >= total;
    if (!take_all && need > 0) {
        int cnt_gt, need_eq;
        block_kth_largest_keys<PICK_T, 0>(keyf, total, need, sm, tau_key, cnt_gt, need_eq);
        auto rowf = [&](int i) -> uint32_t {
            int r, j;
            seg(i, r, j);
            if (abs_key(__int_as_float(packs[(size_t)r * stride + 2 + cap + j])) != tau_key) return 0u;
            return ~(uint32_t)packs[(size_t)r * stride + 2 + j];
        };
        uint32_t cut_key;
        int c2, n2;
        block_kth_largest_keys<PICK_T, 0>(rowf, total, need_eq, sm, cut_key, c2, n2);
        row_cut = ~cut_key;
        __syncthreads();
    }
    if (warp == 0) {
        const int32_t* mine = packs + (size_t)rank * stride;
        int cnt = 0;
        for (int i0 = 0; i0 < n_band_local; i0 += 32) {
            const int i = i0 + lane;
            bool win = false;
            uint32_t row = 0;
            float v = 0.0f;
            if (i < n_band_local && need > 0) {
                row = (uint32_t)mine[2 + i];
                v = __int_as_float(mine[2 + cap + i]);
                const uint32_t key = abs_key(v);
                win = take_all || key > tau_key || (key == tau_key && row <= row_cut);
            }
            const uint32_t bal = __ballot_sync(0xffffffffu, win);
            if (win) {
                const int pos = n_in_local + cnt + __popc(bal & ((1u << lane) - 1u));
                ws.hit_idx[pos] = row - row_offset;
                ws.hit_score[pos] = v;
            }
            cnt += __popc(bal);
        }
        if (lane == 0) {
            ws.sel->n_sel = n_in_local + cnt;
            ws.sel->need = need;
        }
    }
    (void)err;
}

}  // namespace

cudaError_t launch_shard_bound_max(const uint32_t* slots, int world, uint32_t* bound_bits, cudaStream_t st) {
    shard_bound_max_kernel<<<1, 32, 0, st>>>(slots, world, bound_bits);
    return cudaGetLastError();
}

cudaError_t launch_shard_pack(TokenWs ws, uint32_t row_offset, int cap, int32_t* pack, int* err, cudaStream_t st) {
    shard_pack_kernel<<<8, 256, 0, st>>>(ws, row_offset, cap, pack, err);
    return cudaGetLastError();
}

cudaError_t launch_shard_pick(const int32_t* packs, int world, int rank, int cap, int top_k, uint32_t row_offset,
                              TokenWs ws, int* err, cudaStream_t st) {
    if (world > MAX_WORLD) return cudaErrorInvalidValue;
    shard_pick_kernel<<<1, PICK_T, 0, st>>>(packs, world, rank, cap, top_k, row_offset, ws, err);
    return cudaGetLastError();
}

}  // namespace lq
