// Exact top-K by |score| inside one CTA: an 8-bit MSB radix select on the f32
// magnitude bits (non-NaN |v| bit patterns order like unsigned integers), then an
// index-ordered compaction.  Ties at the threshold are resolved towards the lower
// index, which realises the total order (|v| descending, index ascending) of the
// reference's top_k_by_abs
// (crates/larql-vindex/src/index/compute/gate_knn/mod.rs:50-108).
#pragma once
#include "kernels.h"

namespace lq {

// Shared scratch for one CTA of T threads.
template <int T>
struct SelectSmem {
    uint32_t whist[T / 32][256];
    uint32_t total[256];
    int wcnt_a[T / 32];
    int wcnt_b[T / 32];
    int bcast[4];
    float fbcast[2];
};

__device__ __forceinline__ uint32_t abs_key(float v) { return __float_as_uint(fabsf(v)); }

// Each warp owns a contiguous, 32-aligned chunk of [0, n); within it lanes stride.
// Returns chunk size; warp w covers [w*chunk, min(n, (w+1)*chunk)).
__device__ __forceinline__ int warp_chunk(int n, int n_warps) {
    const int per = (n + n_warps - 1) / n_warps;
    return (per + 31) / 32 * 32;
}

// Finds the k-th largest key among vals[0..n) (1 <= k <= n).  Outputs the key, how
// many keys are strictly greater, and how many of the equal ones are still needed.
// The radix passes start at the highest bit in which the keys differ (found with a
// min/max reduction), so keys that share their leading bits - scores of similar
// magnitude, or a narrow band of near-ties - spread over the 256 bins of the first
// pass instead of colliding in one.
// `keyf(i)` returns the 32-bit key of element i; the CTA's first T threads take part
// (threadIdx.x < T), synchronising on named barrier `bar` (0 = the whole CTA).
template <int T, int BAR = 0, typename KeyFn>
__device__ void block_kth_largest_keys(KeyFn keyf, int n, int k, SelectSmem<T>& sm, uint32_t& tau_key, int& cnt_gt,
                                       int& need_eq) {
    auto bsync = [] {
        if (BAR == 0) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(T) : "memory");
    };
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = warp_chunk(n, T / 32);
    const int beg = warp * chunk, end = min(n, beg + chunk);
    // key range
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    for (int i = beg + lane; i < end; i += 32) {
        const uint32_t key = keyf(i);
        kmin = min(kmin, key);
        kmax = max(kmax, key);
    }
    for (int o = 16; o > 0; o >>= 1) {
        kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
        kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    }
    if (lane == 0) {
        sm.wcnt_a[warp] = (int)kmin;
        sm.wcnt_b[warp] = (int)kmax;
    }
    bsync();
    kmin = 0xffffffffu;
    kmax = 0u;
    for (int w = 0; w < T / 32; ++w) {
        kmin = min(kmin, (uint32_t)sm.wcnt_a[w]);
        kmax = max(kmax, (uint32_t)sm.wcnt_b[w]);
    }
    bsync();
    if (kmin == kmax) {  // every key equal
        tau_key = kmin;
        cnt_gt = 0;
        need_eq = k;
        return;
    }
    int hi_bit = 32 - __clz(kmin ^ kmax);  // bits [hi_bit, 32) are common to all keys
    uint32_t prefix = hi_bit < 32 ? (kmax >> hi_bit) << hi_bit : 0u;
    int remaining = k;
    while (hi_bit > 0) {
        const int lo_bit = max(hi_bit - 8, 0);
        const uint32_t dmask = (1u << (hi_bit - lo_bit)) - 1u;
        for (int i = tid; i < (T / 32) * 256; i += T) (&sm.whist[0][0])[i] = 0;
        bsync();
        for (int i = beg + lane; i < end; i += 32) {
            const uint32_t key = keyf(i);
            const bool match = hi_bit >= 32 ? true : ((key >> hi_bit) == (prefix >> hi_bit));
            if (match) atomicAdd(&sm.whist[warp][(key >> lo_bit) & dmask], 1u);
        }
        bsync();
        if (tid < 256) {
            uint32_t t = 0;
#pragma unroll 4
            for (int w = 0; w < T / 32; ++w) t += sm.whist[w][tid];
            sm.total[tid] = t;
        }
        bsync();
        if (warp == 0) {
            // lane owns buckets 8*lane .. 8*lane+7; suffix sums over lanes from the top.
            uint32_t own = 0;
#pragma unroll
            for (int b = 0; b < 8; ++b) own += sm.total[8 * lane + b];
            uint32_t suf = own;  // inclusive suffix: sum over lanes >= lane
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_down_sync(0xffffffffu, suf, o);
                if (lane + o < 32) suf += v;
            }
            const uint32_t above = suf - own;  // keys in buckets of higher lanes
            if (above < (uint32_t)remaining && (uint32_t)remaining <= suf) {
                uint32_t acc = above;
                int b = 7;
                for (; b >= 0; --b) {
                    const uint32_t c = sm.total[8 * lane + b];
                    if (acc + c >= (uint32_t)remaining) break;
                    acc += c;
                }
                sm.bcast[0] = 8 * lane + b;
                sm.bcast[1] = remaining - (int)acc;
            }
        }
        bsync();
        prefix |= ((uint32_t)sm.bcast[0]) << lo_bit;
        remaining = sm.bcast[1];
        hi_bit = lo_bit;
        bsync();
    }
    tau_key = prefix;
    need_eq = remaining;
    cnt_gt = k - remaining;
}

template <int T>
__device__ void block_kth_largest(const float* vals, int n, int k, SelectSmem<T>& sm, uint32_t& tau_key, int& cnt_gt,
                                  int& need_eq) {
    block_kth_largest_keys<T, 0>([vals](int i) { return abs_key(vals[i]); }, n, k, sm, tau_key, cnt_gt, need_eq);
}

// Index-ordered compaction of two classes over [0, n).  cls(i) returns 1 (list A),
// 2 (list B) or 0.  At most limit_b entries go to list B (the first by index).
// Returns the two counts in (na, nb).
template <int T, typename Cls, typename EmitA, typename EmitB>
__device__ void block_compact2(int n, SelectSmem<T>& sm, int limit_b, Cls cls, EmitA emit_a, EmitB emit_b, int& na,
                               int& nb) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = warp_chunk(n, T / 32);
    const int beg = warp * chunk, end = min(n, beg + chunk);
    int ca = 0, cb = 0;
    for (int i0 = beg; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const int c = i < end ? cls(i) : 0;
        ca += __popc(__ballot_sync(0xffffffffu, c == 1));
        cb += __popc(__ballot_sync(0xffffffffu, c == 2));
    }
    if (lane == 0) {
        sm.wcnt_a[warp] = ca;
        sm.wcnt_b[warp] = cb;
    }
    __syncthreads();
    if (warp == 0) {
        int a = lane < T / 32 ? sm.wcnt_a[lane] : 0, b = lane < T / 32 ? sm.wcnt_b[lane] : 0;
        int ia = a, ib = b;
        for (int o = 1; o < 32; o <<= 1) {
            const int va = __shfl_up_sync(0xffffffffu, ia, o), vb = __shfl_up_sync(0xffffffffu, ib, o);
            if (lane >= o) {
                ia += va;
                ib += vb;
            }
        }
        if (lane < T / 32) {
            sm.wcnt_a[lane] = ia - a;  // exclusive offsets
            sm.wcnt_b[lane] = ib - b;
        }
        if (lane == 31) {
            sm.bcast[0] = ia;
            sm.bcast[1] = ib;
        }
    }
    __syncthreads();
    int oa = sm.wcnt_a[warp], ob = sm.wcnt_b[warp];
    for (int i0 = beg; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const int c = i < end ? cls(i) : 0;
        const uint32_t ba = __ballot_sync(0xffffffffu, c == 1), bb = __ballot_sync(0xffffffffu, c == 2);
        const uint32_t lt = (1u << lane) - 1u;
        if (c == 1) emit_a(oa + __popc(ba & lt), i);
        if (c == 2) {
            const int pos = ob + __popc(bb & lt);
            if (pos < limit_b) emit_b(pos, i);
        }
        oa += __popc(ba);
        ob += __popc(bb);
    }
    na = sm.bcast[0];
    nb = min(sm.bcast[1], limit_b);
    __syncthreads();
}

// Final pick: of the n_band rows whose exact scores are in ws.band_exact, the `need`
// best under (|v| desc, index asc) are appended to the hit list after the n_in
// certain rows.  Runs in one CTA of T threads.
// `stage` (optional, stage_cap floats of shared memory) caches the exact scores so the
// passes below do not wait on global memory each time.
template <int T>
__device__ void final_pick_block(TokenWs ws, int* err, SelectSmem<T>& sm, float* stage = nullptr, int stage_cap = 0) {
    const int n_in = ws.sel->n_in, n_band = ws.sel->n_band;
    int need = ws.sel->need;
    if (need <= 0 || n_band <= 0) return;
    // NaN in an exact score: the reference panics.
    const bool staged = stage != nullptr && n_band <= stage_cap;
    for (int i = threadIdx.x; i < n_band; i += T) {
        const float v = ws.band_exact[i];
        if (v != v) set_err(err, DEV_ERR_NAN_SCORE);
        if (staged) stage[i] = v;
    }
    const float* ex = staged ? stage : ws.band_exact;
    __syncthreads();
    if (need >= n_band) {
        for (int i = threadIdx.x; i < n_band; i += T) {
            ws.hit_idx[n_in + i] = ws.band_idx[i];
            ws.hit_score[n_in + i] = ws.band_exact[i];
        }
        return;
    }
    uint32_t tau_key;
    int cnt_gt, need_eq;
    block_kth_largest<T>(ex, n_band, need, sm, tau_key, cnt_gt, need_eq);
    // Ordered compaction: strictly-greater rows and the first need_eq equal rows, merged
    // in index order.  Two passes keep it simple: class 1 = greater, class 2 = equal.
    // Positions: greater rows and equal rows interleave by index, so emit both through
    // one ordered stream by classifying "taken" in a first pass over equals.
    // Equal rows taken = the first need_eq by index -> find the index cut with list B.
    __shared__ int s_cut;
    if (threadIdx.x == 0) s_cut = n_band;  // exclusive upper bound on positions of taken equal rows
    __syncthreads();
    int na, nb;
    block_compact2<T>(
        n_band, sm, need_eq, [&](int i) { return abs_key(ex[i]) == tau_key ? 2 : 0; },
        [&](int, int) {}, [&](int pos, int i) { if (pos == need_eq - 1) s_cut = i + 1; }, na, nb);
    __syncthreads();
    const int cut = s_cut;
    block_compact2<T>(
        n_band, sm, 0,
        [&](int i) {
            const uint32_t key = abs_key(ex[i]);
            return (key > tau_key || (key == tau_key && i < cut)) ? 1 : 0;
        },
        [&](int pos, int i) {
            ws.hit_idx[n_in + pos] = ws.band_idx[i];
            ws.hit_score[n_in + pos] = ex[i];
        },
        [&](int, int) {}, na, nb);
}

}  // namespace lq
