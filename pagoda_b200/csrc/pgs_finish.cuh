// The reference's rule applied to a row's candidate list by one CTA of any size: exact probabilities
// exp((x - max) / t) / sum (sampler.rs:92-114), top-k threshold with every tie kept
// (sampler.rs:116-128), top-p walk by probability descending / id ascending (sampler.rs:130-150),
// then the total and the inverse-CDF walk in id order (sampler.rs:40-55).  Used by the streaming row
// kernel for its own rows and by the merge kernel of the vocabulary-sharded path.
#pragma once

#include <cuda_runtime.h>
#include <cstddef>

#include "pgs_args.cuh"
#include "pgs_block.cuh"

namespace pgs {

constexpr int F_MCAP = 2048;       // longest candidate list (a power of two)
constexpr int F_QUAD = 256;        // lists up to this length are ranked by counting, longer ones by sorting

// Working arrays of the finish, in shared memory: each holds CAP entries (CAP a power of two >= 512, the
// longest list the owner hands in).
template <int CAP>
struct FinishArraysT {
    unsigned long long key[CAP];   // sort keys
    uint32_t sid[CAP];             // ids ascending
    float sp[CAP];                 // probabilities in id order (zeroed when dropped)
    float rp[CAP];                 // probabilities descending (ties: id ascending)
    uint32_t rpos[CAP];            // position in the id-ordered list of the entry at each rank
    float fp[CAP];                 // running sums of the serial folds
    uint32_t n_live;
};
using FinishArrays = FinishArraysT<F_MCAP>;

// Exact left fold of n shared-memory floats, called by one warp: returns the total and leaves every
// running value in pre[0..n).  One lane does the additions: the loads do not depend on the running value, so
// they are requested eight at a time (two 128-bit loads) and the dependent chain is the additions alone
// (warp shuffles would put tens of cycles between two of them).  v and pre: 16-byte aligned arrays whose
// length is a multiple of 8 and at least n (entries past n are read and written, not used).
__device__ __forceinline__ float warp_prefix(const float* v, int n, float* pre) {
    const int lane = threadIdx.x & 31;
    float acc = 0.0f;
    if (lane == 0 && n > 0) {
        float4 lo4 = *reinterpret_cast<const float4*>(v), hi4 = *reinterpret_cast<const float4*>(v + 4);
#pragma unroll 1
        for (int j0 = 0; j0 < n; j0 += 8) {
            float x[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
            if (j0 + 8 < n) {   // the next eight are on their way while these are added
                lo4 = *reinterpret_cast<const float4*>(v + j0 + 8);
                hi4 = *reinterpret_cast<const float4*>(v + j0 + 12);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                acc = fadd(acc, j0 + u < n ? x[u] : 0.0f);
                x[u] = acc;
            }
            *reinterpret_cast<float4*>(pre + j0) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(pre + j0 + 4) = make_float4(x[4], x[5], x[6], x[7]);
        }
    }
    __syncwarp();
    return __shfl_sync(FULL, acc, 0);
}

// First index whose running value satisfies the predicate (mode/target as in seq_scan), or -1; one warp.
__device__ __forceinline__ int warp_find(const float* pre, int n, int mode, float target) {
    const int lane = threadIdx.x & 31;
#pragma unroll 1
    for (int base = 0; base < n; base += 32) {
        const int j = base + lane;
        const unsigned hit = __ballot_sync(FULL, j < n && seq_pred(mode, pre[j], target));
        if (hit) return base + __ffs(hit) - 1;
    }
    return -1;
}

// Ascending bitonic sort of n_pad (a power of two) 64-bit keys in shared memory by a CTA of T threads.
template <int T>
__device__ __forceinline__ void cta_bitonic_sort(unsigned long long* keys, uint32_t n_pad) {
    const uint32_t tid = threadIdx.x;
    __syncthreads();
    for (uint32_t k = 2; k <= n_pad; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t i = tid; i < n_pad / 2; i += T) {   // the i-th pair of this step
                const uint32_t lo = ((i & ~(j - 1u)) << 1) | (i & (j - 1u)), hi = lo | j;
                const unsigned long long a = keys[lo], b = keys[hi];
                const bool up = (lo & k) == 0u;
                if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
            }
            __syncthreads();
        }
    }
}

// Second half of the finish, from ranked candidates: f.sid / f.sp hold the n candidates in id order, f.rp / f.rpos
// the same by (probability descending, id ascending), f.n_live is zero.  Called by every thread; ends with the row's
// outputs written.
template <int T, class FA>
__device__ __forceinline__ void cta_finish_ranked(FA& f, const RowArgs& a, uint32_t row, uint32_t V, uint32_t n, float m,
                                                  float S, uint32_t top_k, float top_p, float u01, uint32_t amax, int status) {
    const int tid = threadIdx.x, lane = tid & 31;
    __syncthreads();
    {   // top-k: every tie at the k-th probability survives; entries with zero probability never matter
        const float thr = (top_k != 0u && top_k <= n) ? f.rp[top_k - 1] : 0.0f;
        for (uint32_t j = tid; j < n; j += T) {
            const bool live = f.rp[j] >= thr && f.rp[j] > 0.0f;
            const bool next_live = j + 1 < n && f.rp[j + 1] >= thr && f.rp[j + 1] > 0.0f;
            if (live && !next_live) f.n_live = j + 1;
        }
    }
    __syncthreads();
    if (tid >= 32) return;
    // one warp: top-p walk in ranked order, then total and inverse-CDF pick in id order
    const uint32_t n_live = f.n_live;
    uint32_t keep = n_live;
    if (!(top_p >= 1.0f) && n_live > 0) {
        warp_prefix(f.rp, (int)n_live, f.fp);
        const int found = warp_find(f.fp, (int)n_live, SEQ_FIND_GE, top_p);
        if (found >= 0) keep = (uint32_t)found + 1;
    }
    for (uint32_t j = keep + lane; j < n; j += 32) f.sp[f.rpos[j]] = 0.0f;
    __syncwarp();
    const float total = warp_prefix(f.sp, (int)n, f.fp);
    int pick = -1;
    if (total > 1e-9f) pick = warp_find(f.fp, (int)n, SEQ_FIND_GT, fmul(u01, total));
    if (lane == 0) {
        uint32_t token = amax;
        int drew = 0;
        if (total > 1e-9f) { token = pick >= 0 ? f.sid[pick] : V - 1; drew = 1; }
        a.token[row] = token; a.status[row] = status;
        if (a.drew) a.drew[row] = (uint8_t)drew;
        if (a.argmax) a.argmax[row] = amax;
        if (a.row_max) a.row_max[row] = m;
        if (a.sumexp) a.sumexp[row] = S;
        if (a.total) a.total[row] = total;
    }
    if (a.n_kept || a.dump_ids || a.dump_probs) {   // diagnostics: the kept set in id order
        uint32_t done = 0;
        for (uint32_t base = 0; base < n; base += 32) {
            const uint32_t j = base + lane;
            const bool kept = j < n && f.sp[j] > 0.0f;
            const unsigned mask = __ballot_sync(FULL, kept);
            const uint32_t at = done + __popc(mask & ((1u << lane) - 1u));
            if (kept && at < a.dump_cap) {
                if (a.dump_ids) a.dump_ids[(size_t)row * a.dump_cap + at] = f.sid[j];
                if (a.dump_probs) a.dump_probs[(size_t)row * a.dump_cap + at] = f.sp[j];
            }
            done += __popc(mask);
        }
        if (lane == 0 && a.n_kept) a.n_kept[row] = done;
    }
}


// Candidates of one row -> token.  Called by every thread of a CTA of T threads (T >= F_QUAD, a multiple of 32)
// with a barrier in front; cand_id / cand_x: the row's n <= F_MCAP candidates in any order (shared memory outside
// of `f`); V: the full vocabulary size (the CDF walk falls through to V - 1, sampler.rs:54).  Ends with the row's
// outputs written; the caller needs a barrier before it reuses `f` or the candidate arrays.
template <int T, class FA>
__device__ __forceinline__ void cta_finish(FA& f, const unsigned long long* exp_tab, const RowArgs& a, uint32_t row,
                                           uint32_t V, const uint32_t* cand_id, const float* cand_x, uint32_t n, float m, float t,
                                           float S, uint32_t top_k, float top_p, float u01, uint32_t amax, int status) {
    static_assert(T >= F_QUAD && T % 32 == 0, "one thread per candidate of a short list");
    const int tid = threadIdx.x;
    const bool norm = S > 1e-9f;
    if (tid == 0) f.n_live = 0u;
    if (n <= (uint32_t)F_QUAD) {
        // short list: every candidate counts the candidates in front of it, by id and by (probability descending,
        // id ascending)
        uint32_t my_id = 0u;
        float my_p = 0.0f;
        if ((uint32_t)tid < n) {
            my_id = cand_id[tid];
            const float e = softmax_num(cand_x[tid], m, t, exp_tab);   // exact expf
            my_p = norm ? fdiv(e, S) : e;
            f.key[tid] = ((unsigned long long)f2u(my_p) << 32) | (unsigned long long)(0xffffffffu - my_id);   // p >= 0
        }
        __syncthreads();
        if ((uint32_t)tid < n) {
            const unsigned long long kj = f.key[tid];
            uint32_t r_id = 0, r_p = 0;
#pragma unroll 8
            for (uint32_t o = 0; o < n; o++) {   // broadcast loads, independent of one another
                const unsigned long long ko = f.key[o];
                r_p += ko > kj;
                r_id += (uint32_t)ko > (uint32_t)kj;   // larger ~id = smaller id
            }
            f.sid[r_id] = my_id; f.sp[r_id] = my_p; f.rp[r_p] = my_p; f.rpos[r_p] = r_id;
        }
    } else {
        // long list: sorted by id, then by (probability, position) -- two sorts of 64-bit keys
        uint32_t npad = 512;
        while (npad < n) npad <<= 1;
        for (uint32_t j = tid; j < npad; j += T) {
            unsigned long long k = ~0ull;   // the padding sorts to the end
            if (j < n) {
                const float e = softmax_num(cand_x[j], m, t, exp_tab);
                k = ((unsigned long long)cand_id[j] << 32) | f2u(norm ? fdiv(e, S) : e);
            }
            f.key[j] = k;
        }
        cta_bitonic_sort<T>(f.key, npad);
        for (uint32_t j = tid; j < n; j += T) { f.sid[j] = (uint32_t)(f.key[j] >> 32); f.sp[j] = u2f((uint32_t)f.key[j]); }
        __syncthreads();
        for (uint32_t j = tid; j < npad; j += T)   // ascending by (p, position descending) = rank descending; padding first
            f.key[j] = j < n ? ((unsigned long long)f2u(f.sp[j]) << 32) | (0xffffffffu - j) : 0ull;
        cta_bitonic_sort<T>(f.key, npad);
        for (uint32_t r = tid; r < n; r += T) {
            const unsigned long long k = f.key[npad - 1u - r];
            f.rp[r] = u2f((uint32_t)(k >> 32));
            f.rpos[r] = 0xffffffffu - (uint32_t)k;
        }
    }
    cta_finish_ranked<T, FA>(f, a, row, V, n, m, S, top_k, top_p, u01, amax, status);
}

}  // namespace pgs
