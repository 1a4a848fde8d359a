// Block-level building blocks of the row kernels: reductions, scans, the exact emulation of an
// f32 left-fold sum, radix select, ordered compaction and a bitonic sort.
//
// All functions are called by every thread of a 1024-thread CTA (no divergent callers) and
// synchronise internally with __syncthreads().
#pragma once

#include <cuda_runtime.h>
#include <limits.h>

#include "pgs_math.cuh"

namespace pgs {

constexpr int NT = 1024;       // threads per CTA
constexpr int NW = NT / 32;    // warps per CTA
constexpr unsigned FULL = 0xffffffffu;

// ---------------------------------------------------------------------------- reductions

struct ReduceSmem {
    float f[NW];
    uint32_t u[NW];
    unsigned long long ull[NW];
    float bf;
    uint32_t bu;
    unsigned long long bull;
};

__device__ __forceinline__ uint32_t block_sum_u32(uint32_t v, ReduceSmem& s) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.u[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint32_t w = s.u[threadIdx.x];
        for (int o = 16; o; o >>= 1) w += __shfl_xor_sync(FULL, w, o);
        if (threadIdx.x == 0) s.bu = w;
    }
    __syncthreads();
    return s.bu;
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, ReduceSmem& s) {
    for (int o = 16; o; o >>= 1) {
        unsigned long long w = __shfl_xor_sync(FULL, v, o);
        v = w > v ? w : v;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.ull[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        unsigned long long w = s.ull[threadIdx.x];
        for (int o = 16; o; o >>= 1) {
            unsigned long long x = __shfl_xor_sync(FULL, w, o);
            w = x > w ? x : w;
        }
        if (threadIdx.x == 0) s.bull = w;
    }
    __syncthreads();
    return s.bull;
}

// exclusive scan of one uint32 per thread; *total receives the block sum
__device__ __forceinline__ uint32_t block_excl_scan_u32(uint32_t v, uint32_t* total, ReduceSmem& s) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t t = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) s.u[w] = inc;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint32_t x = s.u[threadIdx.x], xi = x;
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t t = __shfl_up_sync(FULL, xi, o);
            if (lane >= o) xi += t;
        }
        s.u[threadIdx.x] = xi - x;
        if (threadIdx.x == 31) s.bu = xi;
    }
    __syncthreads();
    *total = s.bu;
    return s.u[w] + inc - v;
}

// exclusive scan of one float per thread (plain adds: only used as an estimate)
__device__ __forceinline__ float block_excl_scan_f32(float v, ReduceSmem& s) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        float t = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) s.f[w] = inc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float x = s.f[threadIdx.x], xi = x;
        for (int o = 1; o < 32; o <<= 1) {
            float t = __shfl_up_sync(FULL, xi, o);
            if (lane >= o) xi += t;
        }
        s.f[threadIdx.x] = xi - x;
    }
    __syncthreads();
    return s.f[w] + (inc - v);
}

// ------------------------------------------------- exact emulation of an f32 left fold
//
// The reference adds probabilities one by one in f32 (sampler.rs:42, :99-113, :136-144).  With
// ~150k terms that fold loses the small terms in a data-dependent way (several 1e-4 relative on
// peaked rows), so a tree reduction does not reproduce it.  It can still be evaluated in
// parallel: while the running value stays inside one binade [2^k, 2^(k+1)) every addition of a
// non-negative term is an integer addition in units of that binade's ulp, and the only thing
// that depends on the running value is the parity of its mantissa (round-half-to-even).  So a
// chunk of terms is summarised by two integers -- the mantissa increment for an even and for
// an odd start -- obtained by running the real float additions from the two canonical starts
// 2^k and 2^k + ulp.  Summaries compose associatively.  The binade k is guessed per chunk from
// a plain prefix sum; a summary is only applied when the exact running value really lies in
// binade k and stays there, otherwise that chunk is re-added term by term.  The result is
// bit-identical to the sequential fold for any input.

constexpr int SEQ_L = 8;                   // terms per thread per tile
constexpr int SEQ_TILE = NT * SEQ_L;
constexpr int SEQ_K_NONE = -1;             // summary unusable: re-add the chunk term by term
constexpr int SEQ_K_IDENT = -2;            // all terms zero: the running value cannot change
constexpr uint32_t SEQ_SAT = 1u << 30;

enum { SEQ_SUM = 0, SEQ_FIND_GE = 1, SEQ_FIND_GT = 2 };

struct SeqSmem {
    float tile[SEQ_TILE];
    uint32_t td0[NT], td1[NT];
    int tk[NT];
    float tstart[NT];
    uint32_t wd0[NW], wd1[NW];
    int wk[NW];
    float wstart[NW];
    int wslow[NW];
    float acc;
    int found;
};

__device__ __forceinline__ bool seq_pred(int mode, float acc, float target) {
    return mode == SEQ_FIND_GE ? (acc >= target) : (target < acc);
}

// try to apply a (k, d0, d1) summary to the exact running value; false = not applicable
__device__ __forceinline__ bool seq_apply(float& a, int k, uint32_t d0, uint32_t d1) {
    if (k == SEQ_K_IDENT) return true;
    if (k == SEQ_K_NONE) return false;
    uint32_t b = f2u(a);
    if ((int)(b & 0x7f800000u) != k) return false;
    uint32_t d = (b & 1u) ? d1 : d0;
    uint32_t m = (b & 0x007fffffu) | 0x00800000u;
    if (d >= SEQ_SAT || m + d >= 0x01000000u) return false;
    a = u2f(b + d);
    return true;
}

// f(i) for i in [0, n) must be finite and >= 0.  Returns the exact left-fold value: over all n
// terms for SEQ_SUM, else up to and including the first index where the predicate holds
// (*found = that index, or -1 when it never holds and the fold ran to the end).
template <class F>
__device__ float seq_scan(F f, int n, float acc0, int mode, float target, int* found, SeqSmem& sm,
                          ReduceSmem& rs) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    __syncthreads();
    if (tid == 0) { sm.acc = acc0; sm.found = INT_MAX; }
    __syncthreads();
    int result_found = -1;
    for (int base = 0; base < n; base += SEQ_TILE) {
        const float a_tile = sm.acc;
        const int o = base + tid * SEQ_L;
        float v[SEQ_L];
        float c = 0.0f;
#pragma unroll
        for (int j = 0; j < SEQ_L; j++) {
            v[j] = (o + j < n) ? f(o + j) : 0.0f;
            sm.tile[tid * SEQ_L + j] = v[j];
            c += v[j];
        }
        const float pre = block_excl_scan_f32(c, rs);
        const float t_guess = a_tile + pre;
        // per-thread summary
        int k;
        uint32_t d0 = 0, d1 = 0;
        const uint32_t e = f2u(t_guess) & 0x7f800000u;
        if (c == 0.0f) {
            k = SEQ_K_IDENT;
        } else if (e == 0u || e == 0x7f800000u) {
            k = SEQ_K_NONE;
        } else {
            k = (int)e;
            float a0 = u2f(e), a1 = u2f(e + 1u);
#pragma unroll
            for (int j = 0; j < SEQ_L; j++) { a0 = fadd(a0, v[j]); a1 = fadd(a1, v[j]); }
            d0 = ((f2u(a0) & 0x7f800000u) == e) ? f2u(a0) - e : SEQ_SAT;
            d1 = ((f2u(a1) & 0x7f800000u) == e) ? f2u(a1) - (e + 1u) : SEQ_SAT;
        }
        sm.tk[tid] = k; sm.td0[tid] = d0; sm.td1[tid] = d1;
        // warp composition: IDENT lanes adopt the warp's binade
        unsigned real = __ballot_sync(FULL, k >= 0);
        unsigned none = __ballot_sync(FULL, k == SEQ_K_NONE);
        int wk;
        uint32_t c0 = d0, c1 = d1;
        if (none) {
            wk = SEQ_K_NONE;
        } else if (!real) {
            wk = SEQ_K_IDENT;
        } else {
            int krep = __shfl_sync(FULL, k, __ffs(real) - 1);
            bool same = __all_sync(FULL, k == krep || k == SEQ_K_IDENT);
            wk = same ? krep : SEQ_K_NONE;
        }
        uint32_t e0 = 0, e1 = 0;  // exclusive prefix of this lane inside its warp
        if (wk >= 0) {
            for (int s = 1; s < 32; s <<= 1) {
                uint32_t l0 = __shfl_up_sync(FULL, c0, s), l1 = __shfl_up_sync(FULL, c1, s);
                if (lane >= s) {
                    // compose(left, mine)(p) = left_p + mine_{(p + left_p) & 1}
                    uint32_t n0 = l0 + ((l0 & 1u) ? c1 : c0);
                    uint32_t n1 = l1 + (((l1 + 1u) & 1u) ? c1 : c0);
                    c0 = (l0 >= SEQ_SAT || n0 >= SEQ_SAT) ? SEQ_SAT : n0;
                    c1 = (l1 >= SEQ_SAT || n1 >= SEQ_SAT) ? SEQ_SAT : n1;
                }
            }
            e0 = __shfl_up_sync(FULL, c0, 1);
            e1 = __shfl_up_sync(FULL, c1, 1);
            if (lane == 0) { e0 = 0; e1 = 0; }
        }
        if (lane == 31) { sm.wk[w] = wk; sm.wd0[w] = c0; sm.wd1[w] = c1; }
        __syncthreads();
        if (tid == 0) {
            float a = a_tile;
            for (int ww = 0; ww < NW; ww++) {
                sm.wstart[ww] = a;
                if (seq_apply(a, sm.wk[ww], sm.wd0[ww], sm.wd1[ww])) { sm.wslow[ww] = 0; continue; }
                sm.wslow[ww] = 1;
                for (int l = 0; l < 32; l++) {
                    const int t = ww * 32 + l;
                    sm.tstart[t] = a;
                    if (!seq_apply(a, sm.tk[t], sm.td0[t], sm.td1[t])) {
                        for (int j = 0; j < SEQ_L; j++) a = fadd(a, sm.tile[t * SEQ_L + j]);
                    }
                }
            }
            sm.acc = a;
        }
        __syncthreads();
        if (mode != SEQ_SUM && seq_pred(mode, sm.acc, target)) {
            float a;
            if (sm.wslow[w]) {
                a = sm.tstart[tid];
            } else {
                a = sm.wstart[w];
                if (wk >= 0) a = u2f(f2u(a) + ((f2u(a) & 1u) ? e1 : e0));
            }
            int idx = INT_MAX;
#pragma unroll
            for (int j = 0; j < SEQ_L; j++) {
                a = fadd(a, v[j]);
                if (idx == INT_MAX && o + j < n && seq_pred(mode, a, target)) idx = o + j;
            }
            if (idx != INT_MAX) atomicMin(&sm.found, idx);
            __syncthreads();
            result_found = sm.found;
            break;
        }
    }
    __syncthreads();
    if (found) *found = result_found;
    return sm.acc;
}

// ---------------------------------------------------------------------------- radix select
//
// Key of the k-th largest element (k is 1-based) of keyf(i), i in [0, n); three passes over 11,
// 11 and 10 key bits with a shared-memory histogram.  Returns 0 when n < k.

struct SelectSmem {
    uint32_t hist[2048];
    uint32_t prefix, k;
};

template <class KF>
__device__ uint32_t radix_select_kth(KF keyf, int n, uint32_t k, SelectSmem& sm, ReduceSmem& rs) {
    if ((uint32_t)n < k) return 0u;
    const int tid = threadIdx.x;
    uint32_t prefix = 0, mask = 0;
    const int shifts[3] = {21, 10, 0};
    const int widths[3] = {11, 11, 10};
    for (int pass = 0; pass < 3; pass++) {
        const int sh = shifts[pass], nb = 1 << widths[pass];
        __syncthreads();
        for (int b = tid; b < 2048; b += NT) sm.hist[b] = 0;
        __syncthreads();
        for (int i = tid; i < n; i += NT) {
            uint32_t key = keyf(i);
            if ((key & mask) == prefix) atomicAdd(&sm.hist[(key >> sh) & (nb - 1)], 1u);
        }
        __syncthreads();
        // thread t owns the bins (from the top) 2t and 2t+1
        uint32_t b_hi = nb - 1 - 2 * tid, b_lo = b_hi - 1;
        uint32_t c_hi = (2 * tid < nb) ? sm.hist[b_hi] : 0u;
        uint32_t c_lo = (2 * tid + 1 < nb) ? sm.hist[b_lo] : 0u;
        uint32_t total;
        uint32_t above = block_excl_scan_u32(c_hi + c_lo, &total, rs);
        if (above < k && k <= above + c_hi) {
            sm.prefix = prefix | (b_hi << sh); sm.k = k - above;
        } else if (above + c_hi < k && k <= above + c_hi + c_lo) {
            sm.prefix = prefix | (b_lo << sh); sm.k = k - above - c_hi;
        }
        __syncthreads();
        prefix = sm.prefix; k = sm.k;
        mask |= (uint32_t)(nb - 1) << sh;
    }
    __syncthreads();
    return prefix;
}

// ---------------------------------------------------------------------------- bitonic sort
//
// Ascending sort of n_pad (a power of two) 64-bit keys by the whole CTA.  `keys` may point to
// shared or global memory.  When the array is larger than the shared tile, the strides below the
// tile size are done tile by tile in shared memory.

constexpr int SORT_TILE = 4096;  // 32 KB of u64

__device__ __forceinline__ void bitonic_step(unsigned long long* a, int i, int j, int k) {
    int ixj = i ^ j;
    if (ixj > i) {
        unsigned long long x = a[i], y = a[ixj];
        bool asc = (i & k) == 0;
        if ((x > y) == asc) { a[i] = y; a[ixj] = x; }
    }
}

__device__ __forceinline__ void bitonic_sort(unsigned long long* keys, int n_pad, unsigned long long* tile /*SORT_TILE*/) {
    const int tid = threadIdx.x;
    __syncthreads();
    if (n_pad <= SORT_TILE) {
        // whole array fits: stage it in the shared tile unless it already lives there
        unsigned long long* a = keys;
        if (keys != tile) {
            for (int i = tid; i < n_pad; i += NT) tile[i] = keys[i];
            a = tile;
            __syncthreads();
        }
        for (int k = 2; k <= n_pad; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int i = tid; i < n_pad; i += NT) bitonic_step(a, i, j, k);
                __syncthreads();
            }
        if (keys != tile) {
            for (int i = tid; i < n_pad; i += NT) keys[i] = tile[i];
            __syncthreads();
        }
        return;
    }
    for (int k = 2; k <= n_pad; k <<= 1) {
        int j = k >> 1;
        for (; j >= SORT_TILE; j >>= 1) {
            for (int i = tid; i < n_pad; i += NT) bitonic_step(keys, i, j, k);
            __syncthreads();
        }
        // remaining strides (< SORT_TILE) touch only elements of the same aligned tile
        for (int t0 = 0; t0 < n_pad; t0 += SORT_TILE) {
            for (int i = tid; i < SORT_TILE; i += NT) tile[i] = keys[t0 + i];
            __syncthreads();
            for (int jj = j; jj > 0; jj >>= 1) {
                for (int i = tid; i < SORT_TILE; i += NT) {
                    int ixj = i ^ jj;
                    if (ixj > i) {
                        unsigned long long x = tile[i], y = tile[ixj];
                        bool asc = ((t0 + i) & k) == 0;
                        if ((x > y) == asc) { tile[i] = y; tile[ixj] = x; }
                    }
                }
                __syncthreads();
            }
            for (int i = tid; i < SORT_TILE; i += NT) keys[t0 + i] = tile[i];
            __syncthreads();
        }
    }
}

}  // namespace pgs
