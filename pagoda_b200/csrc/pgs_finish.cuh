// The reference's rule applied to a row's short candidate list: exact probabilities
// exp((x - max) / t) / sum (sampler.rs:92-114), top-k threshold with every tie kept
// (sampler.rs:116-128), top-p walk by probability descending / id ascending (sampler.rs:130-150),
// then the total and the inverse-CDF walk in id order (sampler.rs:40-55).  Shared by the finish
// kernel of the fused path and by the merge kernel of the vocabulary-sharded path.
#pragma once

#include <cuda_runtime.h>
#include <cstddef>

#include "pgs_args.cuh"
#include "pgs_block.cuh"
#include "pgs_fused.cuh"

namespace pgs {

struct FinishSmem {
    ReduceSmem rs;
    unsigned long long exp_tab[32];
    uint32_t m_id[F_MCAP];          // candidate ids, arrival order
    float p[F_MCAP];                // probabilities, arrival order
    uint32_t sid[F_MCAP];           // ids ascending
    float sp[F_MCAP];               // probabilities in id order (zeroed when dropped)
    float rp[F_MCAP];               // probabilities descending (ties: id ascending)
    uint32_t rpos[F_MCAP];          // position in the id-ordered list of the entry at each rank
    SeqSmem seq;
    uint32_t n_live;
    float bcast_f;
    int bcast_i;
};

// Exact left fold of n shared-memory floats, called by one warp: returns the total and leaves every
// running value in pre[0..n).  One lane does the additions: the loads do not depend on the running value, so
// they are requested eight at a time (two 128-bit loads) and the dependent chain is the additions alone
// (warp shuffles would put tens of cycles between two of them).  v and pre: 16-byte aligned arrays whose
// length is a multiple of 8 and at least n (entries past n are read and written, not used).
__device__ __forceinline__ float warp_prefix(const float* v, int n, float* pre) {
    const int lane = threadIdx.x & 31;
    float acc = 0.0f;
    if (lane == 0) {
#pragma unroll 1
        for (int j0 = 0; j0 < n; j0 += 8) {
            const float4 lo4 = *reinterpret_cast<const float4*>(v + j0), hi4 = *reinterpret_cast<const float4*>(v + j0 + 4);
            float x[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
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


// Called by every thread of a 1024-thread CTA.  cand_id / cand_x: the row's n <= F_MCAP candidates
// (any order); V: the full vocabulary size (the CDF walk falls through to V - 1, sampler.rs:54).
__device__ __forceinline__ void finish_row(FinishSmem& sm, const RowArgs& a, uint32_t row, uint32_t V,
                                           const uint32_t* cand_id, const float* cand_x, uint32_t n, float m,
                                           float t, float S, uint32_t top_k, float top_p, float u01,
                                           uint32_t amax, int status) {
    const int tid = threadIdx.x;
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    const bool use_p = !(top_p >= 1.0f);
    const bool norm = S > 1e-9f;
    __syncthreads();
    for (uint32_t j = tid; j < n; j += NT) {
        sm.m_id[j] = cand_id[j];
        const float e = softmax_num(cand_x[j], m, t, sm.exp_tab);   // exact expf
        sm.p[j] = norm ? fdiv(e, S) : e;
    }
    __syncthreads();
    // rank every candidate by id and by (probability descending, id ascending)
    if (n <= 256u) {
        for (uint32_t j = tid; j < n; j += NT) {
            const uint32_t idj = sm.m_id[j];
            const float pj = sm.p[j];
            uint32_t r_id = 0, r_p = 0;
#pragma unroll 8
            for (uint32_t o = 0; o < n; o++) {   // broadcast loads, independent of one another: requested in batches
                const uint32_t ido = sm.m_id[o];
                const float po = sm.p[o];
                r_id += ido < idj;
                r_p += (po > pj) || (po == pj && ido < idj);
            }
            sm.sid[r_id] = idj;
            sm.sp[r_id] = pj;
            sm.rp[r_p] = pj;
            sm.rpos[r_p] = r_id;
        }
    } else {
        // long lists: two bitonic sorts of 64-bit keys in place of the quadratic counting.  m_id and p are
        // adjacent and together hold F_MCAP keys.
        static_assert(offsetof(FinishSmem, p) == offsetof(FinishSmem, m_id) + sizeof(uint32_t) * F_MCAP, "key space");
        unsigned long long* keys = reinterpret_cast<unsigned long long*>(sm.m_id);
        uint32_t npad = 512;
        while (npad < n) npad <<= 1;
        uint32_t idr[F_MCAP / NT];
        float pr[F_MCAP / NT];
#pragma unroll
        for (int u = 0; u < F_MCAP / NT; u++) {
            const uint32_t j = tid + u * NT;
            idr[u] = j < n ? sm.m_id[j] : 0u;
            pr[u] = j < n ? sm.p[j] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < F_MCAP / NT; u++) {   // by id ascending; the padding sorts to the end
            const uint32_t j = tid + u * NT;
            if (j < npad) keys[j] = j < n ? ((unsigned long long)idr[u] << 32) | f2u(pr[u]) : ~0ull;
        }
        bitonic_sort(keys, (int)npad, keys);
        for (uint32_t j = tid; j < n; j += NT) { sm.sid[j] = (uint32_t)(keys[j] >> 32); sm.sp[j] = u2f((uint32_t)keys[j]); }
        __syncthreads();
        for (uint32_t j = tid; j < npad; j += NT)   // by (p, position descending) ascending = rank descending; padding first
            keys[j] = j < n ? ((unsigned long long)f2u(sm.sp[j]) << 32) | (0xffffffffu - j) : 0ull;
        bitonic_sort(keys, (int)npad, keys);
        for (uint32_t r = tid; r < n; r += NT) {
            const unsigned long long k = keys[npad - 1u - r];
            sm.rp[r] = u2f((uint32_t)(k >> 32));
            sm.rpos[r] = 0xffffffffu - (uint32_t)k;
        }
        __syncthreads();
    }
    if (tid == 0) sm.n_live = 0;
    __syncthreads();
    // top-k: every tie at the k-th probability survives; entries with zero probability never matter
    {
        const float thr = (top_k != 0u && top_k <= n) ? sm.rp[top_k - 1] : 0.0f;
        for (uint32_t j = tid; j < n; j += NT) {
            const bool live = sm.rp[j] >= thr && sm.rp[j] > 0.0f;
            const bool next_live = j + 1 < n && sm.rp[j + 1] >= thr && sm.rp[j + 1] > 0.0f;
            if (live && !next_live) sm.n_live = j + 1;
        }
    }
    __syncthreads();
    const uint32_t n_live = sm.n_live;
    // top-p walk in ranked order
    uint32_t keep = n_live;
    if (use_p && n_live > 0) {
        int found = -1;
        if (tid < 32) {   // one lane folds, at four cycles per term; the parallel emulation only pays beyond this size
            warp_prefix(sm.rp, (int)n_live, sm.p);   // sm.p is free once the candidates are ranked
            found = warp_find(sm.p, (int)n_live, SEQ_FIND_GE, top_p);
            if (tid == 0) sm.bcast_i = found;
        }
        __syncthreads();
        found = sm.bcast_i;
        if (found >= 0) keep = (uint32_t)found + 1;
    }
    __syncthreads();
    for (uint32_t j = keep + tid; j < n; j += NT) sm.sp[sm.rpos[j]] = 0.0f;
    __syncthreads();
    // total and inverse-CDF pick in id order
    float total;
    int pick = -1;
    if (tid < 32) {
        const float tt = warp_prefix(sm.sp, (int)n, sm.p);
        int f = -1;
        if (tt > 1e-9f) f = warp_find(sm.p, (int)n, SEQ_FIND_GT, fmul(u01, tt));
        if (tid == 0) { sm.bcast_f = tt; sm.bcast_i = f; }
    }
    __syncthreads();
    total = sm.bcast_f;
    pick = sm.bcast_i;
    if (tid == 0) {
        uint32_t token = amax;
        int drew = 0;
        if (total > 1e-9f) { token = pick >= 0 ? sm.sid[pick] : V - 1; drew = 1; }
        a.token[row] = token; a.status[row] = status;
        if (a.drew) a.drew[row] = (uint8_t)drew;
        if (a.argmax) a.argmax[row] = amax;
        if (a.row_max) a.row_max[row] = m;
        if (a.sumexp) a.sumexp[row] = S;
        if (a.total) a.total[row] = total;
    }
    if (a.n_kept || a.dump_ids || a.dump_probs) {   // diagnostics: the kept set in id order
        uint32_t done = 0;
        for (uint32_t base = 0; base < n; base += NT) {
            const uint32_t j = base + tid;
            const uint32_t kept = (j < n && sm.sp[j] > 0.0f) ? 1u : 0u;
            uint32_t tot;
            const uint32_t at = done + block_excl_scan_u32(kept, &tot, sm.rs);
            if (kept && at < a.dump_cap) {
                if (a.dump_ids) a.dump_ids[(size_t)row * a.dump_cap + at] = sm.sid[j];
                if (a.dump_probs) a.dump_probs[(size_t)row * a.dump_cap + at] = sm.sp[j];
            }
            done += tot;
        }
        if (tid == 0 && a.n_kept) a.n_kept[row] = done;
    }
}


}  // namespace pgs
