// Fused cluster kernel: the hot path of the sampler.
//
// One thread-block cluster owns one batch row.  The row is read from HBM exactly once, with
// 128-bit coalesced loads, into the distributed shared memory of the cluster (each CTA keeps a
// contiguous slice of the vocabulary as f32), and every later step of the chain
// (pagoda/src/engine.rs:1286-1314, pagoda/src/sampler.rs:28-150) works on that copy:
//
//   load + sanity + grammar bitmask AND + per-thread max      (one pass, from HBM)
//   penalties scattered from a shared-memory id->count table   (history ids of this slice only)
//   cluster-wide max / argmax, lowest id on ties               (DSMEM exchange)
//   top-k: the k-th largest per-thread maximum bounds the k-th largest logit from below, so
//          "logit >= that bound" is a superset of the top-k set that is only slightly larger;
//          those candidates are gathered and the reference's rule is applied to them exactly
//   softmax numerators in place + emulation of the reference's sequential f32 sum
//   candidates: exact probabilities, top-k threshold with ties, top-p walk, inverse-CDF pick
//
// Fidelity of this path: argmax, masks, penalties and candidate sets follow the reference bit
// for bit; candidate numerators use the exact expf; the bulk numerators that only enter the
// running sum use the hardware exp2 (a few ulp), so the sum agrees with the reference's to
// about 1e-6 relative and a decision can differ only when it sits that close to its boundary.
// Rows this kernel cannot hold (top-k off or > 1024, more candidates than its buffers, too many
// distinct history ids in one slice, unaligned rows) are appended to a work list that the
// general row kernel processes afterwards.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "pgs_args.cuh"
#include "pgs_block.cuh"

namespace cg = cooperative_groups;

namespace pgs {

constexpr int F_MAXC = 8;          // largest cluster
constexpr int F_LCAP = 1024;       // candidates per CTA
constexpr int F_MCAP = 2048;       // candidates per row (merged in CTA 0)
constexpr int F_HASH = 2048;       // id->count slots per CTA
constexpr int F_KMAX = 1024;       // largest top-k served here

struct FusedXchg {                  // peers write their slot through DSMEM
    unsigned long long best[F_MAXC];
    int nonfinite[F_MAXC];
    uint32_t ncand[F_MAXC];
    int spill[F_MAXC];
    float approx_total[F_MAXC];
    float acc_in;                   // exact running sum handed over by the previous CTA
    float sum_final;                // written into CTA 0 by the last CTA
};

// Shared-memory workspace of one CTA (the vocabulary slice follows it).  Regions are reused as
// the row moves through its phases:
//   r_a : id->count table (penalties)            -> merged candidate ids / logits (CTA 0)
//   r_b : every CTA's per-thread maxima (top-k)   -> per-thread summaries of the sum emulation
//   the slice itself (softmax numerators)         -> candidate probabilities / sort keys (CTA 0)
struct FusedSmem {
    ReduceSmem rs;
    FusedXchg xchg[2];              // alternates between consecutive rows
    unsigned long long exp_tab[32];
    union {
        struct { uint32_t hkey[F_HASH]; uint32_t hcnt[F_HASH]; } pen;
        struct { uint32_t m_id[F_MCAP]; float m_x[F_MCAP]; } mrg;
    } r_a;
    union {
        float tmax_all[F_MAXC * NT];
        struct { int tk[NT]; uint32_t td[NT]; } seq;
    } r_b;
    uint8_t redo_max[NT];
    SelectSmem sel;
    uint32_t cand_id[F_LCAP];
    float cand_x[F_LCAP];
    uint32_t cand_n;
    uint32_t m_n;
    float acc;
};

struct FusedLaunch {
    uint32_t cluster;       // CTAs per row
    uint32_t slice_len;     // floats per CTA (multiple of 32)
    uint32_t chunk;         // consecutive floats per thread in the sum pass (odd)
    uint32_t* work_rows;    // rows handed to the general kernel
    uint32_t* work_count;
};

__device__ __forceinline__ float ld_stream_f32(const float* p) { return __ldcs(p); }

// exact left fold of `n` shared-memory floats starting from `a`
__device__ __forceinline__ float fold_serial(const float* v, int n, float a) {
    for (int j = 0; j < n; j++) a = fadd(a, v[j]);
    return a;
}

__global__ void __launch_bounds__(NT, 1) fused_row_kernel(const RowArgs a, const FusedLaunch fl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FusedSmem& sm = *reinterpret_cast<FusedSmem*>(smem_raw);
    float* X = reinterpret_cast<float*>(smem_raw + ((sizeof(FusedSmem) + 15) & ~size_t(15)));
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t C = fl.cluster;
    const uint32_t rank = cluster.block_rank();
    const uint32_t n_clusters = gridDim.x / C, cluster_id = blockIdx.x / C;
    const uint32_t V = a.vocab;
    const uint32_t lo = rank * fl.slice_len;
    const uint32_t hi = min(V, lo + fl.slice_len);
    const uint32_t len = hi > lo ? hi - lo : 0u;
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    __syncthreads();
    const unsigned long long* tab = sm.exp_tab;
    uint32_t parity = 0;

    for (uint32_t row = cluster_id; row < a.rows; row += n_clusters) {
        FusedXchg& xc = sm.xchg[parity];
        const uint32_t pbuf = parity;   // exchange buffer of this row; the next synced row takes the other one
        // ------------------------------------------------------------------ parameters
        const float temp = a.temperature ? a.temperature[row] : 0.0f;
        const uint32_t top_k = a.top_k ? a.top_k[row] : 0u;
        const float top_p = a.top_p ? a.top_p[row] : 1.0f;
        const float freq = a.freq ? a.freq[row] : 0.0f;
        const float pres = a.pres ? a.pres[row] : 0.0f;
        const float rep = a.rep ? a.rep[row] : 1.0f;
        const float u01 = a.uniform ? a.uniform[row] : 0.0f;
        bool bad = !finite_f(temp) || !finite_f(top_p) || !finite_f(freq) || !finite_f(pres) ||
                   !finite_f(rep) || !(rep > 0.0f) || !finite_f(u01);
        const uint32_t* mw = nullptr;
        uint32_t gflags = 0;
        if (a.mask_table && a.mask_table[row] >= 0) {
            const int32_t t = a.mask_table[row];
            const int32_t st = a.mask_state ? a.mask_state[row] : 0;
            if (t >= MAX_TABLES || !a.tables[t].live || st < 0 || (uint32_t)st >= a.tables[t].n_states ||
                (unsigned long long)a.tables[t].words_per_state * 32ull < V) {
                bad = true;
            } else {
                mw = a.tables[t].words + (size_t)st * a.tables[t].words_per_state;
                gflags = a.tables[t].flags[st];
            }
        }
        uint32_t h0 = 0, nh = 0;
        if (a.hist_offsets) {
            h0 = a.hist_offsets[row];
            const uint32_t h1 = a.hist_offsets[row + 1];
            if (h1 < h0 || h1 - h0 > a.max_history) bad = true; else nh = h1 - h0;
        }
        if (bad) {
            if (rank == 0 && tid == 0) {
                a.token[row] = 0; a.status[row] = ROW_BAD_PARAM;
                if (a.drew) a.drew[row] = 0;
            }
            continue;
        }
        const bool greedy = temp < 1e-5f;
        const bool use_k = top_k != 0u && top_k < V;
        const bool use_p = !(top_p >= 1.0f);
        // rows this kernel does not serve go to the general kernel (decided identically by every CTA)
        const char* rowp = (const char*)a.logits + (size_t)row * a.row_stride * (a.dtype == 0 ? 4 : 2);
        const bool aligned = (((uintptr_t)rowp & 15) == 0);
        const bool defer = !aligned || (!greedy && (!use_k || top_k > (uint32_t)F_KMAX));
        if (defer) {
            if (rank == 0 && tid == 0) fl.work_rows[atomicAdd(fl.work_count, 1u)] = row;
            continue;
        }

        // ------------------------------- load slice: sanity + bitmask AND + per-thread max
        float tmax = -INFINITY;
        int nonfinite = 0;
        sm.redo_max[tid] = 0;
        if (a.dtype == 0) {
            const float4* src = (const float4*)(rowp) + lo / 4;
            const uint32_t nq = len / 4;   // len is a multiple of 4 except possibly in the last slice
            for (uint32_t q = tid; q < nq; q += NT) {
                float4 v = __ldcs(src + q);
                nonfinite |= !finite_f(v.x) | !finite_f(v.y) | !finite_f(v.z) | !finite_f(v.w);
                if (mw) {
                    const uint32_t bits = __ldg(mw + ((lo >> 5) + (q >> 3))) >> ((q & 7) * 4);
                    if (!(bits & 1u)) v.x = -INFINITY;
                    if (!(bits & 2u)) v.y = -INFINITY;
                    if (!(bits & 4u)) v.z = -INFINITY;
                    if (!(bits & 8u)) v.w = -INFINITY;
                }
                tmax = fmaxf(tmax, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
                ((float4*)X)[q] = v;
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT) {   // ragged tail of the last slice
                float x = __ldcs((const float*)rowp + lo + i);
                nonfinite |= !finite_f(x);
                if (mw && !((__ldg(mw + ((lo + i) >> 5)) >> ((lo + i) & 31)) & 1u)) x = -INFINITY;
                tmax = fmaxf(tmax, x);
                X[i] = x;
            }
        } else {
            const uint2* src = (const uint2*)(rowp) + lo / 4;    // 4 bf16 per 8-byte load
            const uint32_t nq = len / 4;
            for (uint32_t q = tid; q < nq; q += NT) {
                const uint2 r = __ldcs(src + q);
                float4 v;
                v.x = __uint_as_float(r.x << 16); v.y = __uint_as_float(r.x & 0xffff0000u);
                v.z = __uint_as_float(r.y << 16); v.w = __uint_as_float(r.y & 0xffff0000u);
                nonfinite |= !finite_f(v.x) | !finite_f(v.y) | !finite_f(v.z) | !finite_f(v.w);
                if (mw) {
                    const uint32_t bits = __ldg(mw + ((lo >> 5) + (q >> 3))) >> ((q & 7) * 4);
                    if (!(bits & 1u)) v.x = -INFINITY;
                    if (!(bits & 2u)) v.y = -INFINITY;
                    if (!(bits & 4u)) v.z = -INFINITY;
                    if (!(bits & 8u)) v.w = -INFINITY;
                }
                tmax = fmaxf(tmax, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
                ((float4*)X)[q] = v;
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT) {
                float x = __uint_as_float((uint32_t)((const unsigned short*)rowp)[lo + i] << 16);
                nonfinite |= !finite_f(x);
                if (mw && !((__ldg(mw + ((lo + i) >> 5)) >> ((lo + i) & 31)) & 1u)) x = -INFINITY;
                tmax = fmaxf(tmax, x);
                X[i] = x;
            }
        }
        nonfinite = __syncthreads_or(nonfinite);

        // --------------------------------------------------------------- penalties
        const bool do_fp = !(fabsf(freq) < 1e-6f && fabsf(pres) < 1e-6f);
        const bool do_pres = fabsf(pres) > 1e-6f;
        const bool do_rep = rep != 1.0f;
        int spill = 0;
        if (nh > 0 && (do_fp || do_rep) && !nonfinite) {
            for (int s = tid; s < F_HASH; s += NT) { sm.r_a.pen.hkey[s] = 0xffffffffu; sm.r_a.pen.hcnt[s] = 0u; }
            __syncthreads();
            for (uint32_t j = tid; j < nh; j += NT) {
                const uint32_t id = __ldg(a.hist_ids + h0 + j);
                if (id < lo || id >= hi) continue;
                uint32_t s = (id * 2654435761u) >> 21;   // 11 bits
                bool placed = false;
                for (int probe = 0; probe < 64; probe++) {
                    const uint32_t prev = atomicCAS(&sm.r_a.pen.hkey[s], 0xffffffffu, id);
                    if (prev == 0xffffffffu || prev == id) { atomicAdd(&sm.r_a.pen.hcnt[s], 1u); placed = true; break; }
                    s = (s + 1) & (F_HASH - 1);
                }
                if (!placed) spill = 1;
            }
            spill = __syncthreads_or(spill);
            if (!spill) {
                for (int s = tid; s < F_HASH; s += NT) {
                    const uint32_t id = sm.r_a.pen.hkey[s];
                    if (id == 0xffffffffu) continue;
                    const uint32_t i = id - lo;
                    float x = X[i];
                    if (do_rep) x = x > 0.0f ? fdiv(x, rep) : fmul(x, rep);
                    if (do_fp) {
                        x = fsub(x, fmul(freq, (float)sm.r_a.pen.hcnt[s]));
                        if (do_pres) x = fsub(x, pres);
                    }
                    // an overflowed penalty is non-finite; the chain treats that like a masked entry
                    X[i] = finite_f(x) ? x : -INFINITY;
                    // the thread that loaded element i must refresh its maximum
                    const uint32_t owner = (i < (len / 4) * 4) ? ((i >> 2) & (NT - 1)) : ((i - (len / 4) * 4) & (NT - 1));
                    sm.redo_max[owner] = 1;
                }
            }
            __syncthreads();
        }
        // ----------------------------------------------------------------- EOS fix
        if (mw && (gflags & 1u) && a.eos >= 0 && (uint32_t)a.eos >= lo && (uint32_t)a.eos < hi && tid == 0 &&
            !finite_f(X[a.eos - lo])) {
            X[a.eos - lo] = 0.0f;
            const uint32_t i = a.eos - lo;
            sm.redo_max[(i < (len / 4) * 4) ? ((i >> 2) & (NT - 1)) : ((i - (len / 4) * 4) & (NT - 1))] = 1;
        }
        __syncthreads();
        if (sm.redo_max[tid]) {
            tmax = -INFINITY;
            const uint32_t nq = len / 4;
            for (uint32_t q = tid; q < nq; q += NT) {
                const float4 v = ((const float4*)X)[q];
                tmax = fmaxf(tmax, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT) tmax = fmaxf(tmax, X[i]);
        }

        // ------------------------------------------------- slice max / argmax, lowest id
        // block max of the keys, then the lowest index holding it
        unsigned long long best = (unsigned long long)order_key(tmax) << 32;
        best = block_max_u64(best, sm.rs);
        const uint32_t bkey = (uint32_t)(best >> 32);
        if (bkey) {
            const float bval = key_to_float(bkey);
            uint32_t first = 0xffffffffu;
            const uint32_t nq = len / 4;
            for (uint32_t q = tid; q < nq && first == 0xffffffffu; q += NT) {
                const float4 v = ((const float4*)X)[q];
                if (v.x == bval) first = q * 4;
                else if (v.y == bval) first = q * 4 + 1;
                else if (v.z == bval) first = q * 4 + 2;
                else if (v.w == bval) first = q * 4 + 3;
            }
            for (uint32_t i = nq * 4 + tid; i < len && first == 0xffffffffu; i += NT)
                if (X[i] == bval) first = i;
            unsigned long long cand = first == 0xffffffffu ? 0ull
                                                           : ((unsigned long long)bkey << 32) |
                                                                 (unsigned long long)(0xffffffffu - (lo + first));
            best = block_max_u64(cand, sm.rs);
        } else {
            best = 0ull;
        }
        // ------------------------------------------------ cluster exchange #1
        for (uint32_t r = tid; r < C; r += NT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].best[rank] = best;
            peer->xchg[pbuf].nonfinite[rank] = nonfinite;
            peer->xchg[pbuf].spill[rank] = spill;
        }
        if (!greedy) {
            const float tm = tmax;
            for (uint32_t r = 0; r < C; r++) {
                FusedSmem* peer = cluster.map_shared_rank(&sm, r);
                peer->r_b.tmax_all[rank * NT + tid] = tm;
            }
        }
        cluster.sync();
        parity ^= 1u;
        unsigned long long gbest = 0ull;
        int any_nonfinite = 0, any_spill = 0;
        for (uint32_t r = 0; r < C; r++) {
            gbest = xc.best[r] > gbest ? xc.best[r] : gbest;
            any_nonfinite |= xc.nonfinite[r];
            any_spill |= xc.spill[r];
        }
        const bool any = gbest != 0ull;
        const float m = any ? key_to_float((uint32_t)(gbest >> 32)) : -INFINITY;
        const uint32_t amax = any ? 0xffffffffu - (uint32_t)gbest : 0u;
        const int status = any ? ROW_OK : ROW_EMPTY;
        const bool writer = rank == 0 && tid == 0;
        if (any_nonfinite) {
            if (writer) { a.token[row] = 0; a.status[row] = ROW_NONFINITE; if (a.drew) a.drew[row] = 0; }
            continue;
        }
        if (gflags & 2u) {
            if (writer) { a.token[row] = 0; a.status[row] = ROW_DEAD; if (a.drew) a.drew[row] = 0; }
            continue;
        }
        if (any_spill) {
            if (writer) fl.work_rows[atomicAdd(fl.work_count, 1u)] = row;
            continue;
        }
        if (greedy || !any) {
            if (writer) {
                a.token[row] = amax; a.status[row] = status;
                if (a.drew) a.drew[row] = 0;
                if (a.argmax) a.argmax[row] = amax;
                if (a.row_max) a.row_max[row] = m;
                if (a.sumexp) a.sumexp[row] = 0.0f;
                if (a.total) a.total[row] = 0.0f;
                if (a.n_kept) a.n_kept[row] = 0u;
            }
            continue;
        }

        // -------------------------------- top-k bound: k-th largest per-thread maximum
        const float t = fmaxf(temp, 1e-9f);
        const uint32_t kk = radix_select_kth([&](int i) { return order_key(sm.r_b.tmax_all[i]); }, (int)(C * NT),
                                             top_k, sm.sel, sm.rs);
        float cut = -INFINITY;
        if (kk) {
            const float bound = key_to_float(kk);
            // every logit whose probability could still tie with the k-th one stays above the cut
            const float delta = 4.8e-7f * (fabsf(m - bound) + 4.0f * t) + 4.8e-7f * (fabsf(bound) + fabsf(m));
            cut = bound - delta;
        }
        if (tid == 0) sm.cand_n = 0;
        __syncthreads();
        {
            const uint32_t nq = len / 4;
            for (uint32_t q = tid; q < nq; q += NT) {
                const float4 v = ((const float4*)X)[q];
                const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (vv[j] >= cut && finite_f(vv[j])) {
                        const uint32_t at = atomicAdd(&sm.cand_n, 1u);
                        if (at < (uint32_t)F_LCAP) { sm.cand_id[at] = lo + q * 4 + j; sm.cand_x[at] = vv[j]; }
                    }
                }
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT) {
                const float x = X[i];
                if (x >= cut && finite_f(x)) {
                    const uint32_t at = atomicAdd(&sm.cand_n, 1u);
                    if (at < (uint32_t)F_LCAP) { sm.cand_id[at] = lo + i; sm.cand_x[at] = x; }
                }
            }
        }
        __syncthreads();
        const uint32_t my_n = sm.cand_n;

        // --------------- softmax numerators in place (hardware exp2) + per-thread chunk sums
        const float scale = 1.4426950408889634f / t;
        const uint32_t L = fl.chunk;
        const uint32_t c0 = tid * L, c1 = min(len, c0 + L);
        float csum = 0.0f;
        for (uint32_t i = c0; i < c1; i++) {
            const float x = X[i];
            // masked entries are -inf: exp2(-inf) = +0
            const float e = ex2_approx((x - m) * scale);
            X[i] = e;
            csum += e;
        }
        const float pre = block_excl_scan_f32(csum, sm.rs);
        __syncthreads();
        if (tid == NT - 1) sm.acc = pre + csum;    // CTA total (estimate)
        __syncthreads();
        const float cta_total = sm.acc;
        // ------------------------------------------------ cluster exchange #2
        for (uint32_t r = tid; r < C; r += NT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].ncand[rank] = my_n;
            peer->xchg[pbuf].approx_total[rank] = cta_total;
        }
        cluster.sync();
        uint32_t cand_off = 0, cand_total = 0;
        float before = 0.0f;
        bool overflow = false;
        for (uint32_t r = 0; r < C; r++) {
            if (r < rank) { cand_off += xc.ncand[r]; before += xc.approx_total[r]; }
            cand_total += xc.ncand[r];
            overflow |= xc.ncand[r] > (uint32_t)F_LCAP;
        }
        overflow |= cand_total > (uint32_t)F_MCAP;
        if (overflow) {   // identical decision in every CTA
            if (writer) fl.work_rows[atomicAdd(fl.work_count, 1u)] = row;
            continue;
        }
        // candidates -> CTA 0
        {
            FusedSmem* root = cluster.map_shared_rank(&sm, 0);
            for (uint32_t j = tid; j < my_n; j += NT) {
                root->r_a.mrg.m_id[cand_off + j] = sm.cand_id[j];
                root->r_a.mrg.m_x[cand_off + j] = sm.cand_x[j];
            }
            if (rank == 0 && tid == 0) sm.m_n = cand_total;
        }
        // ---------------- per-thread summaries of the sequential sum (see pgs_block.cuh)
        {
            const float t_guess = before + pre;
            const uint32_t e = f2u(t_guess) & 0x7f800000u;
            int k;
            uint32_t d = 0;
            if (csum == 0.0f) {
                k = SEQ_K_IDENT;
            } else if (e == 0u || e == 0x7f800000u) {
                k = SEQ_K_NONE;
            } else {
                k = (int)e;
                float acc = u2f(e);
                for (uint32_t i = c0; i < c1; i++) acc = fadd(acc, X[i]);
                d = ((f2u(acc) & 0x7f800000u) == e) ? f2u(acc) - e : SEQ_SAT;
            }
            sm.r_b.seq.tk[tid] = k;
            sm.r_b.seq.td[tid] = d;
        }
        __syncthreads();
        // ----------- resolve, CTA after CTA: exact prefix while summaries apply, else re-add
        for (uint32_t turn = 0; turn < C; turn++) {
            if (turn == rank) {
                float acc = rank == 0 ? 0.0f : xc.acc_in;
                uint32_t start = 0;
                // warp 0 walks the 1024 thread summaries: 32 at a time, prefix by shuffles
                if (tid < 32) {
                    while (start < (uint32_t)NT) {
                        const uint32_t tt = start + lane;
                        const int k = tt < (uint32_t)NT ? sm.r_b.seq.tk[tt] : SEQ_K_IDENT;
                        uint32_t d = (tt < (uint32_t)NT && k >= 0) ? sm.r_b.seq.td[tt] : 0u;
                        // inclusive prefix of d with saturation
                        uint32_t inc = d;
                        for (int s = 1; s < 32; s <<= 1) {
                            uint32_t up = __shfl_up_sync(FULL, inc, s);
                            if (lane >= s) inc = min(inc + up, SEQ_SAT);
                        }
                        const uint32_t ab = f2u(acc);
                        const uint32_t mant = (ab & 0x007fffffu) | 0x00800000u;
                        const bool ok = k == SEQ_K_IDENT ||
                                        (k >= 0 && (uint32_t)k == (ab & 0x7f800000u) && (ab & 0x7f800000u) != 0u &&
                                         d < SEQ_SAT && inc < SEQ_SAT && mant + inc < 0x01000000u);
                        const unsigned okmask = __ballot_sync(FULL, ok);
                        const int nok = okmask == FULL ? 32 : __ffs(~okmask) - 1;   // leading run of valid lanes
                        if (nok > 0) {
                            const uint32_t adv = __shfl_sync(FULL, inc, nok - 1);
                            acc = u2f(ab + adv);
                        }
                        start += nok;
                        if (nok < 32 && start < (uint32_t)NT) {
                            // chunk `start` does not apply: add its terms one by one
                            const uint32_t b0 = start * L, b1 = min(len, b0 + L);
                            if (b1 > b0) acc = fold_serial(X + b0, (int)(b1 - b0), acc);
                            start += 1;
                        }
                    }
                    if (lane == 0) {
                        if (rank + 1 < C) cluster.map_shared_rank(&sm, rank + 1)->xchg[pbuf].acc_in = acc;
                        else cluster.map_shared_rank(&sm, 0)->xchg[pbuf].sum_final = acc;
                    }
                }
            }
            cluster.sync();
        }
        if (rank != 0) continue;

        // ------------------------------------------ CTA 0: the reference's rule on the candidates
        const float S = xc.sum_final;
        const uint32_t n = sm.m_n;
        unsigned long long* m_key = reinterpret_cast<unsigned long long*>(X);   // [F_MCAP], slice is dead now
        float* m_p = X + 2 * F_MCAP;                                             // [F_MCAP]
        const bool norm = S > 1e-9f;
        // sort by id (ascending) so that the CDF walk runs in id order
        uint32_t npad = 2;
        while (npad < n) npad <<= 1;
        for (uint32_t j = tid; j < npad; j += NT)
            m_key[j] = j < n ? ((unsigned long long)sm.r_a.mrg.m_id[j] << 32) | f2u(sm.r_a.mrg.m_x[j]) : ~0ull;
        bitonic_sort(m_key, (int)npad, m_key);
        for (uint32_t j = tid; j < n; j += NT) {
            const uint32_t id = (uint32_t)(m_key[j] >> 32);
            const float x = u2f((uint32_t)m_key[j]);
            const float e = softmax_num(x, m, t, tab);
            sm.r_a.mrg.m_id[j] = id;
            m_p[j] = norm ? fdiv(e, S) : e;
        }
        __syncthreads();
        // rank by probability descending, id ascending (position in the id-sorted list)
        for (uint32_t j = tid; j < npad; j += NT)
            m_key[j] = j < n ? ((unsigned long long)(~f2u(m_p[j])) << 32) | j : ~0ull;
        bitonic_sort(m_key, (int)npad, m_key);
        // top-k threshold: every tie at the k-th probability survives (sampler.rs:116-128)
        uint32_t n_live = n;
        if (top_k <= n) {
            const float thr = u2f(~(uint32_t)(m_key[top_k - 1] >> 32));
            uint32_t cnt = 0;
            for (uint32_t j = tid; j < n; j += NT) cnt += u2f(~(uint32_t)(m_key[j] >> 32)) >= thr;
            n_live = block_sum_u32(cnt, sm.rs);   // sorted descending: the survivors are a prefix
        }
        // entries with zero probability never matter
        {
            uint32_t cnt = 0;
            for (uint32_t j = tid; j < n_live; j += NT) cnt += u2f(~(uint32_t)(m_key[j] >> 32)) > 0.0f;
            n_live = block_sum_u32(cnt, sm.rs);
        }
        // top-p walk in ranked order, then total and CDF in id order (sampler.rs:130-150, 40-55)
        if (tid == 0) {
            uint32_t keep = n_live;
            if (use_p) {
                float cum = 0.0f;
                for (uint32_t j = 0; j < n_live; j++) {
                    cum = fadd(cum, u2f(~(uint32_t)(m_key[j] >> 32)));
                    if (cum >= top_p) { keep = j + 1; break; }
                }
            }
            sm.m_n = keep;
        }
        __syncthreads();
        const uint32_t keep = sm.m_n;
        for (uint32_t j = keep + tid; j < n; j += NT) m_p[(uint32_t)m_key[j]] = 0.0f;
        __syncthreads();
        if (tid == 0) {
            float total = 0.0f;
            for (uint32_t j = 0; j < n; j++) total = fadd(total, m_p[j]);
            uint32_t token = amax;
            int drew = 0;
            if (total > 1e-9f) {
                const float u = fmul(u01, total);
                float acc = 0.0f;
                token = V - 1;
                for (uint32_t j = 0; j < n; j++) {
                    acc = fadd(acc, m_p[j]);
                    if (u < acc) { token = sm.r_a.mrg.m_id[j]; break; }
                }
                drew = 1;
            }
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
                const uint32_t kept = (j < n && m_p[j] > 0.0f) ? 1u : 0u;
                uint32_t tot;
                const uint32_t at = done + block_excl_scan_u32(kept, &tot, sm.rs);
                if (kept && at < a.dump_cap) {
                    if (a.dump_ids) a.dump_ids[(size_t)row * a.dump_cap + at] = sm.r_a.mrg.m_id[j];
                    if (a.dump_probs) a.dump_probs[(size_t)row * a.dump_cap + at] = m_p[j];
                }
                done += tot;
            }
            if (tid == 0 && a.n_kept) a.n_kept[row] = done;
        }
        __syncthreads();
    }
    // no CTA may exit while a peer can still write into its shared memory
    cluster.sync();
}

// the slice buffer doubles as CTA 0's candidate workspace (sort keys + probabilities)
size_t fused_smem_bytes(uint32_t slice_len) {
    const size_t floats = slice_len > 3u * F_MCAP ? slice_len : 3u * F_MCAP;
    return ((sizeof(FusedSmem) + 15) & ~size_t(15)) + floats * sizeof(float);
}

cudaError_t configure_fused(size_t max_smem) {
    cudaError_t e = cudaFuncSetAttribute(fused_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)max_smem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(fused_row_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
}

// how many clusters of `cluster` CTAs with `smem` bytes each can be resident at once
cudaError_t fused_max_clusters(uint32_t cluster, size_t smem, int* out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaOccupancyMaxActiveClusters(out, fused_row_kernel, &cfg);
}

cudaError_t launch_fused(const RowArgs& a, const FusedLaunch& fl, uint32_t n_clusters, size_t smem,
                         cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_clusters * fl.cluster, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = fl.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, fused_row_kernel, a, fl);
}

}  // namespace pgs
