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
//   softmax numerators in place, then the reference's sequential f32 sum is followed chunk by
//          chunk: every thread folds its consecutive terms with real f32 additions starting
//          from the running value the fold has reached there (estimated by a prefix scan and
//          refined once), so small terms are absorbed exactly where the reference absorbs them
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
    int spill[F_MAXC];
    uint32_t ncand[F_MAXC];
    float true_total[F_MAXC];       // plain sum of the slice's numerators
    double fold1[F_MAXC];           // slice increment of the fold, first estimate
    double fold2[F_MAXC];           // refined
};

// Candidate workspace of CTA 0.  It lives in the slice buffer, which is dead once the sum is known.
struct FusedCand {
    float p[F_MCAP];                // probabilities, arrival order
    uint32_t sid[F_MCAP];           // ids ascending
    float sp[F_MCAP];               // probabilities in id order (zeroed when dropped)
    float rp[F_MCAP];               // probabilities descending (ties: id ascending)
    uint32_t rpos[F_MCAP];          // position in the id-ordered list of the entry at each rank
    SeqSmem seq;
};

// Shared-memory workspace of one CTA (the vocabulary slice follows it).  Regions are reused as
// the row moves through its phases:
//   r_a : id->count table (penalties)             -> merged candidate ids / logits (CTA 0)
//   the slice itself (logits, then numerators)     -> FusedCand (CTA 0)
struct FusedSmem {
    ReduceSmem rs;
    double dscan[NW + 1];
    FusedXchg xchg[2];              // alternates between consecutive rows
    unsigned long long exp_tab[32];
    union {
        struct { uint32_t hkey[F_HASH]; uint32_t hcnt[F_HASH]; } pen;
        struct { uint32_t m_id[F_MCAP]; float m_x[F_MCAP]; } mrg;
    } r_a;
    float tmax_all[F_MAXC * NT];    // every CTA's per-thread maxima
    uint8_t redo_max[NT];
    SelectSmem sel;
    uint32_t cand_id[F_LCAP];
    float cand_x[F_LCAP];
    uint32_t cand_n;
    uint32_t m_n;
    uint32_t n_live, n_keep;
    float bcast_f;
    uint32_t bcast_u;
    int bcast_i;
};

// Optional phase timers (clock64 deltas of thread 0, summed over the rows of each CTA), enabled
// by pointing `prof` at [gridDim.x x 16] counters.
#define PGS_TICK(slot)                                              \
    do {                                                            \
        if (fl.prof && tid == 0) {                                  \
            const long long now_ = clock64();                       \
            fl.prof[blockIdx.x * 16 + (slot)] += now_ - tick_;      \
            tick_ = now_;                                           \
        }                                                           \
    } while (0)

struct FusedLaunch {
    uint32_t cluster;       // CTAs per row
    uint32_t slice_len;     // floats per CTA (multiple of 32)
    uint32_t chunk;         // consecutive floats per thread in the sum pass (odd)
    uint32_t* work_rows;    // rows handed to the general kernel
    uint32_t* work_count;
    long long* prof;
};

// exclusive scan of one double per thread; *total = block sum
__device__ __forceinline__ double block_excl_scan_f64(double v, double* total, double* ws /*NW+1*/) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    double inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        double t = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) ws[w] = inc;
    __syncthreads();
    if (threadIdx.x < 32) {
        double x = ws[threadIdx.x], xi = x;
        for (int o = 1; o < 32; o <<= 1) {
            double t = __shfl_up_sync(FULL, xi, o);
            if (lane >= o) xi += t;
        }
        ws[threadIdx.x] = xi - x;
        if (threadIdx.x == 31) ws[NW] = xi;
    }
    __syncthreads();
    *total = ws[NW];
    return ws[w] + (inc - v);
}

// Exact left fold of n <= 128 shared-memory floats by one warp (values travel by shuffle, so the
// dependent chain is add + shuffle instead of add + shared-memory load).  mode/target as in
// seq_scan; returns the running value, *found = first index where the predicate holds or -1.
__device__ __forceinline__ float warp_fold(const float* v, int n, int mode, float target, int* found) {
    const int lane = threadIdx.x & 31;
    float reg[4];
#pragma unroll
    for (int u = 0; u < 4; u++) reg[u] = (lane + 32 * u < n) ? v[lane + 32 * u] : 0.0f;
    float acc = 0.0f;
    int f = -1;
#pragma unroll
    for (int u = 0; u < 4; u++) {
        for (int l = 0; l < 32; l++) {
            const int j = u * 32 + l;
            if (j >= n || f >= 0) break;
            acc = fadd(acc, __shfl_sync(FULL, reg[u], l));
            if (mode != SEQ_SUM && seq_pred(mode, acc, target)) f = j;
        }
    }
    if (found) *found = f;
    return acc;
}

__device__ __forceinline__ uint32_t load_owner(uint32_t i, uint32_t len) {
    // thread that loaded slice element i: 128-bit groups are dealt round-robin, then the ragged tail
    const uint32_t body = (len / 4) * 4;
    return i < body ? ((i >> 2) & (NT - 1)) : ((i - body) & (NT - 1));
}

__global__ void __launch_bounds__(NT, 1) fused_row_kernel(const RowArgs a, const FusedLaunch fl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FusedSmem& sm = *reinterpret_cast<FusedSmem*>(smem_raw);
    float* X = reinterpret_cast<float*>(smem_raw + ((sizeof(FusedSmem) + 15) & ~size_t(15)));
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x;
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
    long long tick_ = clock64();

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
        const bool writer = rank == 0 && tid == 0;
        if (bad) {
            if (writer) { a.token[row] = 0; a.status[row] = ROW_BAD_PARAM; if (a.drew) a.drew[row] = 0; }
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
            if (writer) fl.work_rows[atomicAdd(fl.work_count, 1u)] = row;
            continue;
        }

        // ------------------------------- load slice: sanity + bitmask AND + per-thread max
        float tmax = -INFINITY;
        int nonfinite = 0;
        sm.redo_max[tid] = 0;
        const uint32_t nq = len / 4;   // 128-bit groups; a ragged tail exists only in the last slice
        auto take4 = [&](uint32_t q, float4 v) {
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
        };
        auto take1 = [&](uint32_t i, float x) {
            nonfinite |= !finite_f(x);
            if (mw && !((__ldg(mw + ((lo + i) >> 5)) >> ((lo + i) & 31)) & 1u)) x = -INFINITY;
            tmax = fmaxf(tmax, x);
            X[i] = x;
        };
        if (a.dtype == 0) {
            const float4* src = (const float4*)(rowp) + lo / 4;
            // four independent 128-bit loads in flight per thread before any of them is consumed
            for (uint32_t q0 = tid; q0 < nq; q0 += 4 * NT) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (q0 + u * NT < nq) v[u] = __ldcs(src + q0 + u * NT);
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (q0 + u * NT < nq) take4(q0 + u * NT, v[u]);
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT) take1(i, __ldcs((const float*)rowp + lo + i));
        } else {
            const uint2* src = (const uint2*)(rowp) + lo / 4;    // 4 bf16 per 8-byte load
            for (uint32_t q0 = tid; q0 < nq; q0 += 4 * NT) {
                uint2 r[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (q0 + u * NT < nq) r[u] = __ldcs(src + q0 + u * NT);
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (q0 + u * NT < nq) {
                        float4 v;   // bf16 -> f32 is a 16-bit shift: exact
                        v.x = __uint_as_float(r[u].x << 16); v.y = __uint_as_float(r[u].x & 0xffff0000u);
                        v.z = __uint_as_float(r[u].y << 16); v.w = __uint_as_float(r[u].y & 0xffff0000u);
                        take4(q0 + u * NT, v);
                    }
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT)
                take1(i, __uint_as_float((uint32_t)__ldcs((const unsigned short*)rowp + lo + i) << 16));
        }
        nonfinite = __syncthreads_or(nonfinite);
        PGS_TICK(0);   // load

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
                    sm.redo_max[load_owner(i, len)] = 1;   // that thread's maximum is stale now
                }
            }
            __syncthreads();
        }
        // ----------------------------------------------------------------- EOS fix
        if (mw && (gflags & 1u) && a.eos >= 0 && (uint32_t)a.eos >= lo && (uint32_t)a.eos < hi && tid == 0 &&
            !finite_f(X[a.eos - lo])) {
            X[a.eos - lo] = 0.0f;
            sm.redo_max[load_owner(a.eos - lo, len)] = 1;
        }
        __syncthreads();
        if (sm.redo_max[tid]) {
            tmax = -INFINITY;
            for (uint32_t q = tid; q < nq; q += NT) {
                const float4 v = ((const float4*)X)[q];
                tmax = fmaxf(tmax, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT) tmax = fmaxf(tmax, X[i]);
        }
        PGS_TICK(1);   // penalties

        // ------------------------------------------------- slice max / argmax, lowest id
        // the winning thread(s) look up the lowest index holding the block maximum
        unsigned long long best = block_max_u64((unsigned long long)order_key(tmax) << 32, sm.rs);
        const uint32_t bkey = (uint32_t)(best >> 32);
        best = 0ull;
        if (bkey && order_key(tmax) == bkey) {
            const float bval = key_to_float(bkey);
            uint32_t first = 0xffffffffu;
            for (uint32_t q = tid; q < nq && first == 0xffffffffu; q += NT) {
                const float4 v = ((const float4*)X)[q];
                if (v.x == bval) first = q * 4;
                else if (v.y == bval) first = q * 4 + 1;
                else if (v.z == bval) first = q * 4 + 2;
                else if (v.w == bval) first = q * 4 + 3;
            }
            for (uint32_t i = nq * 4 + tid; i < len && first == 0xffffffffu; i += NT)
                if (X[i] == bval) first = i;
            if (first != 0xffffffffu)
                best = ((unsigned long long)bkey << 32) | (unsigned long long)(0xffffffffu - (lo + first));
        }
        if (bkey) best = block_max_u64(best, sm.rs);
        PGS_TICK(2);   // argmax
        // ------------------------------------------------ cluster exchange #1
        for (uint32_t r = tid; r < C; r += NT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].best[rank] = best;
            peer->xchg[pbuf].nonfinite[rank] = nonfinite;
            peer->xchg[pbuf].spill[rank] = spill;
        }
        if (!greedy) {
            for (uint32_t r = 0; r < C; r++) cluster.map_shared_rank(&sm, r)->tmax_all[rank * NT + tid] = tmax;
        }
        cluster.sync();
        parity ^= 1u;
        PGS_TICK(3);   // sync 1
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
        const uint32_t kk = radix_select_kth([&](int i) { return order_key(sm.tmax_all[i]); }, (int)(C * NT),
                                             top_k, sm.sel, sm.rs);
        float cut = -INFINITY;
        if (kk) {
            const float bound = key_to_float(kk);
            // every logit whose probability could still tie with the k-th one stays above the cut
            const float delta = 4.8e-7f * (fabsf(m - bound) + 4.0f * t) + 4.8e-7f * (fabsf(bound) + fabsf(m));
            cut = bound - delta;
        }
        PGS_TICK(4);   // select
        if (tid == 0) sm.cand_n = 0;
        __syncthreads();
        {
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
        PGS_TICK(5);   // gather

        // --------------- softmax numerators in place (hardware exp2) + per-thread chunk sums
        const float scale = 1.4426950408889634f / t;
        const uint32_t L = fl.chunk;
        const uint32_t c0 = min(len, tid * L), c1 = min(len, c0 + L);
        float csum = 0.0f;
        for (uint32_t i = c0; i < c1; i++) {
            const float e = ex2_approx((X[i] - m) * scale);   // masked entries are -inf: 2^-inf = +0
            X[i] = e;
            csum += e;
        }
        double dtot;
        const double pre0 = block_excl_scan_f64((double)csum, &dtot, sm.dscan);
        PGS_TICK(6);   // exp pass
        // ------------------------------------------------ cluster exchange #2
        for (uint32_t r = tid; r < C; r += NT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].ncand[rank] = my_n;
            peer->xchg[pbuf].true_total[rank] = (float)dtot;
        }
        cluster.sync();
        PGS_TICK(7);   // sync 2
        uint32_t cand_off = 0, cand_total = 0;
        double before0 = 0.0;
        bool overflow = false;
        for (uint32_t r = 0; r < C; r++) {
            if (r < rank) { cand_off += xc.ncand[r]; before0 += (double)xc.true_total[r]; }
            cand_total += xc.ncand[r];
            overflow |= xc.ncand[r] > (uint32_t)F_LCAP;
        }
        overflow |= cand_total > (uint32_t)F_MCAP;
        if (overflow) {   // identical decision in every CTA
            if (writer) fl.work_rows[atomicAdd(fl.work_count, 1u)] = row;
            continue;
        }
        // candidates -> CTA 0 (lands before exchange #4)
        {
            FusedSmem* root = cluster.map_shared_rank(&sm, 0);
            for (uint32_t j = tid; j < my_n; j += NT) {
                root->r_a.mrg.m_id[cand_off + j] = sm.cand_id[j];
                root->r_a.mrg.m_x[cand_off + j] = sm.cand_x[j];
            }
            if (writer) sm.m_n = cand_total;
        }
        // ---------- the sequential fold, chunk by chunk: first from the plain prefix sums ...
        const float start0 = (float)(before0 + pre0);
        float acc = start0;
        for (uint32_t i = c0; i < c1; i++) acc = fadd(acc, X[i]);
        double inc1 = (double)acc - (double)start0;
        double tot1;
        const double pre1 = block_excl_scan_f64(inc1, &tot1, sm.dscan);
        PGS_TICK(8);   // fold 1
        for (uint32_t r = tid; r < C; r += NT) cluster.map_shared_rank(&sm, r)->xchg[pbuf].fold1[rank] = tot1;
        cluster.sync();   // exchange #3
        double before1 = 0.0;
        for (uint32_t r = 0; r < rank; r++) before1 += xc.fold1[r];
        // ... then once more from the running values that first pass implies
        const float start1 = (float)(before1 + pre1);
        acc = start1;
        for (uint32_t i = c0; i < c1; i++) acc = fadd(acc, X[i]);
        double inc2 = (double)acc - (double)start1;
        double tot2;
        block_excl_scan_f64(inc2, &tot2, sm.dscan);
        if (tid == 0) cluster.map_shared_rank(&sm, 0)->xchg[pbuf].fold2[rank] = tot2;
        cluster.sync();   // exchange #4
        PGS_TICK(9);   // fold 2
        if (rank != 0) continue;

        // ------------------------------------------ CTA 0: the reference's rule on the candidates
        double s2 = 0.0;
        for (uint32_t r = 0; r < C; r++) s2 += xc.fold2[r];
        const float S = (float)s2;
        const uint32_t n = sm.m_n;
        const bool norm = S > 1e-9f;
        FusedCand& cd = *reinterpret_cast<FusedCand*>(X);
        const uint32_t* m_id = sm.r_a.mrg.m_id;
        for (uint32_t j = tid; j < n; j += NT) {
            const float e = softmax_num(sm.r_a.mrg.m_x[j], m, t, tab);   // exact expf for candidates
            cd.p[j] = norm ? fdiv(e, S) : e;
        }
        __syncthreads();
        // rank every candidate by id and by (probability descending, id ascending)
        for (uint32_t j = tid; j < n; j += NT) {
            const uint32_t idj = m_id[j];
            const float pj = cd.p[j];
            uint32_t r_id = 0, r_p = 0;
            for (uint32_t o = 0; o < n; o++) {
                const uint32_t ido = m_id[o];
                const float po = cd.p[o];
                r_id += ido < idj;
                r_p += (po > pj) || (po == pj && ido < idj);
            }
            cd.sid[r_id] = idj;
            cd.sp[r_id] = pj;
            cd.rp[r_p] = pj;
            cd.rpos[r_p] = r_id;
        }
        if (tid == 0) { sm.n_live = 0; }
        __syncthreads();
        // top-k: every tie at the k-th probability survives (sampler.rs:116-128); zeros never matter
        {
            const float thr = top_k <= n ? cd.rp[top_k - 1] : 0.0f;
            for (uint32_t j = tid; j < n; j += NT) {
                const bool live = cd.rp[j] >= thr && cd.rp[j] > 0.0f;
                const bool next_live = j + 1 < n && cd.rp[j + 1] >= thr && cd.rp[j + 1] > 0.0f;
                if (live && !next_live) sm.n_live = j + 1;
            }
        }
        __syncthreads();
        const uint32_t n_live = sm.n_live;
        // top-p walk in ranked order (sampler.rs:130-150)
        uint32_t keep = n_live;
        if (use_p && n_live > 0) {
            int found = -1;
            if (n_live <= 128) {
                if (tid < 32) {
                    warp_fold(cd.rp, (int)n_live, SEQ_FIND_GE, top_p, &found);
                    if (tid == 0) sm.bcast_i = found;
                }
                __syncthreads();
                found = sm.bcast_i;
            } else {
                seq_scan([&](int j) { return cd.rp[j]; }, (int)n_live, 0.0f, SEQ_FIND_GE, top_p, &found, cd.seq, sm.rs);
            }
            if (found >= 0) keep = (uint32_t)found + 1;
        }
        for (uint32_t j = keep + tid; j < n; j += NT) cd.sp[cd.rpos[j]] = 0.0f;
        __syncthreads();
        // total and inverse-CDF pick in id order (sampler.rs:40-55)
        float total;
        int pick = -1;
        if (n <= 128) {
            if (tid < 32) {
                const float tt = warp_fold(cd.sp, (int)n, SEQ_SUM, 0.0f, nullptr);
                int f = -1;
                if (tt > 1e-9f) warp_fold(cd.sp, (int)n, SEQ_FIND_GT, fmul(u01, tt), &f);
                if (tid == 0) { sm.bcast_f = tt; sm.bcast_i = f; }
            }
            __syncthreads();
            total = sm.bcast_f;
            pick = sm.bcast_i;
        } else {
            total = seq_scan([&](int j) { return cd.sp[j]; }, (int)n, 0.0f, SEQ_SUM, 0.0f, nullptr, cd.seq, sm.rs);
            if (total > 1e-9f)
                seq_scan([&](int j) { return cd.sp[j]; }, (int)n, 0.0f, SEQ_FIND_GT, fmul(u01, total), &pick, cd.seq,
                         sm.rs);
        }
        if (tid == 0) {
            uint32_t token = amax;
            int drew = 0;
            if (total > 1e-9f) { token = pick >= 0 ? cd.sid[pick] : V - 1; drew = 1; }
            a.token[row] = token; a.status[row] = status;
            if (a.drew) a.drew[row] = (uint8_t)drew;
            if (a.argmax) a.argmax[row] = amax;
            if (a.row_max) a.row_max[row] = m;
            if (a.sumexp) a.sumexp[row] = S;
            if (a.total) a.total[row] = total;
        }
        PGS_TICK(10);  // candidates
        if (a.n_kept || a.dump_ids || a.dump_probs) {   // diagnostics: the kept set in id order
            uint32_t done = 0;
            for (uint32_t base = 0; base < n; base += NT) {
                const uint32_t j = base + tid;
                const uint32_t kept = (j < n && cd.sp[j] > 0.0f) ? 1u : 0u;
                uint32_t tot;
                const uint32_t at = done + block_excl_scan_u32(kept, &tot, sm.rs);
                if (kept && at < a.dump_cap) {
                    if (a.dump_ids) a.dump_ids[(size_t)row * a.dump_cap + at] = cd.sid[j];
                    if (a.dump_probs) a.dump_probs[(size_t)row * a.dump_cap + at] = cd.sp[j];
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

// the slice buffer doubles as CTA 0's candidate workspace
size_t fused_smem_bytes(uint32_t slice_len) {
    const size_t need = (sizeof(FusedCand) + 3) / 4;
    const size_t floats = slice_len > need ? slice_len : need;
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
