// Fused cluster kernel: the hot path of the sampler.
//
// One thread-block cluster owns one batch row.  The row is read from HBM exactly once -- bulk
// asynchronous copies (TMA, no multicast) for f32, 64-bit coalesced loads for bf16 -- into the
// distributed shared memory of the cluster (each CTA keeps a
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
// A stochastic row leaves this kernel as a record (max, partial folds, candidate list); the
// finish kernel (pgs_finish.cu) applies the reference's top-k / top-p / CDF rule to it.
// Rows this kernel cannot hold (top-k off or > 1024, more candidates than its buffers, too many
// distinct history ids in one slice, unaligned rows) are appended to a work list that the
// general row kernel processes afterwards.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "pgs_args.cuh"
#include "pgs_block.cuh"
#include "pgs_fused.cuh"

namespace cg = cooperative_groups;

namespace pgs {

struct FusedXchg {                  // peers write their slot through DSMEM
    unsigned long long best[F_MAXC];
    int nonfinite[F_MAXC];
    int spill[F_MAXC];
    uint32_t ncand[F_MAXC];
    float true_total[F_MAXC];       // plain sum of the slice's numerators
    double fold1[F_MAXC];           // slice increment of the fold, first estimate
};

// Shared-memory workspace of one CTA (the vocabulary slice follows it).
struct FusedSmem {
    ReduceSmem rs;
    double dscan[NW + 1];
    FusedXchg xchg[2];              // alternates between consecutive rows
    struct { uint32_t hkey[F_HASH]; uint32_t hcnt[F_HASH]; } pen;
    float tmax_all[F_MAXC * NT];    // every CTA's per-thread maxima
    uint8_t redo_max[NT];
    SelectSmem sel;
    uint32_t cand_id[F_LCAP];
    float cand_x[F_LCAP];
    uint32_t cand_n;
    unsigned long long load_bar[8]; // one mbarrier per 32 KB piece of the bulk copy that fills the slice
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

// block sum of one double per thread
__device__ __forceinline__ double block_sum_f64(double v, double* ws /*NW+1*/) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        double w = ws[threadIdx.x];
        for (int o = 16; o; o >>= 1) w += __shfl_xor_sync(FULL, w, o);
        if (threadIdx.x == 0) ws[NW] = w;
    }
    __syncthreads();
    return ws[NW];
}

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

// ---- bulk asynchronous copy (TMA, no tensor map, no multicast) global -> this CTA's shared memory
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Bounded wait for phase `parity` of the barrier: false when the copy has not landed after 2^16 tries
// (each try may park the thread for up to 20 us, so the bound is about a second).
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < (1u << 16); spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)   // let the hardware park the thread for up to 20 us per try
            : "memory");
        if (ok) return true;
    }
    return false;
}
constexpr uint32_t TMA_PIECE = 32768;   // bytes per bulk copy

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
    uint32_t parity = 0;
    uint32_t load_phase = 0;        // parity of the next completion of load_bar
    bool poisoned = false;          // a bulk copy never landed: later rows of this CTA report that too
    if (tid == 0) {
        for (int b = 0; b < 8; b++) mbar_init(&sm.load_bar[b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
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
            if (writer) { a.token[row] = 0; a.status[row] = ROW_BAD_PARAM; if (a.drew) a.drew[row] = 0; fl.recs[row].kind = 0; }
            continue;
        }
        const bool greedy = temp < 1e-5f;
        const bool use_k = top_k != 0u && top_k < V;
        // rows this kernel does not serve go to the general kernel (decided identically by every CTA)
        const char* rowp = (const char*)a.logits + (size_t)row * a.row_stride * (a.dtype == 0 ? 4 : 2);
        const bool aligned = (((uintptr_t)rowp & 15) == 0);
        const bool defer = !aligned || (!greedy && (!use_k || top_k > (uint32_t)F_KMAX));
        if (defer) {
            if (writer) { fl.work_rows[atomicAdd(fl.work_count, 1u)] = row; fl.recs[row].kind = 0; }
            continue;
        }

        // ------------------------------- load slice: sanity + bitmask AND + per-thread max
        float tmax = -INFINITY;
        int nonfinite = 0;
        uint32_t tq = 0;   // slice index of the 128-bit group (or, flagged, the tail element) that holds tmax
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
            const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
            if (m4 > tmax) { tmax = m4; tq = q * 4; }
            ((float4*)X)[q] = v;
        };
        auto take1 = [&](uint32_t i, float x) {
            nonfinite |= !finite_f(x);
            if (mw && !((__ldg(mw + ((lo + i) >> 5)) >> ((lo + i) & 31)) & 1u)) x = -INFINITY;
            if (x > tmax) { tmax = x; tq = i | 0x80000000u; }
            X[i] = x;
        };
        // history ids of this slice -> id->count table; runs while the copy below is in flight
        const bool do_fp = !(fabsf(freq) < 1e-6f && fabsf(pres) < 1e-6f);
        const bool do_pres = fabsf(pres) > 1e-6f;
        const bool do_rep = rep != 1.0f;
        const bool pen = nh > 0 && (do_fp || do_rep);
        int spill = 0;
        auto index_history = [&]() {
            for (int s = tid; s < F_HASH; s += NT) { sm.pen.hkey[s] = 0xffffffffu; sm.pen.hcnt[s] = 0u; }
            __syncthreads();
            for (uint32_t j = tid; j < nh; j += NT) {
                const uint32_t id = __ldg(a.hist_ids + h0 + j);
                if (id < lo || id >= hi) continue;
                uint32_t s = (id * 2654435761u) >> 21;   // 11 bits
                bool placed = false;
                for (int probe = 0; probe < 64; probe++) {
                    const uint32_t prev = atomicCAS(&sm.pen.hkey[s], 0xffffffffu, id);
                    if (prev == 0xffffffffu || prev == id) { atomicAdd(&sm.pen.hcnt[s], 1u); placed = true; break; }
                    s = (s + 1) & (F_HASH - 1);
                }
                if (!placed) spill = 1;
            }
        };
        if (a.dtype == 0) {
            // f32 rows: one thread streams the slice into shared memory with bulk asynchronous copies
            // (32 KB pieces, one mbarrier each); every warp then checks / masks / maximises each piece
            // as soon as it has landed.  (Prefetching the next row's slice into L2 was measured and
            // bought nothing: the copy is not what limits this kernel.)
            const char* gsrc = rowp + (size_t)lo * 4;
            const uint32_t body = nq * 16;
            const uint32_t n_pieces = (body + TMA_PIECE - 1) / TMA_PIECE;   // <= 8 for any slice that fits
            if (tid == 0) {
                if (body && !poisoned) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier generic writes to X
                    for (uint32_t pc = 0; pc < n_pieces; pc++) {
                        const uint32_t off = pc * TMA_PIECE, bytes = min(TMA_PIECE, body - off);
                        mbar_expect_tx(&sm.load_bar[pc], bytes);
                        bulk_g2s((char*)X + off, gsrc + off, bytes, &sm.load_bar[pc]);
                    }
                }
            }
            if (pen) index_history();
            PGS_TICK(11);  // copy issued, history indexed
            float poison = 0.0f;   // 0 * v is NaN exactly when v is infinite or NaN, and NaN sticks
            for (uint32_t pc = 0; pc < n_pieces; pc++) {
                // every warp waits for the piece on its own: one lane polls (bounded), the rest follow
                int ok = 1;
                if (!poisoned && (tid & 31) == 0) ok = mbar_wait(&sm.load_bar[pc], load_phase) ? 1 : 0;
                ok = __shfl_sync(FULL, ok, 0);
                if (!ok) poisoned = true;
                if (poisoned) continue;
                const uint32_t q_end = min(nq, (pc + 1) * (TMA_PIECE / 16));
                for (uint32_t q = pc * (TMA_PIECE / 16) + tid; q < q_end; q += NT) {
                    float4 v = ((const float4*)X)[q];
                    poison = __fmaf_rn(v.x, 0.0f, poison); poison = __fmaf_rn(v.y, 0.0f, poison);
                    poison = __fmaf_rn(v.z, 0.0f, poison); poison = __fmaf_rn(v.w, 0.0f, poison);
                    if (mw) {
                        const uint32_t bits = __ldg(mw + ((lo >> 5) + (q >> 3))) >> ((q & 7) * 4);
                        if (!(bits & 1u)) v.x = -INFINITY;
                        if (!(bits & 2u)) v.y = -INFINITY;
                        if (!(bits & 4u)) v.z = -INFINITY;
                        if (!(bits & 8u)) v.w = -INFINITY;
                        ((float4*)X)[q] = v;
                    }
                    const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                    if (m4 > tmax) { tmax = m4; tq = q * 4; }
                }
            }
            if (n_pieces) load_phase ^= 1u;
            if (poisoned) nonfinite = 2;   // reported as a load timeout after the exchange
            nonfinite |= poison != poison;
            if (!poisoned)
                for (uint32_t i = nq * 4 + tid; i < len; i += NT) take1(i, __ldcs((const float*)rowp + lo + i));
        } else {
            if (pen) index_history();
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
        if (pen && !nonfinite) {
            spill = __syncthreads_or(spill);
            if (!spill) {
                for (int s = tid; s < F_HASH; s += NT) {
                    const uint32_t id = sm.pen.hkey[s];
                    if (id == 0xffffffffu) continue;
                    const uint32_t i = id - lo;
                    float x = X[i];
                    if (do_rep) x = x > 0.0f ? fdiv(x, rep) : fmul(x, rep);
                    if (do_fp) {
                        x = fsub(x, fmul(freq, (float)sm.pen.hcnt[s]));
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
                const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                if (m4 > tmax) { tmax = m4; tq = q * 4; }
            }
            for (uint32_t i = nq * 4 + tid; i < len; i += NT)
                if (X[i] > tmax) { tmax = X[i]; tq = i | 0x80000000u; }
        }
        PGS_TICK(1);   // penalties

        // ------------------------------------------------- slice max / argmax, lowest id
        // each thread knows where its maximum first occurs (its groups are visited in ascending order)
        unsigned long long best = 0ull;
        if (tmax > -INFINITY) {
            uint32_t idx = tq & 0x7fffffffu;
            if (!(tq & 0x80000000u)) {
                const float4 v = *reinterpret_cast<const float4*>(X + idx);
                idx += v.x == tmax ? 0u : v.y == tmax ? 1u : v.z == tmax ? 2u : 3u;
            }
            best = ((unsigned long long)order_key(tmax) << 32) | (unsigned long long)(0xffffffffu - (lo + idx));
        }
        best = block_max_u64(best, sm.rs);
        PGS_TICK(2);   // argmax
        // ------------------------------------------------ cluster exchange #1
        for (uint32_t r = tid; r < C; r += NT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].best[rank] = best;
            peer->xchg[pbuf].nonfinite[rank] = nonfinite;
            peer->xchg[pbuf].spill[rank] = spill;
        }
        // material for the top-k bound: the 32*C warp maxima when there are comfortably more warps than
        // top_k, else all NT*C thread maxima
        const bool warp_bound = !greedy && 2u * top_k <= C * NW;
        if (!greedy) {
            if (warp_bound) {
                float wmax = tmax;
                for (int o = 16; o; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(FULL, wmax, o));
                if ((tid & 31) < (int)C)
                    cluster.map_shared_rank(&sm, tid & 31)->tmax_all[rank * NW + (tid >> 5)] = wmax;
            } else {
                for (uint32_t r = 0; r < C; r++) cluster.map_shared_rank(&sm, r)->tmax_all[rank * NT + tid] = tmax;
            }
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
            if (writer) { a.token[row] = 0; a.status[row] = (any_nonfinite & 2) ? ROW_LOAD_TIMEOUT : ROW_NONFINITE; if (a.drew) a.drew[row] = 0; fl.recs[row].kind = 0; }
            continue;
        }
        if (gflags & 2u) {
            if (writer) { a.token[row] = 0; a.status[row] = ROW_DEAD; if (a.drew) a.drew[row] = 0; fl.recs[row].kind = 0; }
            continue;
        }
        if (any_spill) {
            if (writer) { fl.work_rows[atomicAdd(fl.work_count, 1u)] = row; fl.recs[row].kind = 0; }
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
                fl.recs[row].kind = 0;
            }
            continue;
        }

        // -------------------------------- top-k bound: k-th largest per-thread maximum
        // The C*NT maxima are spread over 2048 equal-width buckets between their smallest finite
        // value and the row maximum (a monotone map), the bucket holding the k-th largest is found
        // from the histogram, and the exact value is picked among that bucket's few members.
        const float t = fmaxf(temp, 1e-9f);
        float cut = -INFINITY;
        if (warp_bound) {
            // k-th largest of the 32*C warp maxima: thread j ranks maximum j against all others
            const uint32_t nvw = C * NW;
            if (tid == 0) sm.sel.hist[0] = 0u;
            __syncthreads();
            if ((uint32_t)tid < nvw) {
                const float v = sm.tmax_all[tid];
                uint32_t gt = 0, ge = 0;
                for (uint32_t o = 0; o < nvw; o++) { const float u = sm.tmax_all[o]; gt += u > v; ge += u >= v; }
                if (finite_f(v) && gt < top_k && top_k <= ge) sm.sel.hist[0] = order_key(v);
            }
            __syncthreads();
            const uint32_t kk = sm.sel.hist[0];
            if (kk) {
                const float bound = key_to_float(kk);
                const float delta = 4.8e-7f * (fabsf(m - bound) + 4.0f * t) + 4.8e-7f * (fabsf(bound) + fabsf(m));
                cut = bound - delta;
            }
        } else {
            const uint32_t nv = C * NT;
            uint32_t fin = 0;
            unsigned long long inv_min = 0ull;
            for (uint32_t i = tid; i < nv; i += NT) {
                const uint32_t key = order_key(sm.tmax_all[i]);
                if (key) { fin++; const unsigned long long iv = 0xffffffffull - key; inv_min = iv > inv_min ? iv : inv_min; }
            }
            const uint32_t n_fin = block_sum_u32(fin, sm.rs);
            inv_min = block_max_u64(inv_min, sm.rs);
            if (n_fin >= top_k) {
                const float lo_v = key_to_float((uint32_t)(0xffffffffull - inv_min));
                const float sc = m > lo_v ? 2047.0f / (m - lo_v) : 0.0f;
                for (int bkt = tid; bkt < 2048; bkt += NT) sm.sel.hist[bkt] = 0u;
                if (tid == 0) { sm.sel.prefix = 0xffffffffu; sm.sel.k = 0u; sm.cand_n = 0u; }
                __syncthreads();
                for (uint32_t i = tid; i < nv; i += NT) {
                    const float v = sm.tmax_all[i];
                    if (finite_f(v)) atomicAdd(&sm.sel.hist[min(2047u, (uint32_t)((v - lo_v) * sc))], 1u);
                }
                __syncthreads();
                {
                    // walk from the top bucket down: warp w owns buckets 2047-64w .. 2047-64w-63 (two per lane)
                    const int w = tid >> 5, lane = tid & 31;
                    const uint32_t h0v = sm.sel.hist[2047 - 64 * w - 2 * lane];
                    const uint32_t h1v = sm.sel.hist[2047 - 64 * w - 2 * lane - 1];
                    uint32_t inc = h0v + h1v;
                    for (int o = 1; o < 32; o <<= 1) {
                        const uint32_t up = __shfl_up_sync(FULL, inc, o);
                        if (lane >= o) inc += up;
                    }
                    if (lane == 31) sm.rs.u[w] = inc;
                    __syncthreads();
                    uint32_t above = 0;
                    for (int ww = 0; ww < w; ww++) above += sm.rs.u[ww];
                    const uint32_t before_me = above + inc - h0v - h1v;   // maxima in higher buckets
                    if (before_me < top_k && before_me + h0v >= top_k) {
                        sm.sel.prefix = 2047 - 64 * w - 2 * lane; sm.sel.k = top_k - before_me;
                    } else if (before_me + h0v < top_k && before_me + h0v + h1v >= top_k) {
                        sm.sel.prefix = 2047 - 64 * w - 2 * lane - 1; sm.sel.k = top_k - before_me - h0v;
                    }
                }
                __syncthreads();
                const uint32_t bsel = sm.sel.prefix, ksel = sm.sel.k;
                // members of the selected bucket -> cand_x (reused as scratch, at most F_LCAP of them)
                for (uint32_t i = tid; i < nv; i += NT) {
                    const float v = sm.tmax_all[i];
                    if (finite_f(v) && min(2047u, (uint32_t)((v - lo_v) * sc)) == bsel) {
                        const uint32_t at = atomicAdd(&sm.cand_n, 1u);
                        if (at < (uint32_t)F_LCAP) sm.cand_x[at] = v;
                    }
                }
                if (tid == 0) sm.sel.hist[0] = 0u;   // reused: order key of the bound
                __syncthreads();
                const uint32_t nm = sm.cand_n;
                if (nm <= (uint32_t)F_LCAP) {
                    for (uint32_t j = tid; j < nm; j += NT) {
                        const float v = sm.cand_x[j];
                        uint32_t gt = 0, ge = 0;
                        for (uint32_t o = 0; o < nm; o++) { gt += sm.cand_x[o] > v; ge += sm.cand_x[o] >= v; }
                        if (gt < ksel && ksel <= ge) sm.sel.hist[0] = order_key(v);
                    }
                } else {
                    // too many equal-bucket maxima: any member bounds the k-th largest from below
                    if (tid == 0) sm.sel.hist[0] = order_key(lo_v);
                }
                __syncthreads();
                const uint32_t kk = sm.sel.hist[0];
                if (kk) {
                    const float bound = key_to_float(kk);
                    // every logit whose probability could still tie with the k-th one stays above the cut
                    const float delta = 4.8e-7f * (fabsf(m - bound) + 4.0f * t) + 4.8e-7f * (fabsf(bound) + fabsf(m));
                    cut = bound - delta;
                }
            }
        }
        PGS_TICK(4);   // select
        __syncthreads();
        if (tid == 0) sm.cand_n = 0;
        __syncthreads();
        // ---- one pass in chunk order: collect the candidates, then overwrite each logit with its
        //      softmax numerator (hardware exp2) and accumulate the plain chunk sum
        // log2(e) / t as a two-float sum, so that the exponent's argument carries no systematic error
        const double scale_d = 1.4426950408889634 / (double)t;
        const float s_hi = (float)scale_d, s_lo2 = (float)((scale_d - (double)(float)scale_d) * 0.6931471805599453);
        const float cut_f = fmaxf(cut, -3.4e38f);   // masked entries (-inf) are never candidates
        const uint32_t L = fl.chunk;   // 4 * odd: 128-bit shared-memory accesses of a warp do not collide
        const uint32_t c0 = min(len, tid * L), c1 = min(len, c0 + L);
        const uint32_t c1b = c0 + ((c1 - c0) & ~3u);   // whole 128-bit groups; a remainder only at the ragged end
        float csum = 0.0f;
        // candidate test, then 2^((x - m) * log2(e) / t): hardware exp2 of the product with the rounded
        // scale, times (1 + ln2 * the part of the scale that rounding dropped), which removes the
        // systematic error; the clamp keeps masked entries (-inf) finite so that they come out as +0
        auto numerator = [&](float x, uint32_t i) -> float {
            if (x >= cut_f) {
                const uint32_t at = atomicAdd(&sm.cand_n, 1u);
                if (at < (uint32_t)F_LCAP) { sm.cand_id[at] = lo + i; sm.cand_x[at] = x; }
            }
            const float a_ = fmaxf(fsub(x, m), -1e30f);
            const float e2 = ex2_approx(fmul(a_, s_hi));
            return __fmaf_rn(e2, fmul(a_, s_lo2), e2);
        };
        for (uint32_t i = c0; i < c1b; i += 4) {
            float4 v = *reinterpret_cast<const float4*>(X + i);
            v.x = numerator(v.x, i); v.y = numerator(v.y, i + 1); v.z = numerator(v.z, i + 2); v.w = numerator(v.w, i + 3);
            *reinterpret_cast<float4*>(X + i) = v;
            csum += (v.x + v.y) + (v.z + v.w);
        }
        for (uint32_t i = c1b; i < c1; i++) { const float e = numerator(X[i], i); X[i] = e; csum += e; }
        __syncthreads();
        const uint32_t my_n = sm.cand_n;
        PGS_TICK(5);   // gather + exp
        const float pre0 = block_excl_scan_f32(csum, sm.rs);
        if (tid == NT - 1) sm.dscan[0] = (double)pre0 + (double)csum;
        __syncthreads();
        const double dtot = sm.dscan[0];
        PGS_TICK(6);   // scan
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
            if (writer) { fl.work_rows[atomicAdd(fl.work_count, 1u)] = row; fl.recs[row].kind = 0; }
            continue;
        }
        // candidates -> global memory, in slice order, for the finish kernel
        for (uint32_t j = tid; j < my_n; j += NT) {
            fl.cand_id[(size_t)row * F_MCAP + cand_off + j] = sm.cand_id[j];
            fl.cand_x[(size_t)row * F_MCAP + cand_off + j] = sm.cand_x[j];
        }
        // ---------- the sequential fold, chunk by chunk: first from the plain prefix sums ...
        const float start0 = (float)before0 + pre0;
        auto fold_chunk = [&](float acc_) -> float {
            for (uint32_t i = c0; i < c1b; i += 4) {
                const float4 v = *reinterpret_cast<const float4*>(X + i);
                acc_ = fadd(fadd(fadd(fadd(acc_, v.x), v.y), v.z), v.w);
            }
            for (uint32_t i = c1b; i < c1; i++) acc_ = fadd(acc_, X[i]);
            return acc_;
        };
        float acc = fold_chunk(start0);
        const float inc1 = fsub(acc, start0);   // exact: both ends lie within a factor two or the chunk is re-folded
        const float pre1 = block_excl_scan_f32(inc1, sm.rs);
        __syncthreads();
        if (tid == NT - 1) sm.dscan[0] = (double)pre1 + (double)inc1;
        __syncthreads();
        const double tot1 = sm.dscan[0];
        PGS_TICK(8);   // fold 1
        for (uint32_t r = tid; r < C; r += NT) cluster.map_shared_rank(&sm, r)->xchg[pbuf].fold1[rank] = tot1;
        cluster.sync();   // exchange #3
        double before1 = 0.0;
        for (uint32_t r = 0; r < rank; r++) before1 += xc.fold1[r];
        // ... then once more, for the chunks whose binade that first pass got wrong or crossed
        const float start1 = (float)before1 + pre1;
        const uint32_t e0 = f2u(start0) & 0x7f800000u;
        double inc2 = (double)inc1;
        if ((f2u(start1) & 0x7f800000u) != e0 || (f2u(acc) & 0x7f800000u) != e0) {
            acc = fold_chunk(start1);
            inc2 = (double)acc - (double)start1;
        }
        for (int o = 16; o; o >>= 1) inc2 += __shfl_xor_sync(FULL, inc2, o);
        if ((tid & 31) == 0) fl.recs[row].part[rank * NW + (tid >> 5)] = inc2;   // the finish kernel adds the warps up
        if (writer) {
            RowRec& rec = fl.recs[row];
            rec.kind = 1; rec.n_cand = cand_total; rec.amax = amax; rec.status = status;
            rec.m = m; rec.t = t; rec.n_parts = C * NW;
        }
        PGS_TICK(9);   // fold 2
    }
    // no CTA may exit while a peer can still write into its shared memory
    cluster.sync();
}

size_t fused_smem_bytes(uint32_t slice_len) {
    return ((sizeof(FusedSmem) + 15) & ~size_t(15)) + (size_t)slice_len * sizeof(float);
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
