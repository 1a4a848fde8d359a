// Fused cluster kernel: the hot path of the sampler.
//
// One thread-block cluster (1 to 8 CTAs of 1024 threads, one CTA per SM) owns one batch row at a time and
// walks through its share of the batch.  The row is read from HBM exactly once -- bulk asynchronous copies
// (TMA, no multicast) for f32, 64-bit coalesced loads for bf16 -- into the distributed shared memory of the
// cluster (each CTA keeps a contiguous slice of the vocabulary as f32), and every later step of the chain
// (pagoda/src/engine.rs:1286-1314, pagoda/src/sampler.rs:28-150) works on that copy.  Rows in flight are
// bounded by shared memory (a row occupies its cluster from the copy to the last fold), so the host picks
// the cluster size that minimises waves x row time for the batch (3 CTAs at 256 x 151936 f32).
//
// Per row:
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

// The kernel runs FNT threads per CTA.  (Measured alternatives on 256 x 151936: 512 threads with two CTAs
// per SM and clusters of 8, 141 us; 256 threads, 146 us; 1024 threads with clusters of 4, 135 us, of 3,
// 128 us.  Warp collectives -- shuffles, votes, redux -- run at about one per cycle and SM and cost 30 to
// 130 cycles of latency each here, function calls cost more than the code they save, and straight-line code
// that is executed once per row runs at 20 to 30 cycles per instruction and warp, so cold loops stay rolled.)
// The per-thread maxima that bound the top-k threshold are kept for FVT "virtual threads": 128-bit group q
// of a slice belongs to virtual thread q mod FVT, and a real thread plays VG = FVT / FNT of them (groups q
// with q mod FVT = g * FNT + tid, g < VG).
constexpr int FNT = 1024;
constexpr int FNW = FNT / 32;
constexpr int FVT = 1024;
constexpr int FVW = FVT / 32;
constexpr int VG = FVT / FNT;
static_assert(F_MAXC * FVW <= 256, "a warp-maximum slot number fits the low 8 bits of its key");
static_assert(VG == 1 || VG == 2 || VG == 4, "the bf16 loader assumes VG divides 4");

struct FusedXchg {                  // peers write their slot through DSMEM
    unsigned long long best[F_MAXC];
    int flags[F_MAXC];              // non-finite / load-timeout bits, bit 8 = history table overflow
    uint32_t ncand[F_MAXC];
    float true_total[F_MAXC];       // plain sum of the slice's numerators
    double fold1[F_MAXC];           // slice increment of the fold, first estimate
};

// Everything the kernel needs to know about a row, read and validated by one thread while the CTA still works
// on the row before it.
struct RowCtl {
    const char* rowp;       // first logit of the row
    const uint32_t* mw;     // grammar mask words of the row's state, or null
    float temp, freq, pres, rep;
    float s_hi, s_lo;       // log2(e) / max(temp, 1e-9) as a two-float sum with s_lo > 0
    uint32_t top_k, gflags, h0, nh;
    uint32_t kind;          // 0 serve, 1 bad parameters, 2 defer to the general kernel
};

constexpr int F_NB = 1024;          // buckets of the per-thread-maxima histogram
static_assert(F_NB % FNT == 0, "every thread walks F_NB / FNT buckets");
struct BoundSmem { uint32_t hist[F_NB]; uint32_t prefix, k; };

// Shared-memory workspace of one CTA.  Two more regions follow it: the exchange region -- every CTA's
// per-thread (or per-warp) maxima, C * FVT floats, written by the peers; once the top-k bound is known the
// same space holds this slice's candidate list (peers only write the next row's maxima after this row's last
// cluster barrier) -- and then the vocabulary slice.
struct FusedSmem {
    RowCtl ctl[2];                  // alternates between consecutive rows of this CTA
    uint32_t red_key[FNW], red_idx[FNW];              // one set of warp slots per reduction site
    unsigned long long red_min[FNW];
    uint32_t red_fin[FNW], walk[FNW];
    float scan_sum[FNW], scan_fold[FNW];
    FusedXchg xchg[2];              // alternates between consecutive rows
    union alignas(16) {             // the id -> count table is dead once the penalties are applied
        struct { uint32_t hkey[F_HASH]; uint32_t hcnt[F_HASH]; } pen;
        struct { BoundSmem sel; float members[F_LCAP]; } s;
    } ua;
    float tmax_s[FVT];              // each virtual thread's maximum after the load pass
    uint8_t redo_max[FVT];
    uint32_t cand_n, memb_n, bound_key;
    long long prof_acc[16];         // phase timers of thread 0
    uint32_t hash_dirty;            // the id -> count table holds leftovers and must be reset before use
    unsigned long long load_bar[8]; // one mbarrier per piece of the bulk copy that fills the slice
};

// Optional phase timers (clock64 deltas of thread 0, summed over the rows of each CTA in shared memory and
// written out when the CTA is done), enabled by pointing `prof` at [gridDim.x x 16] counters.
#define PGS_TICK(slot)                                              \
    do {                                                            \
        if (fl.prof && tid == 0) {                                  \
            const long long now_ = clock64();                       \
            sm.prof_acc[slot] += now_ - tick_;                      \
            tick_ = now_;                                           \
        }                                                           \
    } while (0)

// ---- CTA-wide helpers for FNW warps with ONE barrier each: every warp leaves its partial in `slots`, and
// after the barrier every warp combines all partials itself.  A call site owns its slots; they may be
// written again only after another barrier (every site runs once per row, rows are barriers apart).
__device__ __forceinline__ unsigned long long fblock_max_u64(unsigned long long v, unsigned long long* slots) {
    const int lane = threadIdx.x & 31;
    for (int o = 16; o; o >>= 1) {
        const unsigned long long x = __shfl_xor_sync(FULL, v, o);
        v = x > v ? x : v;
    }
    if (lane == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    v = slots[lane % FNW];
    for (int o = FNW / 2; o; o >>= 1) {
        const unsigned long long x = __shfl_xor_sync(FULL, v, o);
        v = x > v ? x : v;
    }
    return v;
}
__device__ __forceinline__ uint32_t fblock_sum_u32(uint32_t v, uint32_t* slots) {
    const int lane = threadIdx.x & 31;
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    if (lane == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    v = lane < FNW ? slots[lane] : 0u;
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}
// exclusive scan of one float per thread (plain adds: only used as an estimate); *total = CTA sum
__device__ __forceinline__ float fblock_excl_scan_f32(float v, float* total, float* slots) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) slots[w] = inc;
    __syncthreads();
    const float x = lane < FNW ? slots[lane] : 0.0f;
    float xi = x;
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(FULL, xi, o);
        if (lane >= o) xi += t;
    }
    *total = __shfl_sync(FULL, xi, 31);
    return __shfl_sync(FULL, xi - x, w) + (inc - v);
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
#pragma unroll 1
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
constexpr uint32_t TMA_PIECE = 131072;   // bytes per bulk copy (measured: 32 KB pieces 110.6 us per step, 64 KB 108.6, 128 KB 107.5)

// Top-k bound from all per-thread maxima (used when top_k is too large for the warp maxima): the C*FVT
// maxima are spread over F_NB equal-width buckets between their smallest finite value and the row maximum
// (a monotone map), the bucket holding the k-th largest is found from the histogram, and the exact value
// is picked among that bucket's few members.  Returns the bound's order key, 0 if fewer than top_k maxima
// are finite.  Called by every thread of the CTA.
__device__ __forceinline__ uint32_t thread_bound_key(FusedSmem& sm, const float* TM, uint32_t C, uint32_t top_k, float m) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    if (tid == 0) sm.hash_dirty = 1u;   // the histogram below lives in the table's space
    const uint32_t nv = C * FVT;
    uint32_t fin = 0;
    unsigned long long inv_min = 0ull;
#pragma unroll 1
    for (uint32_t i = tid; i < nv; i += FNT) {
        const uint32_t key = order_key(TM[i]);
        if (key) { fin++; const unsigned long long iv = 0xffffffffull - key; inv_min = iv > inv_min ? iv : inv_min; }
    }
    const uint32_t n_fin = fblock_sum_u32(fin, sm.red_fin);
    inv_min = fblock_max_u64(inv_min, sm.red_min);
    if (n_fin < top_k) return 0u;
    const float lo_v = key_to_float((uint32_t)(0xffffffffull - inv_min));
    const float sc = m > lo_v ? (float)(F_NB - 1) / (m - lo_v) : 0.0f;
#pragma unroll 1
    for (int bkt = tid; bkt < F_NB; bkt += FNT) sm.ua.s.sel.hist[bkt] = 0u;
    if (tid == 0) { sm.ua.s.sel.prefix = 0xffffffffu; sm.ua.s.sel.k = 0u; sm.memb_n = 0u; }
    __syncthreads();
#pragma unroll 1
    for (uint32_t i = tid; i < nv; i += FNT) {
        const float v = TM[i];
        if (finite_f(v)) atomicAdd(&sm.ua.s.sel.hist[min((uint32_t)(F_NB - 1), (uint32_t)((v - lo_v) * sc))], 1u);
    }
    __syncthreads();
    {
        // walk from the top bucket down: thread j owns the BPT buckets F_NB-1 - j*BPT - u, u < BPT
        constexpr int BPT = F_NB / FNT;
        uint32_t hv[BPT], own = 0;
#pragma unroll
        for (int u = 0; u < BPT; u++) { hv[u] = sm.ua.s.sel.hist[(F_NB - 1) - tid * BPT - u]; own += hv[u]; }
        uint32_t inc = own;
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(FULL, inc, o);
            if (lane >= o) inc += up;
        }
        if (lane == 31) sm.walk[w] = inc;
        __syncthreads();
        uint32_t before = inc - own;   // maxima in higher buckets
#pragma unroll 1
        for (int ww = 0; ww < w; ww++) before += sm.walk[ww];
#pragma unroll
        for (int u = 0; u < BPT; u++) {
            if (before < top_k && before + hv[u] >= top_k) {
                sm.ua.s.sel.prefix = (F_NB - 1) - tid * BPT - u; sm.ua.s.sel.k = top_k - before;
            }
            before += hv[u];
        }
    }
    __syncthreads();
    const uint32_t bsel = sm.ua.s.sel.prefix, ksel = sm.ua.s.sel.k;
    // members of the selected bucket (at most F_LCAP of them are kept)
#pragma unroll 1
    for (uint32_t i = tid; i < nv; i += FNT) {
        const float v = TM[i];
        if (finite_f(v) && min((uint32_t)(F_NB - 1), (uint32_t)((v - lo_v) * sc)) == bsel) {
            const uint32_t at = atomicAdd(&sm.memb_n, 1u);
            if (at < (uint32_t)F_LCAP) sm.ua.s.members[at] = v;
        }
    }
    if (tid == 0) sm.ua.s.sel.hist[0] = 0u;   // reused: order key of the bound
    __syncthreads();
    const uint32_t nm = sm.memb_n;
    if (nm <= (uint32_t)F_LCAP) {
#pragma unroll 1
        for (uint32_t j = tid; j < nm; j += FNT) {
            const float v = sm.ua.s.members[j];
            uint32_t gt = 0, ge = 0;
#pragma unroll 1
            for (uint32_t o = 0; o < nm; o++) { gt += sm.ua.s.members[o] > v; ge += sm.ua.s.members[o] >= v; }
            if (gt < ksel && ksel <= ge) sm.ua.s.sel.hist[0] = order_key(v);
        }
    } else {
        // too many equal-bucket maxima: any member bounds the k-th largest from below
        if (tid == 0) sm.ua.s.sel.hist[0] = order_key(lo_v);
    }
    __syncthreads();
    return sm.ua.s.sel.hist[0];
}

// One more top-k candidate of this slice (rare next to the logits that are not)
__device__ __forceinline__ void add_candidate(FusedSmem& sm, uint32_t* CID, float* CX, uint32_t id, float x) {
    const uint32_t at = atomicAdd(&sm.cand_n, 1u);
    if (at < (uint32_t)F_LCAP) { CID[at] = id; CX[at] = x; }
}

// The sequential f32 fold of one chunk of numerators from a given running value (the refinement pass;
// the first pass has its own inlined copy)
__device__ __forceinline__ float refold_chunk(const float* X, uint32_t c0, uint32_t c1b, uint32_t c1, float acc) {
#pragma unroll 1
    for (uint32_t i = c0; i < c1b; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(X + i);
        acc = fadd(fadd(fadd(fadd(acc, v.x), v.y), v.z), v.w);
    }
#pragma unroll 1
    for (uint32_t i = c1b; i < c1; i++) acc = fadd(acc, X[i]);
    return acc;
}

// Per-thread result of a load pass: the maximum of each virtual thread, where it sits, and the sanity bit
struct ThreadMax { float tm[VG]; uint32_t tq[VG]; int nonfinite; };

// bf16 rows: 64-bit coalesced loads, widened to f32 in shared memory (a 16-bit shift: exact), with the
// sanity check, the grammar mask and the per-thread maxima on the way.  Covers the whole 128-bit groups of the
// slice.
__device__ __forceinline__ ThreadMax load_bf16_body(float* X, const char* rowp, const uint32_t* mw, uint32_t lo, uint32_t nq) {
    const int tid = threadIdx.x;
    ThreadMax r;
#pragma unroll
    for (int g = 0; g < VG; g++) { r.tm[g] = -INFINITY; r.tq[g] = 0u; }
    r.nonfinite = 0;
    const uint2* src = (const uint2*)(rowp) + lo / 4;    // 4 bf16 per 8-byte load
#pragma unroll 1
    for (uint32_t q0 = tid; q0 < nq; q0 += 4 * FNT) {
        uint2 raw[4];
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (q0 + u * FNT < nq) raw[u] = __ldcs(src + q0 + u * FNT);
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (q0 + u * FNT < nq) {
                const uint32_t q = q0 + u * FNT;
                const int g = u % VG;   // q0 - tid is a multiple of 4 * FNT
                float4 v;
                v.x = __uint_as_float(raw[u].x << 16); v.y = __uint_as_float(raw[u].x & 0xffff0000u);
                v.z = __uint_as_float(raw[u].y << 16); v.w = __uint_as_float(raw[u].y & 0xffff0000u);
                r.nonfinite |= !finite_f(v.x) | !finite_f(v.y) | !finite_f(v.z) | !finite_f(v.w);
                if (mw) {
                    const uint32_t bits = __ldg(mw + ((lo >> 5) + (q >> 3))) >> ((q & 7) * 4);
                    if (!(bits & 1u)) v.x = -INFINITY;
                    if (!(bits & 2u)) v.y = -INFINITY;
                    if (!(bits & 4u)) v.z = -INFINITY;
                    if (!(bits & 8u)) v.w = -INFINITY;
                }
                const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                if (m4 > r.tm[g]) { r.tm[g] = m4; r.tq[g] = q * 4; }
                ((float4*)X)[q] = v;
            }
    }
    return r;
}

__device__ __forceinline__ uint32_t load_owner(uint32_t i, uint32_t len) {
    // thread that loaded slice element i: 128-bit groups are dealt round-robin, then the ragged tail
    const uint32_t body = (len / 4) * 4;
    return i < body ? ((i >> 2) & (FVT - 1)) : ((i - body) & (FVT - 1));
}

// One thread reads and validates a row's parameters (same rules as the general kernel).
__device__ __forceinline__ void prepare_row(const RowArgs& a, uint32_t row, RowCtl& c) {
const uint32_t V = a.vocab;
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
    const bool greedy = temp < 1e-5f;
    const bool use_k = top_k != 0u && top_k < V;
    // rows this kernel does not serve go to the general kernel
    const char* rowp = (const char*)a.logits + (size_t)row * a.row_stride * (a.dtype == 0 ? 4 : 2);
    const bool aligned = (((uintptr_t)rowp & 15) == 0);
    const bool defer = !aligned || (!greedy && (!use_k || top_k > (uint32_t)F_KMAX));
    // log2(e) / t as a two-float sum s_hi + s_lo with s_lo > 0, so that the exponent's argument carries
    // no systematic error and a masked entry (-inf) stays -inf through both products
    const double scale_d = 1.4426950408889634 / (double)fmaxf(temp, 1e-9f);
    float s_hi = (float)scale_d;
    if ((double)s_hi >= scale_d) s_hi = u2f(f2u(s_hi) - 1u);
    c.s_hi = s_hi; c.s_lo = (float)(scale_d - (double)s_hi);
    c.rowp = rowp; c.mw = mw; c.temp = temp; c.freq = freq; c.pres = pres; c.rep = rep;
    c.top_k = top_k; c.gflags = gflags; c.h0 = h0; c.nh = nh;
    c.kind = bad ? 1u : defer ? 2u : 0u;
}

__host__ __device__ constexpr size_t fused_fixed_bytes() { return (sizeof(FusedSmem) + 15) & ~size_t(15); }
__host__ __device__ inline size_t fused_exchange_bytes(uint32_t cluster) {
    const size_t maxima = (size_t)cluster * FVT * sizeof(float), cands = (size_t)F_LCAP * 8;
    return maxima > cands ? maxima : cands;
}

__global__ void __launch_bounds__(FNT, FNT <= 512 ? 2 : 1) fused_row_kernel(const RowArgs a, const FusedLaunch fl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FusedSmem& sm = *reinterpret_cast<FusedSmem*>(smem_raw);
    float* TM = reinterpret_cast<float*>(smem_raw + fused_fixed_bytes());   // maxima of all CTAs, later the candidates
    uint32_t* CID = reinterpret_cast<uint32_t*>(TM);
    float* CX = TM + F_LCAP;
    float* X = reinterpret_cast<float*>(smem_raw + fused_fixed_bytes() + fused_exchange_bytes(fl.cluster));
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
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
#pragma unroll 1
        for (int i = 0; i < 16; i++) sm.prof_acc[i] = 0;
        sm.hash_dirty = 1u;
#pragma unroll 1
        for (int b = 0; b < 8; b++) mbar_init(&sm.load_bar[b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    constexpr int PREP_TID = FNT - 32;   // lane 0 of the last warp
    if (tid == PREP_TID && cluster_id < a.rows) prepare_row(a, cluster_id, sm.ctl[0]);
    long long tick_ = clock64();
    uint32_t it = 0;
    for (uint32_t row = cluster_id; row < a.rows; row += n_clusters, it++) {
        // this row's parameters are complete, and every warp is done with the slice of the row before
        __syncthreads();
        FusedXchg& xc = sm.xchg[parity];
        const uint32_t pbuf = parity;   // exchange buffer of this row; the next synced row takes the other one
        PGS_TICK(12);  // row barrier
        const RowCtl& ctl = sm.ctl[it & 1];
        if (tid == PREP_TID && row + n_clusters < a.rows) prepare_row(a, row + n_clusters, sm.ctl[(it + 1) & 1]);
        const bool writer = rank == 0 && tid == 0;
        if (ctl.kind == 1u) {
            if (writer) { a.token[row] = 0; a.status[row] = ROW_BAD_PARAM; if (a.drew) a.drew[row] = 0; fl.recs[row].kind = 0; }
            continue;
        }
        if (ctl.kind == 2u) {
            if (writer) { fl.work_rows[atomicAdd(fl.work_count, 1u)] = row; fl.recs[row].kind = 0; }
            continue;
        }
        const float temp = ctl.temp, freq = ctl.freq, pres = ctl.pres, rep = ctl.rep;
        const uint32_t top_k = ctl.top_k, gflags = ctl.gflags, h0 = ctl.h0, nh = ctl.nh;
        const uint32_t* mw = ctl.mw;
        const char* rowp = ctl.rowp;
        const bool greedy = temp < 1e-5f;

        // ------------------------------- load slice: sanity + bitmask AND + per-thread max
        float tm[VG];        // running maximum of each virtual thread this thread plays
        uint32_t tqs[VG];    // slice index of the 128-bit group (or, flagged, the tail element) that holds it
#pragma unroll
        for (int g = 0; g < VG; g++) { tm[g] = -INFINITY; tqs[g] = 0; sm.redo_max[g * FNT + tid] = 0; }
        if (tid == 0) sm.cand_n = 0u;
        int nonfinite = 0;
        const uint32_t nq = len / 4;   // 128-bit groups; a ragged tail exists only in the last slice
        auto take1 = [&](uint32_t i, float x) {
            nonfinite |= !finite_f(x);
            if (mw && !((__ldg(mw + ((lo + i) >> 5)) >> ((lo + i) & 31)) & 1u)) x = -INFINITY;
            if (x > tm[0]) { tm[0] = x; tqs[0] = i | 0x80000000u; }   // the tail has at most 3 elements: threads 0..2
            X[i] = x;
        };
        // history ids of this slice -> id->count table; runs while the copy below is in flight
        const bool do_fp = !(fabsf(freq) < 1e-6f && fabsf(pres) < 1e-6f);
        const bool do_pres = fabsf(pres) > 1e-6f;
        const bool do_rep = rep != 1.0f;
        const bool pen = nh > 0 && (do_fp || do_rep);
        int spill = 0;
        // the first id of every thread is requested before anything else, so that its latency hides behind the
        // table reset and the copy's issue
        const uint32_t hid0 = (pen && (uint32_t)tid < nh) ? __ldg(a.hist_ids + h0 + tid) : 0xffffffffu;
        auto index_history = [&]() {
            // the penalty pass hands every slot back empty, so a reset is only needed after a row that left
            // entries behind or used the space for something else
            if (sm.hash_dirty) {
#pragma unroll 1
                for (int s = tid; s < F_HASH; s += FNT) { sm.ua.pen.hkey[s] = 0xffffffffu; sm.ua.pen.hcnt[s] = 0u; }
                __syncthreads();
                if (tid == 0) sm.hash_dirty = 0u;
            }
#pragma unroll 1
            for (uint32_t j = tid; j < nh; j += FNT) {
                const uint32_t id = j == (uint32_t)tid ? hid0 : __ldg(a.hist_ids + h0 + j);
                if (id < lo || id >= hi) continue;
                uint32_t s = (id * 2654435761u) >> (32 - F_HASH_BITS);
                bool placed = false;
#pragma unroll 1
                for (int probe = 0; probe < 64; probe++) {
                    const uint32_t prev = atomicCAS(&sm.ua.pen.hkey[s], 0xffffffffu, id);
                    if (prev == 0xffffffffu || prev == id) { atomicAdd(&sm.ua.pen.hcnt[s], 1u); placed = true; break; }
                    s = (s + 1) & (F_HASH - 1);
                }
                if (!placed) spill = 1;
            }
        };
        // f32 rows: one thread streams the slice into shared memory with bulk asynchronous copies
        // (128 KB pieces, one mbarrier each); every warp then checks / masks / maximises it in two halves
        // as they land.  All clusters reach this point at about the same time, so the copies of a whole wave
        // of rows compete for HBM; once this row has landed the next row's slice is therefore prefetched into
        // L2, where the memory system is idle, and the next copy is then served from L2.
        const uint32_t body = nq * 16;
        const uint32_t n_pieces = a.dtype == 0 ? (body + TMA_PIECE - 1) / TMA_PIECE : 0u;   // <= 8 for any slice that fits
        if (a.dtype == 0) {
            const char* gsrc = rowp + (size_t)lo * 4;
            if (tid == 0) {
                if (body && !poisoned) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier generic writes to X
#pragma unroll 1
                    for (uint32_t pc = 0; pc < n_pieces; pc++) {
                        const uint32_t off = pc * TMA_PIECE, bytes = min(TMA_PIECE, body - off);
                        mbar_expect_tx(&sm.load_bar[pc], bytes);
                        bulk_g2s((char*)X + off, gsrc + off, bytes, &sm.load_bar[pc]);
                    }
                }
            }
        }
        if (pen) index_history();
        PGS_TICK(11);  // copy issued, history indexed
        if (a.dtype == 0) {
            float poison = 0.0f, poison1 = 0.0f;   // 0 * v is NaN exactly when v is infinite or NaN, and NaN sticks
            // The slice is checked in two halves, each in one tight loop once its pieces have landed (a loop per
            // piece spends more on waiting and set-up than on the few groups a thread has in it).  Every warp
            // waits on its own: one lane polls (bounded), the rest follow.
            constexpr uint32_t PQ = TMA_PIECE / 16;   // 128-bit groups per piece, a whole number of FVT groups
            const uint32_t split = (n_pieces + 1u) / 2u;
#pragma unroll 1
            for (uint32_t half = 0; half < 2u; half++) {
                const uint32_t p0 = half ? split : 0u, p1 = half ? n_pieces : split;
                int ok = 1;
                const long long w0_ = fl.prof ? clock64() : 0;
                if (!poisoned && lane == 0)
                    for (uint32_t pc = p0; pc < p1 && ok; pc++) ok = mbar_wait(&sm.load_bar[pc], load_phase) ? 1 : 0;
                ok = __shfl_sync(FULL, ok, 0);
                if (fl.prof && tid == 0) sm.prof_acc[14] += clock64() - w0_;   // waiting for the copy (also inside slot 0)
                if (!ok) poisoned = true;
                if (poisoned) continue;
                const uint32_t q_end = min(nq, p1 * PQ);
#pragma unroll 1
                for (uint32_t q0 = p0 * PQ + tid; q0 < q_end; q0 += 2 * FNT) {   // two groups per round, both requested first
                    const bool has1 = q0 + FNT < q_end;
                    float4 v0 = ((const float4*)X)[q0];
                    float4 v1 = has1 ? ((const float4*)X)[q0 + FNT] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    poison = __fmaf_rn(v0.x, 0.0f, poison); poison = __fmaf_rn(v0.y, 0.0f, poison);
                    poison = __fmaf_rn(v0.z, 0.0f, poison); poison = __fmaf_rn(v0.w, 0.0f, poison);
                    poison1 = __fmaf_rn(v1.x, 0.0f, poison1); poison1 = __fmaf_rn(v1.y, 0.0f, poison1);
                    poison1 = __fmaf_rn(v1.z, 0.0f, poison1); poison1 = __fmaf_rn(v1.w, 0.0f, poison1);
                    if (mw) {
                        const uint32_t b0 = __ldg(mw + ((lo >> 5) + (q0 >> 3))) >> ((q0 & 7) * 4);
                        if (!(b0 & 1u)) v0.x = -INFINITY;
                        if (!(b0 & 2u)) v0.y = -INFINITY;
                        if (!(b0 & 4u)) v0.z = -INFINITY;
                        if (!(b0 & 8u)) v0.w = -INFINITY;
                        ((float4*)X)[q0] = v0;
                        if (has1) {
                            const uint32_t q1 = q0 + FNT;
                            const uint32_t b1 = __ldg(mw + ((lo >> 5) + (q1 >> 3))) >> ((q1 & 7) * 4);
                            if (!(b1 & 1u)) v1.x = -INFINITY;
                            if (!(b1 & 2u)) v1.y = -INFINITY;
                            if (!(b1 & 4u)) v1.z = -INFINITY;
                            if (!(b1 & 8u)) v1.w = -INFINITY;
                            ((float4*)X)[q1] = v1;
                        }
                    }
                    // the round's groups belong to virtual threads (q0 / FNT) % VG and the next one
                    const int g0 = (int)((q0 / FNT) % VG), g1 = (int)((q0 / FNT + 1) % VG);
                    const float m0 = fmaxf(fmaxf(v0.x, v0.y), fmaxf(v0.z, v0.w));
                    if (m0 > tm[g0]) { tm[g0] = m0; tqs[g0] = q0 * 4; }
                    const float m1 = fmaxf(fmaxf(v1.x, v1.y), fmaxf(v1.z, v1.w));
                    if (has1 && m1 > tm[g1]) { tm[g1] = m1; tqs[g1] = (q0 + FNT) * 4; }
                }
            }
            if (tid == 0 && !poisoned && row + n_clusters < a.rows) {   // next row of this cluster -> L2
                const char* nsrc = (const char*)a.logits + (size_t)(row + n_clusters) * a.row_stride * 4 + (size_t)lo * 4;
                if (((uintptr_t)nsrc & 15) == 0) {
#pragma unroll 1
                    for (uint32_t off = 0; off < body; off += TMA_PIECE)
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(nsrc + off), "r"(min(TMA_PIECE, body - off)) : "memory");
                }
            }
            poison += poison1;
            if (n_pieces) load_phase ^= 1u;
            if (poisoned) nonfinite = 2;   // reported as a load timeout after the exchange
            nonfinite |= poison != poison;
            if (!poisoned)
#pragma unroll 1
                for (uint32_t i = nq * 4 + tid; i < len; i += FNT) take1(i, __ldcs((const float*)rowp + lo + i));
        } else {
            const ThreadMax r = load_bf16_body(X, rowp, mw, lo, nq);
#pragma unroll
            for (int g = 0; g < VG; g++) { tm[g] = r.tm[g]; tqs[g] = r.tq[g]; }
            nonfinite |= r.nonfinite;
#pragma unroll 1
            for (uint32_t i = nq * 4 + tid; i < len; i += FNT)
                take1(i, __uint_as_float((uint32_t)__ldcs((const unsigned short*)rowp + lo + i) << 16));
        }
#pragma unroll
        for (int g = 0; g < VG; g++) sm.tmax_s[g * FNT + tid] = tm[g];
        {
            const int both = __syncthreads_or(nonfinite | (spill << 8));
            nonfinite = both & 0xff;
            spill = both >> 8;
        }
        PGS_TICK(0);   // load

        // --------------------------------------------------------------- penalties
        if (pen && (nonfinite || spill) && tid == 0) sm.hash_dirty = 1u;   // the table keeps this row's entries
        if (pen && !nonfinite) {
            if (!spill) {
#pragma unroll
                for (int s = tid; s < F_HASH; s += FNT) {
                    const uint32_t id = sm.ua.pen.hkey[s];
                    if (id == 0xffffffffu) continue;
                    const float cnt = (float)sm.ua.pen.hcnt[s];
                    sm.ua.pen.hkey[s] = 0xffffffffu; sm.ua.pen.hcnt[s] = 0u;   // hand the slot back empty
                    const uint32_t i = id - lo;
                    const float old = X[i];
                    float x = old;
                    if (do_rep) x = x > 0.0f ? fdiv(x, rep) : fmul(x, rep);
                    if (do_fp) {
                        x = fsub(x, fmul(freq, cnt));
                        if (do_pres) x = fsub(x, pres);
                    }
                    // an overflowed penalty is non-finite; the chain treats that like a masked entry
                    x = finite_f(x) ? x : -INFINITY;
                    X[i] = x;
                    // the owner's maximum is stale only if this entry held it, or now reaches it
                    const uint32_t ow = load_owner(i, len);
                    const float om = sm.tmax_s[ow];
                    if (old >= om || x >= om) sm.redo_max[ow] = 1;
                }
            }
            __syncthreads();
        }
        // ----------------------------------------------------------------- EOS fix
        if (mw && (gflags & 1u) && a.eos >= 0 && (uint32_t)a.eos >= lo && (uint32_t)a.eos < hi) {   // CTA-uniform
            if (tid == 0 && !finite_f(X[a.eos - lo])) {
                X[a.eos - lo] = 0.0f;
                sm.redo_max[load_owner(a.eos - lo, len)] = 1;
            }
            __syncthreads();
        }
#pragma unroll
        for (int g = 0; g < VG; g++) {
            if (!sm.redo_max[g * FNT + tid]) continue;
            tm[g] = -INFINITY;
#pragma unroll 1
            for (uint32_t q = g * FNT + tid; q < nq; q += FVT) {
                const float4 v = ((const float4*)X)[q];
                const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                if (m4 > tm[g]) { tm[g] = m4; tqs[g] = q * 4; }
            }
            if (g == 0)
#pragma unroll 1
                for (uint32_t i = nq * 4 + tid; i < len; i += FNT)
                    if (X[i] > tm[0]) { tm[0] = X[i]; tqs[0] = i | 0x80000000u; }
        }
        PGS_TICK(1);   // penalties

        // ------------------------------------------------- slice max / argmax, lowest id
        // each thread knows where its maximum first occurs (its groups are visited in ascending order)
        uint32_t bkey = 0u, bidx = 0xffffffffu;   // largest order key, lowest id holding it
#pragma unroll
        for (int g = 0; g < VG; g++) {
            if (!(tm[g] > -INFINITY)) continue;
            uint32_t idx = tqs[g] & 0x7fffffffu;
            if (!(tqs[g] & 0x80000000u)) {
                const float4 v = *reinterpret_cast<const float4*>(X + idx);
                idx += v.x == tm[g] ? 0u : v.y == tm[g] ? 1u : v.z == tm[g] ? 2u : 3u;
            }
            const uint32_t k = order_key(tm[g]);
            if (k > bkey || (k == bkey && lo + idx < bidx)) { bkey = k; bidx = lo + idx; }
        }
        {
            const uint32_t wk = __reduce_max_sync(FULL, bkey);
            const uint32_t wi = __reduce_min_sync(FULL, bkey == wk ? bidx : 0xffffffffu);
            if (lane == 0) { sm.red_key[w] = wk; sm.red_idx[w] = wi; }
            __syncthreads();
            const uint32_t k2 = sm.red_key[lane % FNW], i2 = sm.red_idx[lane % FNW];
            bkey = __reduce_max_sync(FULL, k2);
            bidx = __reduce_min_sync(FULL, k2 == bkey ? i2 : 0xffffffffu);
        }
        const unsigned long long best = bkey ? ((unsigned long long)bkey << 32) | (unsigned long long)(0xffffffffu - bidx) : 0ull;
        PGS_TICK(2);   // argmax
        // ------------------------------------------------ cluster exchange #1
#pragma unroll 1
        for (uint32_t r = tid; r < C; r += FNT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].best[rank] = best;
            peer->xchg[pbuf].flags[rank] = nonfinite | (spill << 8);
        }
        // material for the top-k bound: the 32*C warp maxima when there are comfortably more warps than
        // top_k, else all FVT*C thread maxima
        const bool warp_bound = !greedy && 8u * top_k <= 7u * C * FVW;
        if (!greedy) {
            if (warp_bound) {
#pragma unroll
                for (int g = 0; g < VG; g++) {   // virtual warp g * FNW + w
                    const uint32_t wk = __reduce_max_sync(FULL, order_key(tm[g]));
                    const float wmax = wk ? key_to_float(wk) : -INFINITY;
                    if (lane < (int)C) cluster.map_shared_rank(TM, lane)[rank * FVW + g * FNW + w] = wmax;
                }
            } else {
#pragma unroll 1
                for (uint32_t r = 0; r < C; r++) {
                    float* dst = cluster.map_shared_rank(TM, r) + rank * FVT + tid;
#pragma unroll
                    for (int g = 0; g < VG; g++) dst[g * FNT] = tm[g];
                }
            }
        }
        cluster.sync();
        parity ^= 1u;
        PGS_TICK(3);   // sync 1
        // lane r looks at CTA r's slot; warp-wide reductions combine them
        const unsigned long long rb = (uint32_t)lane < C ? xc.best[lane] : 0ull;
        const uint32_t gkey = __reduce_max_sync(FULL, (uint32_t)(rb >> 32));
        const uint32_t ginv = __reduce_max_sync(FULL, (uint32_t)(rb >> 32) == gkey ? (uint32_t)rb : 0u);
        const uint32_t gfl = __reduce_or_sync(FULL, (uint32_t)lane < C ? (uint32_t)xc.flags[lane] : 0u);
        const int any_nonfinite = (int)(gfl & 0xffu), any_spill = (int)(gfl >> 8);
        const bool any = gkey != 0u;
        const float m = any ? key_to_float(gkey) : -INFINITY;
        const uint32_t amax = any ? 0xffffffffu - ginv : 0u;
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
        // The C*FVT maxima are spread over F_NB equal-width buckets between their smallest finite
        // value and the row maximum (a monotone map), the bucket holding the k-th largest is found
        // from the histogram, and the exact value is picked among that bucket's few members.
        const float t = fmaxf(temp, 1e-9f);
        float cut = -INFINITY;
        PGS_TICK(13);  // exchange #1 read
        uint32_t kk;   // order key of a value that at least top_k logits reach, 0 if there is none
        if (warp_bound) {
            // k-th largest of the FVW*C warp maxima.  Their order keys are made distinct by replacing the
            // low 8 bits with the slot number (the bound can only move down by that, so it stays a bound),
            // so a key's rank is the number of larger keys.  Every warp holds all keys, a few per lane, and
            // ranks its share of them with warp-wide sums; exactly one key has rank top_k - 1.
            const uint32_t nvw = C * FVW;   // <= 256
            constexpr int KPL = F_MAXC * FVW / 32;   // keys per lane at the largest cluster
            uint32_t u[KPL];
#pragma unroll
            for (int q = 0; q < KPL; q++) {
                const uint32_t slot = q * 32 + lane;
                u[q] = slot < nvw ? ((order_key(TM[slot]) & ~0xffu) | slot) : 0u;
            }
            const uint32_t per = (nvw + FNW - 1) / FNW;
            uint32_t found = 0u;
#pragma unroll 1
            for (uint32_t j = w * per; j < min(nvw, (w + 1) * per); j++) {   // warp-uniform
                const uint32_t kj = (order_key(TM[j]) & ~0xffu) | j;
                uint32_t above = 0;
#pragma unroll
                for (int q = 0; q < KPL; q++) above += u[q] > kj;
                if (__reduce_add_sync(FULL, above) == top_k - 1u) found = kj;
            }
            if (found && lane == 0) sm.bound_key = found & ~0xffu;
            __syncthreads();
            PGS_TICK(15);  // warp maxima ranked
            kk = sm.bound_key;
        } else {
            kk = thread_bound_key(sm, TM, C, top_k, m);
        }
        if (kk) {
            const float bound = key_to_float(kk);
            // every logit whose probability could still tie with the k-th one stays above the cut
            const float delta = 4.8e-7f * (fabsf(m - bound) + 4.0f * t) + 4.8e-7f * (fabsf(bound) + fabsf(m));
            cut = bound - delta;
        }
        PGS_TICK(4);   // select (no barrier needed here: the maxima were last read before a barrier above)
        // ---- one pass in chunk order: collect the candidates, then overwrite each logit with its
        //      softmax numerator (hardware exp2) and accumulate the plain chunk sum
        const float s_hi = ctl.s_hi, s_lo = ctl.s_lo;   // log2(e) / t as a two-float sum
        const float cut_f = fmaxf(cut, -3.4e38f);   // masked entries (-inf) are never candidates
        const uint32_t L = fl.chunk;   // 4 * odd: 128-bit shared-memory accesses of a warp do not collide
        const uint32_t c0 = min(len, tid * L), c1 = min(len, c0 + L);
        const uint32_t c1b = c0 + ((c1 - c0) & ~3u);   // whole 128-bit groups; a remainder only at the ragged end
        float csum = 0.0f;
        auto candidate = [&](float x, uint32_t i) {
            if (x >= cut_f) add_candidate(sm, CID, CX, lo + i, x);
        };
        // 2^((x - m) * log2(e) / t) by the hardware exp2 (a few ulp; results below the normal range are
        // flushed to zero, far below anything the sum can see)
        auto numerator = [&](float x) -> float {
            const float a_ = fsub(x, m);
            return ex2_approx_ftz(__fmaf_rn(a_, s_hi, fmul(a_, s_lo)));
        };
        auto group = [&](float4 v, uint32_t i) -> float {
            if (fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)) >= cut_f) {
                candidate(v.x, i); candidate(v.y, i + 1); candidate(v.z, i + 2); candidate(v.w, i + 3);
            }
            v.x = numerator(v.x); v.y = numerator(v.y); v.z = numerator(v.z); v.w = numerator(v.w);
            *reinterpret_cast<float4*>(X + i) = v;
            return (v.x + v.y) + (v.z + v.w);
        };
        uint32_t ib = c0;
        for (; ib + 8 <= c1b; ib += 8) {   // two groups per round, both requested before either is used
            const float4 v0 = *reinterpret_cast<const float4*>(X + ib);
            const float4 v1 = *reinterpret_cast<const float4*>(X + ib + 4);
            const float g0 = group(v0, ib), g1 = group(v1, ib + 4);
            csum += g0 + g1;
        }
        if (ib < c1b) csum += group(*reinterpret_cast<const float4*>(X + ib), ib);
#pragma unroll 1
        for (uint32_t i = c1b; i < c1; i++) { candidate(X[i], i); const float e = numerator(X[i]); X[i] = e; csum += e; }
        PGS_TICK(5);   // gather + exp
        float ftot0;
        const float pre0 = fblock_excl_scan_f32(csum, &ftot0, sm.scan_sum);
        const double dtot = (double)ftot0;
        const uint32_t my_n = sm.cand_n;   // complete: the scan's barrier is behind every thread's pass
        PGS_TICK(6);   // scan
        // ------------------------------------------------ cluster exchange #2
#pragma unroll 1
        for (uint32_t r = tid; r < C; r += FNT) {
            FusedSmem* peer = cluster.map_shared_rank(&sm, r);
            peer->xchg[pbuf].ncand[rank] = my_n;
            peer->xchg[pbuf].true_total[rank] = (float)dtot;
        }
        cluster.sync();
        PGS_TICK(7);   // sync 2
        const uint32_t rn = (uint32_t)lane < C ? xc.ncand[lane] : 0u;
        const uint32_t cand_total = __reduce_add_sync(FULL, rn);
        const uint32_t cand_off = __reduce_add_sync(FULL, (uint32_t)lane < rank ? rn : 0u);
        bool overflow = __reduce_max_sync(FULL, rn) > (uint32_t)F_LCAP;
        // ranks below this one; every group of F_MAXC lanes adds up the same values
        double before0 = (uint32_t)(lane % F_MAXC) < rank ? (double)xc.true_total[lane % F_MAXC] : 0.0;
        for (int o = F_MAXC / 2; o; o >>= 1) before0 += __shfl_xor_sync(FULL, before0, o);
        overflow |= cand_total > (uint32_t)F_MCAP;
        if (overflow) {   // identical decision in every CTA
            if (writer) { fl.work_rows[atomicAdd(fl.work_count, 1u)] = row; fl.recs[row].kind = 0; }
            continue;
        }
        // candidates -> global memory, in slice order, for the finish kernel
#pragma unroll 1
        for (uint32_t j = tid; j < my_n; j += FNT) {
            fl.cand_id[(size_t)row * F_MCAP + cand_off + j] = CID[j];
            fl.cand_x[(size_t)row * F_MCAP + cand_off + j] = CX[j];
        }
        // ---------- the sequential fold, chunk by chunk: first from the plain prefix sums ...
        const float start0 = (float)before0 + pre0;
        auto fold_chunk = [&](float acc_) -> float {
            for (uint32_t i = c0; i < c1b; i += 4) {
                const float4 v = *reinterpret_cast<const float4*>(X + i);
                acc_ = fadd(fadd(fadd(fadd(acc_, v.x), v.y), v.z), v.w);
            }
#pragma unroll 1
            for (uint32_t i = c1b; i < c1; i++) acc_ = fadd(acc_, X[i]);
            return acc_;
        };
        float acc = fold_chunk(start0);
        const float inc1 = fsub(acc, start0);   // exact: both ends lie within a factor two or the chunk is re-folded
        float ftot1;
        const float pre1 = fblock_excl_scan_f32(inc1, &ftot1, sm.scan_fold);
        const double tot1 = (double)ftot1;
        PGS_TICK(8);   // fold 1
#pragma unroll 1
        for (uint32_t r = tid; r < C; r += FNT) cluster.map_shared_rank(&sm, r)->xchg[pbuf].fold1[rank] = tot1;
        cluster.sync();   // exchange #3
        double before1 = (uint32_t)(lane % F_MAXC) < rank ? xc.fold1[lane % F_MAXC] : 0.0;
        for (int o = F_MAXC / 2; o; o >>= 1) before1 += __shfl_xor_sync(FULL, before1, o);
        // ... then once more, for the chunks whose binade that first pass got wrong or crossed
        const float start1 = (float)before1 + pre1;
        const uint32_t e0 = f2u(start0) & 0x7f800000u;
        double inc2 = (double)inc1;
        if ((f2u(start1) & 0x7f800000u) != e0 || (f2u(acc) & 0x7f800000u) != e0) {
            acc = refold_chunk(X, c0, c1b, c1, start1);
            inc2 = (double)acc - (double)start1;
        }
        for (int o = 16; o; o >>= 1) inc2 += __shfl_xor_sync(FULL, inc2, o);
        if (lane == 0) fl.recs[row].part[rank * FNW + w] = inc2;   // the finish kernel adds the warps up
        if (writer) {
            RowRec& rec = fl.recs[row];
            rec.kind = 1; rec.n_cand = cand_total; rec.amax = amax; rec.status = status;
            rec.m = m; rec.t = t; rec.n_parts = C * FNW;
        }
        PGS_TICK(9);   // fold 2
    }
    if (fl.prof && tid == 0)
#pragma unroll 1
        for (int i = 0; i < 16; i++) fl.prof[blockIdx.x * 16 + i] += sm.prof_acc[i];
    // no CTA may exit while a peer can still write into its shared memory
    cluster.sync();
}

uint32_t fused_threads() { return FNT; }
uint32_t fused_piece_bytes() { return TMA_PIECE; }

size_t fused_smem_bytes(uint32_t slice_len, uint32_t cluster) {
    return fused_fixed_bytes() + fused_exchange_bytes(cluster) + (size_t)slice_len * sizeof(float);
}

cudaError_t configure_fused(size_t max_smem) {
    cudaError_t e = cudaFuncSetAttribute(fused_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)max_smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(fused_row_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(fused_row_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
}

// how many CTAs with `smem` bytes each one SM can hold
cudaError_t fused_ctas_per_sm(size_t smem, int* out) {
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(out, fused_row_kernel, FNT, smem);
}

// how many clusters of `cluster` CTAs with `smem` bytes each can be resident at once
cudaError_t fused_max_clusters(uint32_t cluster, size_t smem, int* out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1);
    cfg.blockDim = dim3(FNT, 1, 1);
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
    cfg.blockDim = dim3(FNT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = fl.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, fused_row_kernel, a, fl);
}

}  // namespace pgs
