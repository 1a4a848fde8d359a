// Streaming row kernel: the hot path of the sampler.
//
// One CTA of 512 threads (two per SM) owns one batch row at a time and reads it twice with plain 128-bit
// coalesced loads, sixteen logits per thread and piece.  Inside a pass nothing synchronises the warps, so the
// loads of some overlap the arithmetic of the others, and what a piece costs beyond its logits (addresses, table
// look-ups, warp reductions, loop control) is paid once per sixteen logits:
//
//   pass 1, last piece first, from HBM: sanity, penalties, grammar bitmask, EOS fix; per thread its running
//           maximum and four more (one per piece number mod 4) that bound the top-k threshold; per warp and piece the
//           plain sum of the softmax numerators relative to the warp's own maximum;
//   between: row maximum and argmax (lowest id: the threads that hold the maximum look at that piece again); a bound for the top-k threshold: the k-th largest of the 2048
//           per-thread maxima is reached by at least k logits, so "logit >= that bound" is a superset of the
//           top-k set that is only slightly larger; and, from the rescaled plain sums, the value the reference's
//           running sum has when it reaches each warp's 512 logits of each piece, to within 1e-3;
//   pass 2, first piece first, from L2 (the pieces read last in pass 1 are the freshest there): the same
//           processed logits again, candidates above the bound, softmax numerators by the hardware exp2, and
//           the reference's sequential f32 sum;
//   finish: exact probabilities of the candidates, top-k with ties, top-p walk, inverse-CDF pick.
//
// A row is 600 KB, more than one SM holds, and its maximum must be known before the first numerator: the row
// is therefore read a second time.  What the second pass finds in L2 is what the first pass read last, which is
// why the passes run in opposite directions; with a whole batch in flight that is about a third of the row.
// The loops have no registers for a second piece in flight, so every warp asks for the piece it will read two
// iterations later with an L2 prefetch.  An optional gate (a counter of rows that finished pass 1, bounded
// polling, off unless the launch asks for a cohort) can hold rows back so that fewer are in their first pass at
// once.
//
// Small batches: when all rows fit as resident clusters, a thread-block cluster of 4 or 8 CTAs shares every row
// (see stream_row_kernel below): a row alone on one CTA is bound by the latency of its own instructions.
//
// The f32 left fold (pagoda/src/sampler.rs:99-113): while the running value stays inside one binade, adding a
// non-negative term is an integer addition in units of that binade's ulp which depends on the running value only
// through its parity.  Wherever the estimate above puts the running value safely inside one binade for a warp's
// whole share of a piece, every thread adds its sixteen numerators to that binade's lower end (real f32
// additions) and the increments are summed as integers; the few shares in which the running value may change
// binade are folded 128 bits at a time from their own estimates of the running value, which reproduces the
// crossing.  Ties of round-half-even are decided by the parity of a stand-in, not of the true running value: the
// sum agrees with the reference's to about 1e-6 relative, and a decision can differ only when it sits that close
// to its boundary.
//
// Fidelity of this path: argmax, masks, penalties and candidate sets follow the reference bit for bit
// (pagoda/src/engine.rs:1286-1314, pagoda/src/sampler.rs:28-150); candidate numerators use the exact expf.
// Rows this kernel does not serve (top-k off or > 1024, more candidates than its buffers, histories beyond its
// id -> count table, rows that are not 16-byte aligned) are appended to a work list for the general row kernel.
#include <cuda_runtime.h>

#include <cooperative_groups.h>

#include "pgs_args.cuh"
#include "pgs_block.cuh"
#include "pgs_finish.cuh"
#include "pgs_stream.cuh"

namespace pgs {

constexpr int SNT = 512;                 // threads per CTA
constexpr int SNW = SNT / 32;            // warps per CTA
constexpr int S_EPT = 16;                // logits per thread and piece
constexpr int S_PIECE = SNT * S_EPT;     // logits per piece
constexpr int S_REGION = 32 * S_EPT;     // consecutive logits of one warp in a piece
constexpr int S_MAX_REGIONS = S_MAX_VOCAB / S_REGION;
constexpr int S_NCELL = 4;               // running maxima per thread (piece number mod S_NCELL)
constexpr int S_CELLS = S_NCELL * SNT;   // per-thread maxima that bound the top-k threshold
constexpr int S_NB = 1024;               // buckets of their histogram
constexpr int S_BPT = S_NB / SNT;        // buckets per thread
constexpr int S_RPT = S_MAX_REGIONS / SNT;   // regions per thread in the CTA-wide walks over regions
constexpr uint32_t S_NIL = 0xffffffffu;
static_assert(SNW <= 32, "warp slots are combined by one warp");

// Everything the kernel needs to know about a row, read and validated by one thread while the CTA still works
// on the row before it.
struct SRowCtl {
    const char* rowp;       // first logit of the row
    const uint32_t* mw;     // grammar mask words of the row's state, or null
    float temp, freq, pres, rep, top_p, u01;
    float sc, sc_lo;        // log2(e) / max(temp, 1e-9) as a two-float sum
    uint32_t top_k, gflags, h0, nh;
    uint32_t kind;          // 0 serve, 1 bad parameters, 2 defer to the general kernel
};

// What the pass loops need to know about the row they work on.
enum : uint32_t { PF_PEN = 1u, PF_REP = 2u, PF_FP = 4u, PF_PRES = 8u };
struct PassArgs {
    const char* rowp;
    const uint32_t* mw;
    float sc, sc_lo, c_hi, c_lo, cut_f, freq, pres, rep;
    uint32_t V, n_full, n_regions, flags;
    uint32_t eos_piece, eos_tid, eos_sub;
    // a row shared by the CTAs of a cluster: this CTA works on the pieces q0, q0 + qstep, ...; the candidates of all of
    // them are collected by the first CTA (pointers into its shared memory)
    uint32_t q0, qstep;
    uint32_t* cand_n_p;
    uint32_t* cand_id_p;
    float* cand_x_p;
};

struct StreamSmem {
    SRowCtl ctl[2];
    PassArgs pa;
    unsigned long long exp_tab[32];
    uint32_t red_key[SNW], red_lo[SNW], red_fin[SNW], red_flag[SNW];
    uint32_t scan_u[SNW];
    float scan_f[SNW];
    double wacc[SNW];               // per-warp share of the fold
    uint32_t cand_n, sel_bucket, amax;
    // cluster mode: one slot per CTA of the cluster, written by that CTA into every CTA's copy (xk .. xflag) or into
    // the first CTA's copy (xs, xam)
    uint32_t xk[8], xlo[8], xfin[8], xflag[8], xam[8];
    double xs[8];
    uint32_t cand_id[F_MCAP];
    float cand_x[F_MCAP];
    long long prof_acc[16];
    // Two lives of one area: the tables of a row while it streams, and the arrays of the finish once its
    // candidates are known (nothing of the first is needed by then).
    union {
        struct {
            uint32_t hist[S_NB];
            float cell[S_CELLS];             // [S_NCELL][SNT]
            float t_am[SNT], t_max[SNT];     // per-thread results of pass 1 over the whole pieces
            uint32_t t_q[SNT];
            // per warp region of the row (512 consecutive logits): pass 1 leaves the warp's maximum and the plain sum
            // of its numerators relative to it; then the binade's lower end the fold has there (0 = fold this region the
            // careful way) and the estimate of the running value at its start.  While the history is indexed, reg_a
            // counts the distinct history ids per region.
            float reg_a[S_MAX_REGIONS], reg_b[S_MAX_REGIONS];
            float reg_t[S_MAX_REGIONS];      // a logit below this adds exactly nothing to the fold in this region
            // distinct history ids grouped by region: those of region r are the entries rs[r] .. rs[r + 1]
            uint16_t rs[S_MAX_REGIONS + 2];
            uint32_t pmask[S_MAX_REGIONS / 32];   // bit r: region r holds history ids
            uint16_t pid[S_MAX_HASH / 2];    // position inside the region
            uint32_t pval[S_MAX_HASH / 2];   // count, then (after pass 1) the bits of the penalised logit
            // id -> count table while the history is indexed (hkey[H], hcnt[H]), then per-warp staging of a piece
            // while penalties are applied to it (SNW x S_REGION floats)
            union alignas(16) {
                uint32_t hash[2 * S_MAX_HASH];
                float stage[SNW * S_REGION];
            } u;
        };
        FinishArrays fin;
        unsigned long long tpkey[SNT];   // vocabulary-sharded mode: one candidate per thread while a record is ranked
    };
};

static_assert(sizeof(StreamSmem) <= 113 * 1024, "two CTAs per SM");

#define PGS_STICK(slot)                                             \
    do {                                                            \
        if (sl.prof && tid == 0) {                                  \
            const long long now_ = clock64();                       \
            sm.prof_acc[slot] += now_ - tick_;                      \
            tick_ = now_;                                           \
        }                                                           \
    } while (0)

__device__ __forceinline__ float max3f(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// max(|a|, |b|, |c|), NaN if any of them is
__device__ __forceinline__ float absmax3_nan(float a, float b, float c) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(fabsf(a)), "f"(fabsf(b)), "f"(fabsf(c)));
    return r;
}
__device__ __forceinline__ float max_ept(const float (&x)[S_EPT]) {
    static_assert(S_EPT % 8 == 0, "eight logits per round");
    float m[S_EPT / 8];
#pragma unroll
    for (int j = 0; j < S_EPT; j += 8)
        m[j / 8] = max3f(max3f(x[j], x[j + 1], x[j + 2]), max3f(x[j + 3], x[j + 4], x[j + 5]), fmaxf(x[j + 6], x[j + 7]));
    float r = m[0];
#pragma unroll
    for (int j = 1; j + 1 < S_EPT / 8; j += 2) r = max3f(r, m[j], m[j + 1]);
    if ((S_EPT / 8) % 2 == 0) r = fmaxf(r, m[S_EPT / 8 - 1]);
    return r;
}
__device__ __forceinline__ float absmax_ept_nan(float am, const float (&x)[S_EPT]) {
    float m[S_EPT / 8];
#pragma unroll
    for (int j = 0; j < S_EPT; j += 8)
        m[j / 8] = absmax3_nan(absmax3_nan(x[j], x[j + 1], x[j + 2]), absmax3_nan(x[j + 3], x[j + 4], x[j + 5]), absmax3_nan(x[j + 6], x[j + 7], x[j + 7]));
#pragma unroll
    for (int j = 0; j + 1 < S_EPT / 8; j += 2) am = absmax3_nan(am, m[j], m[j + 1]);
    if ((S_EPT / 8) % 2 == 1) am = absmax3_nan(am, m[S_EPT / 8 - 1], m[S_EPT / 8 - 1]);
    return am;
}

// One piece's share of a thread as it comes from memory: f32 rows eight 128-bit groups of four logits, bf16 rows
// four groups of eight.
template <bool BF16> struct Geo {
    static constexpr int G = BF16 ? S_EPT / 8 : S_EPT / 4;   // groups per thread and piece
    static constexpr int GE = S_EPT / G;        // logits per group
    static constexpr int GS = 32 * GE;          // logits between two groups of a thread
};

// id of the thread's j-th logit of a piece whose first group starts at e0
template <bool BF16> __device__ __forceinline__ uint32_t elem_id(uint32_t e0, int j) {
    return e0 + (uint32_t)(j / Geo<BF16>::GE) * Geo<BF16>::GS + (uint32_t)(j % Geo<BF16>::GE);
}

// ---- CTA-wide exclusive scans for SNW warps (one barrier each; `slots` may be written again after another barrier)
__device__ __forceinline__ uint32_t sblock_excl_scan_u32(uint32_t v, uint32_t* total, uint32_t* slots) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) slots[w] = inc;
    __syncthreads();
    const uint32_t x = lane < SNW ? slots[lane] : 0u;
    *total = __reduce_add_sync(FULL, x);
    return __reduce_add_sync(FULL, lane < w ? x : 0u) + inc - v;
}
__device__ __forceinline__ float sblock_excl_scan_f32(float v, float* total, float* slots) {   // plain adds: estimates only
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) slots[w] = inc;
    __syncthreads();
    const float x = lane < SNW ? slots[lane] : 0.0f;
    float xi = x;
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(FULL, xi, o);
        if (lane >= o) xi += t;
    }
    *total = __shfl_sync(FULL, xi, 31);
    return __shfl_sync(FULL, xi - x, w) + (inc - v);
}

// One thread reads and validates a row's parameters (same rules as the general kernel).
template <bool BF16>
__device__ __forceinline__ void sprepare_row(const RowArgs& a, const StreamLaunch& sl, uint32_t row, SRowCtl& c) {
    const uint32_t V = a.vocab;
    const float temp = a.temperature ? a.temperature[row] : 0.0f;
    // (vocabulary-sharded mode: the record's length takes the place of top-k; top-p and the draw belong to the merge)
    const uint32_t top_k = a.tp_records ? a.tp_cand : a.top_k ? a.top_k[row] : 0u;
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
        if (h1 < h0 || h1 - h0 > a.max_history || (h1 > h0 && !a.hist_ids)) bad = true; else nh = h1 - h0;
    }
    const bool greedy = temp < 1e-5f;
    const bool use_k = top_k != 0u && top_k < V;
    const char* rowp = (const char*)a.logits + (size_t)row * a.row_stride * (BF16 ? 2 : 4);
    const bool aligned = (((uintptr_t)rowp & 15) == 0) && (V % Geo<BF16>::GE) == 0;
    const bool pen = nh > 0 && (!(fabsf(freq) < 1e-6f && fabsf(pres) < 1e-6f) || rep != 1.0f);
    const bool defer = !aligned || (!greedy && (!use_k || top_k > (uint32_t)S_KMAX)) || (pen && 2u * nh > sl.hash_slots);
    c.rowp = rowp; c.mw = mw; c.temp = temp; c.freq = freq; c.pres = pres; c.rep = rep; c.top_p = top_p; c.u01 = u01;
    const double scale_d = 1.4426950408889634 / (double)fmaxf(temp, 1e-9f);
    // rounded down, so that the second float is positive and a masked entry (-inf) stays -inf through both products
    float sc_hi = (float)scale_d;
    if ((double)sc_hi >= scale_d) sc_hi = u2f(f2u(sc_hi) - 1u);
    c.sc = sc_hi;
    c.sc_lo = (float)(scale_d - (double)sc_hi);
    c.top_k = top_k; c.gflags = gflags; c.h0 = h0; c.nh = nh;
    c.kind = bad ? 1u : defer ? 2u : 0u;
}

// Vocabulary-sharded mode: the candidates of one row (n <= SNT, one per thread) -> this shard's record: the
// tp_cand largest by (logit descending, id ascending) behind the head.  Called by every thread; the caller has a
// barrier in front.
__device__ __forceinline__ void semit_tp(StreamSmem& sm, const RowArgs& a, uint32_t row, uint32_t n, float m, float S,
                                         uint32_t amax) {
    const int tid = threadIdx.x;
    TpRecHead* head = reinterpret_cast<TpRecHead*>(a.tp_records + (size_t)row * a.tp_rec_bytes);
    float* rx = reinterpret_cast<float*>(head + 1);
    uint32_t* rid = reinterpret_cast<uint32_t*>(rx + a.tp_cand);
    const uint32_t want = a.tp_cand < n ? a.tp_cand : n;
    if ((uint32_t)tid < n)
        sm.tpkey[tid] = ((unsigned long long)order_key(sm.cand_x[tid]) << 32) | (unsigned long long)(0xffffffffu - sm.cand_id[tid]);
    __syncthreads();
    if ((uint32_t)tid < n) {
        const unsigned long long kj = sm.tpkey[tid];
        uint32_t r = 0;
#pragma unroll 8
        for (uint32_t o = 0; o < n; o++) r += sm.tpkey[o] > kj;
        if (r < want) { rx[r] = sm.cand_x[tid]; rid[r] = a.id_base + sm.cand_id[tid]; }
    }
    if (tid == 0) tp_write_head(a, row, m, S, want, ROW_OK, amax);
}

// ------------------------------------------------------------------------------------------------------------
// The two passes.  Their loops over the whole pieces of a row are functions of their own (not inlined), so that
// the registers of each loop are allocated for that loop alone (sixteen logits and a dozen values of state: no
// spills in the loops).  What they need to know about the row is in shared
// memory (PassArgs); the ragged last piece of a row, if any, is handled by the caller with the same piece code.

template <bool BF16> struct Raw;
template <> struct Raw<false> { float4 v[4]; };
template <> struct Raw<true> { uint4 v[2]; };

// a whole piece: no bounds checks
template <bool BF16>
__device__ __forceinline__ void raw_load(Raw<BF16>& r, const char* p) {
    constexpr int G = Geo<BF16>::G, STEP = Geo<BF16>::GS * (BF16 ? 2 : 4);
#pragma unroll
    for (int h = 0; h < G; h++) {
        if constexpr (BF16) r.v[h] = __ldcg(reinterpret_cast<const uint4*>(p + h * STEP));
        else r.v[h] = __ldcg(reinterpret_cast<const float4*>(p + h * STEP));
    }
}
// the ragged last piece: groups past the end of the row read as zeros
template <bool BF16>
__device__ __forceinline__ void raw_load_tail(Raw<BF16>& r, const char* p, uint32_t e0, uint32_t V) {
    constexpr int G = Geo<BF16>::G, GS = Geo<BF16>::GS, STEP = GS * (BF16 ? 2 : 4);
#pragma unroll
    for (int h = 0; h < G; h++) {
        if constexpr (BF16) r.v[h] = e0 + h * GS < V ? __ldcg(reinterpret_cast<const uint4*>(p + h * STEP)) : make_uint4(0u, 0u, 0u, 0u);
        else r.v[h] = e0 + h * GS < V ? __ldcg(reinterpret_cast<const float4*>(p + h * STEP)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
}
template <bool BF16>
__device__ __forceinline__ void raw_unpack(float (&x)[S_EPT], const Raw<BF16>& r) {
    if constexpr (BF16) {
#pragma unroll
        for (int h = 0; h < Geo<true>::G; h++) {
            const uint32_t u4[4] = {r.v[h].x, r.v[h].y, r.v[h].z, r.v[h].w};
#pragma unroll
            for (int u = 0; u < 4; u++) {   // a 16-bit shift widens bf16 to f32 exactly
                x[h * 8 + 2 * u] = __uint_as_float(u4[u] << 16);
                x[h * 8 + 2 * u + 1] = __uint_as_float(u4[u] & 0xffff0000u);
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < Geo<false>::G; h++) { x[4 * h] = r.v[h].x; x[4 * h + 1] = r.v[h].y; x[4 * h + 2] = r.v[h].z; x[4 * h + 3] = r.v[h].w; }
    }
}

// Raw logits of piece q -> the logits the chain sees: penalties (through the warp's staging area: the owner of a
// history id is whichever lane holds it), grammar mask / end of row, EOS fix.  PASS 1 computes the penalised
// values and leaves them where the counts were; PASS 2 takes them from there.
template <bool BF16, bool MASK, bool TAIL, int PASS>
__device__ __forceinline__ void fix_x(StreamSmem& sm, float (&x)[S_EPT], uint32_t q) {
    constexpr int G = Geo<BF16>::G, GE = Geo<BF16>::GE, GS = Geo<BF16>::GS;
    const PassArgs& pa = sm.pa;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const uint32_t region = q * SNW + (uint32_t)w;
    if ((pa.flags & PF_PEN) && ((sm.pmask[region >> 5] >> (region & 31u)) & 1u)) {   // warp-uniform
        float* stg = sm.u.stage + w * S_REGION;
        const uint32_t c0 = sm.rs[region], c1 = sm.rs[region + 1];
#pragma unroll
        for (int j = 0; j < S_EPT; j += 4)
            *reinterpret_cast<float4*>(stg + (j / GE) * GS + lane * GE + (j % GE)) = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
        __syncwarp();
#pragma unroll 1
        for (uint32_t i = c0 + lane; i < c1; i += 32) {
            const uint32_t off = sm.pid[i];
            if (PASS == 1) {
                float v = stg[off];
                if (pa.flags & PF_REP) v = v > 0.0f ? fdiv(v, pa.rep) : fmul(v, pa.rep);
                if (pa.flags & PF_FP) {
                    v = fsub(v, fmul(pa.freq, (float)sm.pval[i]));
                    if (pa.flags & PF_PRES) v = fsub(v, pa.pres);
                }
                v = finite_f(v) ? v : -INFINITY;   // an overflowed penalty counts as masked
                stg[off] = v;
                sm.pval[i] = f2u(v);
            } else {
                stg[off] = u2f(sm.pval[i]);
            }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < S_EPT; j += 4) {
            const float4 v = *reinterpret_cast<const float4*>(stg + (j / GE) * GS + lane * GE + (j % GE));
            x[j] = v.x; x[j + 1] = v.y; x[j + 2] = v.z; x[j + 3] = v.w;
        }
        __syncwarp();   // the next piece's staging must not overtake these reads
    }
    if (MASK || TAIL) {
        const uint32_t e0 = q * S_PIECE + (uint32_t)w * S_REGION + (uint32_t)lane * GE;
        const uint32_t mshift = ((uint32_t)lane * GE) & 31u;
#pragma unroll
        for (int h = 0; h < G; h++) {
            const uint32_t idx = e0 + h * GS;
            uint32_t bits = 0xffffffffu;
            if (MASK) bits = (!TAIL || idx < pa.V) ? __ldg(pa.mw + (idx >> 5)) >> mshift : 0u;
            else if (idx >= pa.V) bits = 0u;
#pragma unroll
            for (int c = 0; c < GE; c++)
                if (!((bits >> c) & 1u)) x[h * GE + c] = -INFINITY;
        }
        if (MASK && q == pa.eos_piece && threadIdx.x == pa.eos_tid) {   // the EOS fix (engine.rs:1307-1312)
#pragma unroll
            for (int j = 0; j < S_EPT; j++)
                if ((uint32_t)j == pa.eos_sub && !finite_f(x[j])) x[j] = 0.0f;
        }
    }
}

// pass 1 on one piece
template <bool BF16, bool MASK, bool TAIL, bool STOCH>
__device__ __forceinline__ void p1_piece(StreamSmem& sm, const Raw<BF16>& raw, uint32_t q, float& am, float& tmx, uint32_t& tqx) {
    float x[S_EPT];
    raw_unpack<BF16>(x, raw);
    am = absmax_ept_nan(am, x);   // max |raw logit|, NaN-propagating: the sanity check
    fix_x<BF16, MASK, TAIL, 1>(sm, x, q);
    const float pm = max_ept(x);
    if (pm >= tmx) { tmx = pm; tqx = q; }   // pieces arrive in descending order: an equal maximum here has the lower id
    if (STOCH) {
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
        const float sc = sm.pa.sc;
        // one of the per-thread maxima that bound the top-k threshold
        const uint32_t ci = (q % S_NCELL) * SNT + threadIdx.x;
        if (pm > sm.cell[ci]) sm.cell[ci] = pm;
        // plain sum of the numerators of the warp's 512 logits, relative to their own maximum
        const uint32_t pb = f2u(pm);
        const uint32_t wkey = __reduce_max_sync(FULL, pb ^ (((uint32_t)((int32_t)pb >> 31)) | 0x80000000u));   // monotone; -inf lowest
        const float wm = u2f((wkey & 0x80000000u) ? (wkey & 0x7fffffffu) : ~wkey);
        const float cc = -wm * sc;
        float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
        for (int j = 0; j < S_EPT; j += 4) {
            p0 += ex2_approx_ftz(__fmaf_rn(x[j], sc, cc));
            p1 += ex2_approx_ftz(__fmaf_rn(x[j + 1], sc, cc));
            p2 += ex2_approx_ftz(__fmaf_rn(x[j + 2], sc, cc));
            p3 += ex2_approx_ftz(__fmaf_rn(x[j + 3], sc, cc));
        }
        // summed over the warp in fixed point (a lane's sum is at most 16, and an estimate is all that is needed); an
        // all-masked region has NaN here, which converts to 0
        const uint32_t ws = __reduce_add_sync(FULL, __float2uint_rn(((p0 + p1) + (p2 + p3)) * 1048576.0f));
        if (lane == 0) {
            const uint32_t region = q * SNW + (uint32_t)w;
            sm.reg_a[region] = wm; sm.reg_b[region] = (float)ws * (1.0f / 1048576.0f);
        }
    }
}

// This warp's share of the fold (the same value in all its lanes): a count of ulps of the binade cur_bb, folded into
// accd whenever the binade changes.
struct FoldAcc {
    double accd;
    unsigned long long cur_n;
    uint32_t cur_bb;
    __device__ __forceinline__ void flush() {
        accd += (double)cur_n * ((double)u2f(cur_bb) * 1.1920928955078125e-07);   // units of that binade's ulp
        cur_n = 0ull;
    }
};

// pass 2 on one piece
template <bool BF16, bool MASK, bool TAIL, bool CL = false>
__device__ __forceinline__ void p2_piece(StreamSmem& sm, const Raw<BF16>& raw, uint32_t q, FoldAcc& fa) {
    constexpr int G = Geo<BF16>::G, GE = Geo<BF16>::GE;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const float sc = sm.pa.sc, c_hi = sm.pa.c_hi, c_lo = sm.pa.c_lo, cut_f = sm.pa.cut_f;
    float x[S_EPT];
    raw_unpack<BF16>(x, raw);
    fix_x<BF16, MASK, TAIL, 2>(sm, x, q);
    const float pm = max_ept(x);
    if (pm >= cut_f) {
        const uint32_t e0 = q * S_PIECE + (uint32_t)w * S_REGION + (uint32_t)lane * GE;
#pragma unroll
        for (int j = 0; j < S_EPT; j++)
            if (x[j] >= cut_f) {
                if (CL) {
                    const uint32_t at = atomicAdd(sm.pa.cand_n_p, 1u);
                    if (at < (uint32_t)F_MCAP) { sm.pa.cand_id_p[at] = elem_id<BF16>(e0, j); sm.pa.cand_x_p[at] = x[j]; }
                } else {
                    const uint32_t at = atomicAdd(&sm.cand_n, 1u);
                    if (at < (uint32_t)F_MCAP) { sm.cand_id[at] = elem_id<BF16>(e0, j); sm.cand_x[at] = x[j]; }
                }
            }
    }
    const uint32_t region = q * SNW + (uint32_t)w;
    if (TAIL && region >= sm.pa.n_regions) return;   // warp-uniform: past the end of the row
    // nothing here is large enough to move the running value: the usual case once the sum has grown
    if (__all_sync(FULL, pm < sm.reg_t[region])) return;
    if (BF16) {
        // bf16 rows hold every value thousands of times, and a numerator that is off by 1e-6 in the same direction for
        // all of them moves whole groups of additions across a rounding boundary: scale and constant as two floats
        const float sc_lo = sm.pa.sc_lo;
#pragma unroll
        for (int j = 0; j < S_EPT; j++) x[j] = __fmaf_rn(x[j], sc, c_hi) + __fmaf_rn(x[j], sc_lo, c_lo);   // -inf stays -inf
    } else {
#pragma unroll
        for (int j = 0; j < S_EPT; j++) x[j] = __fmaf_rn(x[j], sc, c_hi);   // -inf stays -inf
        if (c_lo != 0.0f) {   // CTA-uniform: the constant needs its second float (cold rows, large maxima)
#pragma unroll
            for (int j = 0; j < S_EPT; j++) x[j] += c_lo;
        }
    }
#pragma unroll
    for (int j = 0; j < S_EPT; j++) x[j] = ex2_approx_ftz(x[j]);   // -inf -> 0
    const float base = sm.reg_a[region];
    const uint32_t bb = f2u(base);
    const bool quick = bb != 0u;
    if (quick) {
        // every thread from the lower end of the binade the fold is in (the table guarantees that nobody leaves it);
        // four chains: the increments do not depend on the order
        float ac[4] = {base, base, base, base};
#pragma unroll
        for (int j = 0; j < S_EPT / 4; j++) {
#pragma unroll
            for (int c = 0; c < 4; c++) ac[c] = fadd(ac[c], x[c * (S_EPT / 4) + j]);
        }
        const uint32_t ws = __reduce_add_sync(FULL, ((f2u(ac[0]) - bb) + (f2u(ac[1]) - bb)) + ((f2u(ac[2]) - bb) + (f2u(ac[3]) - bb)));   // < 32 * 2^25
        if (bb != fa.cur_bb) { fa.flush(); fa.cur_bb = bb; }
        fa.cur_n += ws;
    }
    if (!quick) {
        // the running value may leave its binade here (or the fold starts here): every 128-bit group from its own
        // estimate of the running value, real additions, so that a crossing is reproduced
        float stv[G], run = 0.0f;
#pragma unroll
        for (int h = 0; h < G; h++) {
            float gs = 0.0f;
#pragma unroll
            for (int c = 0; c < GE; c++) gs += x[h * GE + c];
            float inc = gs;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(FULL, inc, o);
                if (lane >= o) inc += up;
            }
            stv[h] = run + (inc - gs);
            run += __shfl_sync(FULL, inc, 31);
        }
        const float R0 = sm.reg_b[region];
        float tinc = 0.0f;
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float R = fadd(R0, stv[h]);
            float a2 = R;
#pragma unroll
            for (int c = 0; c < GE; c++) a2 = fadd(a2, x[h * GE + c]);
            tinc = fadd(tinc, fsub(a2, R));
        }
        double td = (double)tinc;
#pragma unroll
        for (int o = 16; o; o >>= 1) td += __shfl_xor_sync(FULL, td, o);
        fa.accd += td;
    }
}

// The loops below wait for their loads with nothing else to do (there are no registers for a second piece), so the
// pieces they will need next are requested ahead of time as plain L2 prefetches: memory stays busy while the warps
// compute, and the loads that follow find their lines in L2.  One 128-byte line per lane of the lower half-warp.
#ifndef PGS_PF_DIST
#define PGS_PF_DIST 2
#endif
template <bool BF16>
__device__ __forceinline__ void prefetch_piece(const char* warp_piece) {
    constexpr int LINES = S_REGION * (BF16 ? 2 : 4) / 128;   // 16 (f32) or 8 (bf16)
    const int lane = threadIdx.x & 31;
    if (lane < LINES) asm volatile("prefetch.global.L2 [%0];" ::"l"(warp_piece + lane * 128));
}

// pass 1 over the whole pieces n_full-1 .. 0; the thread's results go to sm.t_*[tid]
template <bool BF16, bool MASK, bool STOCH, bool CL>
__device__ __noinline__ void pass1_whole(StreamSmem& sm) {
    constexpr int PB = S_PIECE * (BF16 ? 2 : 4);
    const uint32_t lane_e0 = (threadIdx.x >> 5) * S_REGION + (threadIdx.x & 31) * Geo<BF16>::GE;
    const uint32_t n = sm.pa.n_full;   // >= 1
    if (CL) {   // the pieces q0, q0 + qstep, ... of the row, last one first
        float am = 0.0f, tmx = -INFINITY;
        uint32_t tqx = 0u;
        const int q0 = (int)sm.pa.q0, qs = (int)sm.pa.qstep;
        if (q0 < (int)n) {
            int q = q0 + (((int)n - 1 - q0) / qs) * qs;
            const size_t step = (size_t)qs * PB;
            const char* p = sm.pa.rowp + (size_t)lane_e0 * (BF16 ? 2 : 4) + (size_t)q * PB;
            const char* wp = sm.pa.rowp + (size_t)((threadIdx.x >> 5) * S_REGION) * (BF16 ? 2 : 4) + (size_t)q * PB;
            if (q - qs >= q0) prefetch_piece<BF16>(wp - step);
#pragma unroll 1
            for (; q >= q0; q -= qs, p -= step, wp -= step) {
                if (q - 2 * qs >= q0) prefetch_piece<BF16>(wp - 2 * step);
                Raw<BF16> b;
                raw_load<BF16>(b, p);
                p1_piece<BF16, MASK, false, STOCH>(sm, b, (uint32_t)q, am, tmx, tqx);
            }
        }
        sm.t_am[threadIdx.x] = am; sm.t_max[threadIdx.x] = tmx; sm.t_q[threadIdx.x] = tqx;
        return;
    }
    const char* p = sm.pa.rowp + (size_t)lane_e0 * (BF16 ? 2 : 4) + (size_t)(n - 1u) * PB;
    float am = 0.0f, tmx = -INFINITY;
    uint32_t tqx = 0u;
    const char* wp = sm.pa.rowp + (size_t)((threadIdx.x >> 5) * S_REGION) * (BF16 ? 2 : 4) + (size_t)(n - 1u) * PB;   // the warp's 512 logits of a piece
#pragma unroll 1
    for (uint32_t d = 1; d < (uint32_t)PGS_PF_DIST && d < n; d++) prefetch_piece<BF16>(wp - (size_t)d * PB);
#pragma unroll 1
    for (uint32_t q = n; q-- > 0u; p -= PB, wp -= PB) {
        if (q >= (uint32_t)PGS_PF_DIST) prefetch_piece<BF16>(wp - (size_t)PGS_PF_DIST * PB);
        Raw<BF16> b;
        raw_load<BF16>(b, p);
        p1_piece<BF16, MASK, false, STOCH>(sm, b, q, am, tmx, tqx);
    }
    sm.t_am[threadIdx.x] = am; sm.t_max[threadIdx.x] = tmx; sm.t_q[threadIdx.x] = tqx;
}

// pass 2 over the whole pieces 0 .. n_full-1; the warp's share of the fold is added to sm.wacc[w]
template <bool BF16, bool MASK, bool CL>
__device__ __noinline__ void pass2_whole(StreamSmem& sm) {
    constexpr int PB = S_PIECE * (BF16 ? 2 : 4);
    const uint32_t lane_e0 = (threadIdx.x >> 5) * S_REGION + (threadIdx.x & 31) * Geo<BF16>::GE;
    const uint32_t n = sm.pa.n_full;   // >= 1
    const char* p = sm.pa.rowp + (size_t)lane_e0 * (BF16 ? 2 : 4);
    FoldAcc fa;
    fa.accd = 0.0; fa.cur_n = 0ull; fa.cur_bb = 0u;
    if (CL) {   // the pieces q0, q0 + qstep, ... of the row, first one first
        const uint32_t q0 = sm.pa.q0, qs = sm.pa.qstep;
        const size_t step = (size_t)qs * PB;
        p += (size_t)q0 * PB;
        const char* wp = sm.pa.rowp + (size_t)((threadIdx.x >> 5) * S_REGION) * (BF16 ? 2 : 4) + (size_t)q0 * PB;
        if (q0 + qs < n) prefetch_piece<BF16>(wp + step);
#pragma unroll 1
        for (uint32_t q = q0; q < n; q += qs, p += step, wp += step) {
            if (q + 2u * qs < n) prefetch_piece<BF16>(wp + 2 * step);
            Raw<BF16> b;
            raw_load<BF16>(b, p);
            p2_piece<BF16, MASK, false, true>(sm, b, q, fa);
        }
        fa.flush();
        if ((threadIdx.x & 31) == 0) sm.wacc[threadIdx.x >> 5] += fa.accd;
        return;
    }
    const char* wp = sm.pa.rowp + (size_t)((threadIdx.x >> 5) * S_REGION) * (BF16 ? 2 : 4);
#pragma unroll 1
    for (uint32_t d = 1; d < (uint32_t)PGS_PF_DIST && d < n; d++) prefetch_piece<BF16>(wp + (size_t)d * PB);
#pragma unroll 1
    for (uint32_t q = 0u; q < n; q++, p += PB, wp += PB) {
        if (q + (uint32_t)PGS_PF_DIST < n) prefetch_piece<BF16>(wp + (size_t)PGS_PF_DIST * PB);
        Raw<BF16> b;
        raw_load<BF16>(b, p);
        p2_piece<BF16, MASK, false>(sm, b, q, fa);
    }
    fa.flush();
    if ((threadIdx.x & 31) == 0) sm.wacc[threadIdx.x >> 5] += fa.accd;
}

// CL: a thread-block cluster of 2, 4 or 8 CTAs shares every row (small batches: a row alone on one CTA is bound by
// the latency of its own loads and dependent instructions).  CTA k of the cluster takes the pieces k, k + size, ...;
// the CTAs exchange their maxima, region tables, histograms, candidates and fold shares through distributed shared
// memory around four cluster barriers per row, and the first CTA finishes the row.  Every decision that ends a row
// early is taken from values all CTAs of the cluster hold alike, so they always meet at the same barriers.
template <bool BF16, bool CL>
__global__ void __launch_bounds__(SNT, 2) stream_row_kernel(const RowArgs a, const StreamLaunch sl) {
    namespace cg = cooperative_groups;
    constexpr int GE = Geo<BF16>::GE, GS = Geo<BF16>::GS;
    constexpr int ESZ = BF16 ? 2 : 4;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    StreamSmem& sm = *reinterpret_cast<StreamSmem*>(smem_raw);
    const uint32_t H = sl.hash_slots;
    uint32_t* hkey = sm.u.hash;
    uint32_t* hcnt = sm.u.hash + H;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const uint32_t V = a.vocab;
    const uint32_t n_full = V / S_PIECE;                        // whole pieces
    const bool has_tail = (V % S_PIECE) != 0u;                  // plus a ragged one at the end of the row
    const uint32_t n_regions = (V + S_REGION - 1) / S_REGION;
    const uint32_t lane_e0 = (uint32_t)w * S_REGION + (uint32_t)lane * GE;   // first element of the thread inside a piece
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    if (tid == 0)
#pragma unroll 1
        for (int i = 0; i < 16; i++) sm.prof_acc[i] = 0;
    constexpr int PREP_TID = SNT - 32;   // lane 0 of the last warp
    uint32_t crank = 0u, csize = 1u;
    if (CL) { crank = cg::this_cluster().block_rank(); csize = cg::this_cluster().num_blocks(); }
    const uint32_t first_row = CL ? blockIdx.x / csize : blockIdx.x, row_step = CL ? gridDim.x / csize : gridDim.x;
    const uint32_t tail_owner = n_full % csize;   // the CTA that takes the ragged piece
    if (tid == PREP_TID && first_row < a.rows) sprepare_row<BF16>(a, sl, first_row, sm.ctl[0]);
    long long tick_ = clock64();
    uint32_t it = 0;
    for (uint32_t row = first_row; row < a.rows; row += row_step, it++) {
        // ---- gate: at most `cohort` rows ahead of the rows that have left their first pass
        if (!CL && tid == 0 && row >= sl.cohort) {
            const uint32_t need = row - sl.cohort + 1u;
            const volatile uint32_t* done = sl.p1_done;
#pragma unroll 1
            for (uint32_t poll = 0; poll < sl.gate_polls; poll++) {
                if (*done - sl.done_base >= need) break;
                __nanosleep(200);
            }
        }
        // this row's parameters are complete, and every warp is done with the row before
        __syncthreads();
        PGS_STICK(0);   // gate + row barrier
        const SRowCtl& ctl = sm.ctl[it & 1];
        if (tid == PREP_TID && row + row_step < a.rows) sprepare_row<BF16>(a, sl, row + row_step, sm.ctl[(it + 1) & 1]);
        const bool writer = tid == 0 && crank == 0u;   // one thread of the row's (first) CTA
        if (ctl.kind != 0u) {
            if (writer) {
                if (ctl.kind == 1u) {
                    if (a.tp_records) tp_write_head(a, row, -INFINITY, 0.0f, 0u, ROW_BAD_PARAM, 0u);
                    else { a.token[row] = 0; a.status[row] = ROW_BAD_PARAM; if (a.drew) a.drew[row] = 0; }
                } else sl.work_rows[atomicAdd(sl.work_count, 1u)] = row;
                atomicAdd(sl.p1_done, 1u);
            }
            continue;
        }
        const float temp = ctl.temp;
        const uint32_t top_k = ctl.top_k, gflags = ctl.gflags, h0 = ctl.h0, nh = ctl.nh;
        const char* rowp = ctl.rowp;
        const float sc = ctl.sc;
        const bool greedy = temp < 1e-5f;
        const bool has_mask = ctl.mw != nullptr;
        const bool do_fp = !(fabsf(ctl.freq) < 1e-6f && fabsf(ctl.pres) < 1e-6f);
        const bool do_rep = ctl.rep != 1.0f;
        const bool pen = nh > 0 && (do_fp || do_rep);
        if (tid == 0) {   // what the pass loops read
            PassArgs& pa = sm.pa;
            pa.rowp = rowp; pa.mw = ctl.mw; pa.sc = sc; pa.sc_lo = ctl.sc_lo; pa.c_hi = 0.0f; pa.c_lo = 0.0f; pa.cut_f = 0.0f;
            pa.freq = ctl.freq; pa.pres = ctl.pres; pa.rep = ctl.rep;
            pa.V = V; pa.n_full = n_full; pa.n_regions = n_regions;
            pa.q0 = crank; pa.qstep = csize;
            pa.cand_n_p = &sm.cand_n; pa.cand_id_p = sm.cand_id; pa.cand_x_p = sm.cand_x;
            if (CL) {
                cg::cluster_group cluster = cg::this_cluster();
                pa.cand_n_p = cluster.map_shared_rank(&sm.cand_n, 0);
                pa.cand_id_p = cluster.map_shared_rank(sm.cand_id, 0);
                pa.cand_x_p = cluster.map_shared_rank(sm.cand_x, 0);
            }
            pa.flags = (pen ? PF_PEN : 0u) | (do_rep ? PF_REP : 0u) | (do_fp ? PF_FP : 0u) | (fabsf(ctl.pres) > 1e-6f ? PF_PRES : 0u);
            // the EOS fix touches one logit: where it sits in the piece / thread / register layout
            pa.eos_piece = 0xffffffffu; pa.eos_tid = 0u; pa.eos_sub = 0u;
            if (has_mask && (gflags & 1u) && a.eos >= 0 && (uint32_t)a.eos < V) {
                const uint32_t r = (uint32_t)a.eos % S_PIECE, p = r % S_REGION;
                pa.eos_piece = (uint32_t)a.eos / S_PIECE;
                pa.eos_tid = (r / S_REGION) * 32u + (p % GS) / GE;
                pa.eos_sub = (p / GS) * GE + p % GE;
            }
        }

        // the pieces the first pass starts with are requested now, so that they arrive while the history is indexed
        if (n_full > 0u) {
            constexpr int PB = S_PIECE * ESZ;
            const uint32_t qs = CL ? csize : 1u;
            if (n_full > crank) {
                const uint32_t qlast = crank + ((n_full - 1u - crank) / qs) * qs;
                const char* wp = rowp + (size_t)(w * S_REGION) * ESZ + (size_t)qlast * PB;
                prefetch_piece<BF16>(wp);
                if (qlast >= qs + crank) prefetch_piece<BF16>(wp - (size_t)qs * PB);
            }
        }
        // ---- history: distinct ids with their counts, grouped by the warp region they fall into
        bool defer_row = false;
        if (pen) {
            uint32_t* rcnt = reinterpret_cast<uint32_t*>(sm.reg_a);   // distinct ids per region, then the scatter cursor
            // the first id of every thread is requested before the tables are cleared
            const uint32_t hid0 = (uint32_t)tid < nh ? __ldg(a.hist_ids + h0 + tid) : S_NIL;
#pragma unroll 1
            for (uint32_t s = tid; s < H; s += SNT) { hkey[s] = S_NIL; hcnt[s] = 0u; }
#pragma unroll 1
            for (uint32_t r = tid; r < n_regions; r += SNT) rcnt[r] = 0u;
#pragma unroll 1
            for (uint32_t r = tid; r < (uint32_t)(S_MAX_REGIONS / 32); r += SNT) sm.pmask[r] = 0u;
            __syncthreads();
            int spilled = 0;
#pragma unroll 1
            for (uint32_t j = tid; j < nh; j += SNT) {
                const uint32_t id = (j == (uint32_t)tid ? hid0 : __ldg(a.hist_ids + h0 + j)) - a.id_base;   // ids below a shard wrap around
                if (id >= V) continue;   // engine.rs:1562
                uint32_t s = (id * 2654435761u) & (H - 1u);
                bool placed = false;
#pragma unroll 1
                for (int probe = 0; probe < 128; probe++) {
                    const uint32_t prev = atomicCAS(&hkey[s], S_NIL, id);
                    if (prev == S_NIL) {
                        atomicAdd(&rcnt[id / S_REGION], 1u);
                        atomicOr(&sm.pmask[id / (S_REGION * 32)], 1u << ((id / S_REGION) & 31u));
                    }
                    if (prev == S_NIL || prev == id) { atomicAdd(&hcnt[s], 1u); placed = true; break; }
                    s = (s + 1u) & (H - 1u);
                }
                if (!placed) spilled = 1;
            }
            spilled = __syncthreads_or(spilled);
            if (spilled && !CL) {   // CTA-uniform
                if (writer) { sl.work_rows[atomicAdd(sl.work_count, 1u)] = row; atomicAdd(sl.p1_done, 1u); }
                continue;
            }
            // (A cluster must meet at its barriers whatever one of its CTAs finds here: the CTA goes through the first
            // pass without penalties and says so in the exchange behind it, where all CTAs give the row up together.)
            if (CL && spilled) { defer_row = true; if (tid == 0) sm.pa.flags = 0u; }
            if (!spilled) {
            // exclusive scan of the counts in region order; thread t owns the regions t * rpt ..
            const uint32_t rpt = (n_regions + SNT - 1) / SNT;   // <= S_RPT
            uint32_t cnt[S_RPT], own = 0u;
#pragma unroll
            for (int j = 0; j < S_RPT; j++) {
                const uint32_t r = (uint32_t)tid * rpt + j;
                cnt[j] = ((uint32_t)j < rpt && r < n_regions) ? rcnt[r] : 0u;
                own += cnt[j];
            }
            uint32_t total;
            uint32_t before = sblock_excl_scan_u32(own, &total, sm.scan_u);
#pragma unroll
            for (int j = 0; j < S_RPT; j++) {
                const uint32_t r = (uint32_t)tid * rpt + j;
                if ((uint32_t)j < rpt && r < n_regions) { sm.rs[r] = (uint16_t)before; rcnt[r] = before; }
                before += cnt[j];
            }
            if (tid == 0) sm.rs[n_regions] = (uint16_t)total;
            __syncthreads();
#pragma unroll 1
            for (uint32_t s = tid; s < H; s += SNT) {
                const uint32_t id = hkey[s];
                if (id == S_NIL) continue;
                const uint32_t at = atomicAdd(&rcnt[id / S_REGION], 1u);
                sm.pid[at] = (uint16_t)(id % S_REGION);
                sm.pval[at] = hcnt[s];
            }
            }
        }
#pragma unroll
        for (int c = 0; c < S_NCELL; c++) sm.cell[c * SNT + tid] = -INFINITY;
        __syncthreads();   // the id -> count table is dead from here on (its space is the staging area); PassArgs are set
        PGS_STICK(1);   // history indexed

        // ================================================================ pass 1 (HBM, last piece first)
        float am = 0.0f;            // max |raw logit|
        float tmx = -INFINITY;      // the thread's running maximum, and the lowest piece that holds it
        uint32_t tqx = 0u;
        const bool my_tail = has_tail && (!CL || tail_owner == crank);
        if (my_tail) {
            Raw<BF16> raw;
            raw_load_tail<BF16>(raw, rowp + ((size_t)n_full * S_PIECE + lane_e0) * ESZ, n_full * S_PIECE + lane_e0, V);
            if (has_mask) { if (greedy) p1_piece<BF16, true, true, false>(sm, raw, n_full, am, tmx, tqx); else p1_piece<BF16, true, true, true>(sm, raw, n_full, am, tmx, tqx); }
            else { if (greedy) p1_piece<BF16, false, true, false>(sm, raw, n_full, am, tmx, tqx); else p1_piece<BF16, false, true, true>(sm, raw, n_full, am, tmx, tqx); }
        }
        if (n_full > 0u) {
            if (has_mask) { if (greedy) pass1_whole<BF16, true, false, CL>(sm); else pass1_whole<BF16, true, true, CL>(sm); }
            else { if (greedy) pass1_whole<BF16, false, false, CL>(sm); else pass1_whole<BF16, false, true, CL>(sm); }
            am = absmax3_nan(am, sm.t_am[tid], 0.0f);
            if (sm.t_max[tid] >= tmx) { tmx = sm.t_max[tid]; tqx = sm.t_q[tid]; }   // the whole pieces come before the ragged one
        }
        PGS_STICK(2);   // pass 1

        // ---- row maximum, sanity, and the material for the top-k bound
        {
            uint32_t lo = 0xffffffffu, fin = 0u;
            if (!greedy) {
#pragma unroll
                for (int c = 0; c < S_NCELL; c++) {
                    const uint32_t k = order_key(sm.cell[c * SNT + tid]);
                    if (!k) continue;
                    lo = umin(lo, k);
                    fin++;
                }
            }
            const uint32_t wk = __reduce_max_sync(FULL, order_key(tmx));
            const uint32_t wlo = __reduce_min_sync(FULL, lo);
            const uint32_t wfin = __reduce_add_sync(FULL, fin);
            const uint32_t wbad = __any_sync(FULL, !(am < INFINITY)) ? 1u : 0u;
            if (lane == 0) { sm.red_key[w] = wk; sm.red_lo[w] = wlo; sm.red_fin[w] = wfin; sm.red_flag[w] = wbad; sm.wacc[w] = 0.0; }
#pragma unroll
            for (int u = 0; u < S_BPT; u++) sm.hist[u * SNT + tid] = 0u;
            if (tid == 0) { sm.cand_n = 0u; sm.sel_bucket = 0u; sm.amax = 0xffffffffu; }
        }
        __syncthreads();
        uint32_t gkey = __reduce_max_sync(FULL, lane < SNW ? sm.red_key[lane] : 0u);
        uint32_t lo_key = __reduce_min_sync(FULL, lane < SNW ? sm.red_lo[lane] : 0xffffffffu);
        uint32_t n_fin = __reduce_add_sync(FULL, lane < SNW ? sm.red_fin[lane] : 0u);
        bool nonfinite = __any_sync(FULL, lane < SNW && sm.red_flag[lane] != 0u);
        if (CL) {
            // First barrier: every CTA of the cluster is through its first pass, so nobody still uses the space of the
            // region table for its history counts, and everybody is done with the row before.  Then every CTA hands its
            // part of the region table and its four numbers to all the others; second barrier; combine.
            cg::cluster_group cluster = cg::this_cluster();
            cluster.sync();
            if (!greedy) {
#pragma unroll 1
                for (uint32_t r = tid; r < n_regions; r += SNT) {
                    const uint32_t q = r / SNW;
                    if ((q < n_full ? q % csize : tail_owner) != crank) continue;
                    const float ra = sm.reg_a[r], rb = sm.reg_b[r];
                    for (uint32_t k = 0; k < csize; k++) {
                        if (k == crank) continue;
                        *cluster.map_shared_rank(&sm.reg_a[r], k) = ra;
                        *cluster.map_shared_rank(&sm.reg_b[r], k) = rb;
                    }
                }
            }
            if ((uint32_t)tid < csize) {
                *cluster.map_shared_rank(&sm.xk[crank], tid) = gkey;
                *cluster.map_shared_rank(&sm.xlo[crank], tid) = lo_key;
                *cluster.map_shared_rank(&sm.xfin[crank], tid) = n_fin;
                *cluster.map_shared_rank(&sm.xflag[crank], tid) = (nonfinite ? 1u : 0u) | (defer_row ? 2u : 0u);
            }
            cluster.sync();
            gkey = 0u; lo_key = 0xffffffffu; n_fin = 0u; nonfinite = false; defer_row = false;
            for (uint32_t k = 0; k < csize; k++) {
                gkey = umax(gkey, sm.xk[k]); lo_key = umin(lo_key, sm.xlo[k]); n_fin += sm.xfin[k];
                nonfinite |= (sm.xflag[k] & 1u) != 0u; defer_row |= (sm.xflag[k] & 2u) != 0u;
            }
        }
        const bool any = gkey != 0u;
        const float m = any ? key_to_float(gkey) : -INFINITY;
        const int status = any ? ROW_OK : ROW_EMPTY;
        if (writer) atomicAdd(sl.p1_done, 1u);
        // ---- argmax: the lowest id that holds the maximum.  Every thread whose own maximum is the row's looks at
        // the lowest of its pieces that holds it once more (the penalised values are in place by now).
        if (any && !nonfinite && !(gflags & 2u)) {
            // (the piece code is a warp-wide operation, so a warp goes through the pieces its lanes ask for one by
            // one; nearly always that is a single piece of a single warp)
            unsigned pending = __ballot_sync(FULL, order_key(tmx) == gkey);
#pragma unroll 1
            while (pending) {   // warp-uniform
                const uint32_t q = __shfl_sync(FULL, tqx, __ffs(pending) - 1);
                Raw<BF16> raw;
                raw_load_tail<BF16>(raw, rowp + ((size_t)q * S_PIECE + lane_e0) * ESZ, q * S_PIECE + lane_e0, V);
                float x[S_EPT];
                raw_unpack<BF16>(x, raw);
                if (has_mask) fix_x<BF16, true, true, 2>(sm, x, q); else fix_x<BF16, false, true, 2>(sm, x, q);
                const bool mine = ((pending >> lane) & 1u) && tqx == q;
                if (mine) {
                    int j0 = 0;
#pragma unroll
                    for (int j = S_EPT - 1; j >= 0; j--) if (x[j] == m) j0 = j;
                    atomicMin(&sm.amax, elem_id<BF16>(q * S_PIECE + lane_e0, j0));
                }
                pending &= ~__ballot_sync(FULL, mine);
            }
            __syncthreads();
        }
        uint32_t amax = any ? sm.amax : 0u;
        if (defer_row || nonfinite || (gflags & 2u) || greedy || !any) {
            if (CL) {   // the lowest id over all CTAs; the first CTA writes the row
                cg::cluster_group cluster = cg::this_cluster();
                if (tid == 0) *cluster.map_shared_rank(&sm.xam[crank], 0) = sm.amax;
                cluster.sync();
                if (crank != 0u) continue;
                uint32_t am_all = 0xffffffffu;
                for (uint32_t k = 0; k < csize; k++) am_all = umin(am_all, sm.xam[k]);
                amax = any ? am_all : 0u;
            }
            if (defer_row) {   // (cluster mode only) a CTA could not index the history: the general kernel takes the row
                if (writer) sl.work_rows[atomicAdd(sl.work_count, 1u)] = row;
                continue;
            }
            if (writer && a.tp_records) {
                if (nonfinite) {
                    tp_write_head(a, row, NAN, 0.0f, 0u, ROW_NONFINITE, 0u);
                    if (a.faulted) atomicAdd(a.faulted, 1ull);
                } else if (gflags & 2u) tp_write_head(a, row, -INFINITY, 0.0f, 0u, ROW_DEAD, 0u);
                else tp_write_head(a, row, m, 0.0f, 0u, ROW_OK, amax);   // greedy or empty: maximum + argmax alone
            } else if (writer) {
                if (nonfinite) {
                    a.token[row] = 0; a.status[row] = ROW_NONFINITE; if (a.drew) a.drew[row] = 0;
                    if (a.faulted) atomicAdd(a.faulted, 1ull);
                } else if (gflags & 2u) {
                    a.token[row] = 0; a.status[row] = ROW_DEAD; if (a.drew) a.drew[row] = 0;
                } else {
                    a.token[row] = amax; a.status[row] = status;
                    if (a.drew) a.drew[row] = 0;
                    if (a.argmax) a.argmax[row] = amax;
                    if (a.row_max) a.row_max[row] = m;
                    if (a.sumexp) a.sumexp[row] = 0.0f;
                    if (a.total) a.total[row] = 0.0f;
                    if (a.n_kept) a.n_kept[row] = 0u;
                }
            }
            PGS_STICK(3);
            continue;
        }

        PGS_STICK(6);   // reductions + argmax
        // ---- top-k bound.  The per-thread maxima are spread over S_NB equal-width buckets between their
        // smallest finite value and the row maximum (a monotone map); with b the highest bucket such that the
        // buckets b.. hold at least top_k maxima, every logit of bucket b - 1 or higher is a candidate.
        const float t = fmaxf(temp, 1e-9f);
        float cut = -INFINITY;
        if (n_fin >= top_k) {   // CTA-uniform
            const float lo_v = key_to_float(lo_key);
            const float scb = m > lo_v ? (float)(S_NB - 1) / (m - lo_v) : 0.0f;
#pragma unroll
            for (int c = 0; c < S_NCELL; c++) {
                const float cv = sm.cell[c * SNT + tid];
                if (finite_f(cv)) atomicAdd(&sm.hist[min((uint32_t)(S_NB - 1), (uint32_t)((cv - lo_v) * scb))], 1u);
            }
            __syncthreads();
            // thread j owns the S_BPT buckets S_NB-1 - j*S_BPT - u; `above` = maxima in higher buckets
            uint32_t hv[S_BPT], own = 0u;
            if (CL) {   // third barrier: the histograms of all CTAs stand; every CTA adds them up for itself
                cg::cluster_group cluster = cg::this_cluster();
                cluster.sync();
#pragma unroll
                for (int u = 0; u < S_BPT; u++) {
                    hv[u] = 0u;
                    for (uint32_t k = 0; k < csize; k++) hv[u] += *cluster.map_shared_rank(&sm.hist[(S_NB - 1) - tid * S_BPT - u], k);
                    own += hv[u];
                }
            } else
#pragma unroll
            for (int u = 0; u < S_BPT; u++) { hv[u] = sm.hist[(S_NB - 1) - tid * S_BPT - u]; own += hv[u]; }
            uint32_t total;
            uint32_t above = sblock_excl_scan_u32(own, &total, sm.scan_u);
#pragma unroll
            for (int u = 0; u < S_BPT; u++) {
                if (above < top_k && top_k <= above + hv[u]) sm.sel_bucket = (uint32_t)((S_NB - 1) - tid * S_BPT - u);
                above += hv[u];
            }
            __syncthreads();
            const uint32_t bsel = sm.sel_bucket;
            const float bound = (bsel >= 1u && scb > 0.0f) ? lo_v + ((float)bsel - 1.0f) / scb : lo_v;
            // every logit whose probability could still tie with the k-th one stays above the cut
            const float delta = 4.8e-7f * (fabsf(m - bound) + 4.0f * t) + 4.8e-7f * (fabsf(bound) + fabsf(m));
            cut = bound - delta;
        }
        PGS_STICK(7);   // top-k bound
        // numerator = 2^(x * sc + c): c = -m * sc as c_hi + c_lo (c_lo only when it matters: the numerators then keep
        // the reference's scale to 1e-7, which the fold needs where many logits are equal); what is left of c scales
        // the final sum
        const double scale_d = BF16 ? (double)sc + (double)ctl.sc_lo : (double)sc;
        const double c_d = -(double)m * scale_d;
        const float c_hi = (float)c_d;
        float c_lo = (float)(c_d - (double)c_hi);
        if (!BF16 && fabsf(c_lo) < 1e-7f) c_lo = 0.0f;
        const double c_rest = c_d - (double)c_hi - (double)c_lo;
        if (tid == 0) { sm.pa.c_hi = c_hi; sm.pa.c_lo = c_lo; sm.pa.cut_f = fmaxf(cut, -3.4e38f); }   // masked entries (-inf) are never candidates

        // ---- where the fold stands at every warp region.  The plain sums overestimate the fold's running value
        // by up to a few 1e-4 (the small terms it drops), so a region takes the quick path only if the whole
        // interval [start * (1 - slack), end * (1 + slack)], slack >= 2^-9, lies inside one binade.
        {
            float carry = 0.0f;
#pragma unroll 1
            for (uint32_t r0 = 0; r0 < n_regions; r0 += SNT) {   // CTA-uniform trip count
                const uint32_t r = r0 + (uint32_t)tid;
                float P = 0.0f;
                if (r < n_regions && sm.reg_b[r] > 0.0f) P = sm.reg_b[r] * ex2_approx_ftz((sm.reg_a[r] - m) * sc);
                float tot;
                const float pre = carry + sblock_excl_scan_f32(P, &tot, sm.scan_f);
                if (r < n_regions) {
                    // (the plain sums carry the rounding of their exponents' constant: 2^-24 of |max * sc|)
                    const float slack = 0.001953125f + 1e-7f * fabsf(m * sc);
                    const float lo_e = pre * (1.0f - slack), hi_e = (pre + P) * (1.0f + slack);
                    const uint32_t kb = f2u(lo_e) & 0x7f800000u;
                    // quick: one binade for the whole region, and the region's own sum stays below that binade's
                    // lower end, so that no thread's additions from there can leave the binade either
                    const bool quick = kb != 0u && kb == (f2u(hi_e) & 0x7f800000u) && P * (1.0f + slack) < 0.999f * u2f(kb);
                    sm.reg_a[r] = quick ? u2f(kb) : 0.0f;
                    sm.reg_b[r] = pre;
                    // A numerator below half an ulp of the running value leaves it unchanged, and lo_e never exceeds the
                    // running value: a logit with x * scale + c < exponent(lo_e) - 24 (less a margin for the hardware
                    // exp2) adds exactly nothing.  In units of logits:
                    float thr = -INFINITY;
                    if (kb != 0u) {
                        const double lim = (double)((int)(kb >> 23) - 127 - 24) - 0.02;
                        thr = (float)((lim - c_d) / scale_d);
                        thr -= 4e-7f * fabsf(thr) + 1e-30f;
                    }
                    sm.reg_t[r] = thr;
                }
                carry += tot;
                __syncthreads();   // scan_f is reused by the next round; after the last one the table and PassArgs are complete
            }
        }
        PGS_STICK(3);   // fold table

        // ================================================================ pass 2 (L2, first piece first)
        if (my_tail) {
            Raw<BF16> raw;
            raw_load_tail<BF16>(raw, rowp + ((size_t)n_full * S_PIECE + lane_e0) * ESZ, n_full * S_PIECE + lane_e0, V);
            FoldAcc fa;
            fa.accd = 0.0; fa.cur_n = 0ull; fa.cur_bb = 0u;
            if (has_mask) p2_piece<BF16, true, true, CL>(sm, raw, n_full, fa); else p2_piece<BF16, false, true, CL>(sm, raw, n_full, fa);
            fa.flush();
            if (lane == 0) sm.wacc[w] += fa.accd;
        }
        if (n_full > 0u) {
            if (has_mask) pass2_whole<BF16, true, CL>(sm); else pass2_whole<BF16, false, CL>(sm);
        }
        __syncthreads();   // the candidate list and the warps' shares are complete
        PGS_STICK(4);   // pass 2
        double s_d = lane < SNW ? sm.wacc[lane] : 0.0;
#pragma unroll
        for (int o = 16; o; o >>= 1) s_d += __shfl_xor_sync(FULL, s_d, o);
        if (CL) {   // the fold shares and the argmax candidates of all CTAs meet in the first one
            cg::cluster_group cluster = cg::this_cluster();
            if (tid == 0) { *cluster.map_shared_rank(&sm.xs[crank], 0) = s_d; *cluster.map_shared_rank(&sm.xam[crank], 0) = sm.amax; }
            cluster.sync();
            if (crank != 0u) continue;
            s_d = 0.0;
            uint32_t am_all = 0xffffffffu;
            for (uint32_t k = 0; k < csize; k++) { s_d += sm.xs[k]; am_all = umin(am_all, sm.xam[k]); }
            amax = am_all;
        }
        const float S = (float)(s_d * exp2(c_rest));
        const uint32_t n_cand = sm.cand_n;
        if (n_cand > (uint32_t)F_MCAP) {   // CTA-uniform
            if (writer) { sl.work_rows[atomicAdd(sl.work_count, 1u)] = row; }
            continue;
        }
        if (a.tp_records) {   // CTA-uniform
            if (n_cand > (uint32_t)SNT) {
                if (writer) { sl.work_rows[atomicAdd(sl.work_count, 1u)] = row; }
                continue;
            }
            semit_tp(sm, a, row, n_cand, m, S, amax);
        } else {
            cta_finish<SNT>(sm.fin, sm.exp_tab, a, row, V, sm.cand_id, sm.cand_x, n_cand, m, t, S, top_k, ctl.top_p, ctl.u01, amax,
                            status);
        }
        PGS_STICK(5);   // finish
    }
    if (sl.prof && tid == 0)
#pragma unroll 1
        for (int i = 0; i < 16; i++) sl.prof[blockIdx.x * 16 + i] += sm.prof_acc[i];
}

size_t stream_smem_bytes() { return sizeof(StreamSmem); }
uint32_t stream_threads() { return SNT; }

template <bool BF16, bool CL>
static cudaError_t configure_one() {
    cudaError_t e = cudaFuncSetAttribute(stream_row_kernel<BF16, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(StreamSmem));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(stream_row_kernel<BF16, CL>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

cudaError_t configure_stream() {
    cudaError_t e = configure_one<false, false>();
    if (e == cudaSuccess) e = configure_one<true, false>();
    if (e == cudaSuccess) e = configure_one<false, true>();
    if (e == cudaSuccess) e = configure_one<true, true>();
    return e;
}

// CTAs of this kernel that one SM holds
cudaError_t stream_ctas_per_sm(int* out) {
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(out, stream_row_kernel<false, false>, SNT, sizeof(StreamSmem));
}

// Clusters of `csize` CTAs of this kernel that the device holds at once (csize 2, 4 or 8)
cudaError_t stream_max_clusters(int csize, int* out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)csize, 1, 1);
    cfg.blockDim = dim3(SNT, 1, 1);
    cfg.dynamicSmemBytes = sizeof(StreamSmem);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)csize; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaOccupancyMaxActiveClusters(out, stream_row_kernel<false, true>, &cfg);
}

// csize == 1: one CTA per row, `grid` CTAs.  csize > 1: `grid` clusters of csize CTAs, one cluster per row at a time.
cudaError_t launch_stream(const RowArgs& a, const StreamLaunch& sl, uint32_t grid, uint32_t csize, cudaStream_t stream) {
    if (csize <= 1u) {
        if (a.dtype == 0) stream_row_kernel<false, false><<<grid, SNT, sizeof(StreamSmem), stream>>>(a, sl);
        else stream_row_kernel<true, false><<<grid, SNT, sizeof(StreamSmem), stream>>>(a, sl);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid * csize, 1, 1);
    cfg.blockDim = dim3(SNT, 1, 1);
    cfg.dynamicSmemBytes = sizeof(StreamSmem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (a.dtype == 0) return cudaLaunchKernelEx(&cfg, stream_row_kernel<false, true>, a, sl);
    return cudaLaunchKernelEx(&cfg, stream_row_kernel<true, true>, a, sl);
}

}  // namespace pgs
