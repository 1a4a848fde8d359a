// Finish kernel: one CTA per batch row turns the record the fused kernel left behind (row max,
// the f32 sum, a short candidate list that contains the whole top-k set) into a token.  All rows
// run side by side, so the short serial folds of one row overlap with those of every other row.
#include "pgs_finish.cuh"

namespace pgs {

constexpr int FS_NT = 128;   // rows with at most this many candidates take finish_small_kernel

// (At most 48 registers per thread: a CTA of this kernel must fit on an SM beside the CTAs of
// finish_small_kernel, or the usually empty pass would queue behind them and lengthen every step.)
__global__ void __maxnreg__(48) finish_kernel(const RowArgs a, const FusedLaunch fl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FinishSmem& sm = *reinterpret_cast<FinishSmem*>(smem_raw);
    // a small grid walks the rows: usually none of them has a long list, and the pass must then cost next to nothing
    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        if (fl.recs[row].kind != 1u || fl.recs[row].n_cand <= (uint32_t)FS_NT) continue;   // small rows: finish_small_kernel
        const RowRec& rec = fl.recs[row];
        if (threadIdx.x < 32) {   // the partial folds of the row, added up by one warp
            double s2 = 0.0;
            for (uint32_t r = threadIdx.x; r < rec.n_parts; r += 32) s2 += rec.part[r];
            for (int o = 16; o; o >>= 1) s2 += __shfl_xor_sync(FULL, s2, o);
            if (threadIdx.x == 0) sm.bcast_f = (float)s2;
        }
        __syncthreads();
        const float S = sm.bcast_f;   // finish_row opens with a barrier before anything reuses the slot
        finish_row(sm, a, row, a.vocab, fl.cand_id + (size_t)row * F_MCAP, fl.cand_x + (size_t)row * F_MCAP, rec.n_cand,
                   rec.m, rec.t, S, a.top_k ? a.top_k[row] : 0u, a.top_p ? a.top_p[row] : 1.0f,
                   a.uniform ? a.uniform[row] : 0.0f, rec.amax, rec.status);
        __syncthreads();
    }
}

// ---- small rows: at most 128 candidates (top-k 50 leaves about 60).  Four warps per row are enough,
// every row of the batch is resident at once, and the exact folds are short serial chains of one lane.

struct alignas(16) FinishSmallSmem {
    unsigned long long exp_tab[32];
    unsigned long long key[FS_NT];   // (probability bits << 32) | ~id: one comparison ranks by (p descending, id ascending)
    float p[FS_NT];                  // scratch of the folds
    uint32_t sid[FS_NT];
    float sp[FS_NT];
    float rp[FS_NT];
    uint32_t rpos[FS_NT];
    uint32_t n_live;
    float S;
};

__global__ void __launch_bounds__(FS_NT) finish_small_kernel(const RowArgs a, const FusedLaunch fl) {
    __shared__ FinishSmallSmem sm;
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t row = blockIdx.x;
    const RowRec& rec = fl.recs[row];
    // the record's header first (one cache line); everything else the row needs is then requested at once, so
    // that the kernel pays two round trips to memory, not one per item
    const uint32_t n = rec.n_cand, V = a.vocab;
    if (rec.kind != 1u || n > (uint32_t)FS_NT) return;
    const uint32_t n_parts = rec.n_parts;
    const float m = rec.m, t = rec.t;
    const uint32_t top_k = a.top_k ? a.top_k[row] : 0u;
    const float top_p = a.top_p ? a.top_p[row] : 1.0f;
    const float u01 = a.uniform ? a.uniform[row] : 0.0f;
    const uint32_t my_id = (uint32_t)tid < n ? fl.cand_id[(size_t)row * F_MCAP + tid] : 0u;
    const float my_x = (uint32_t)tid < n ? fl.cand_x[(size_t)row * F_MCAP + tid] : 0.0f;
    if (tid < 32) {
        sm.exp_tab[tid] = kExp2TableDev[tid];
        double s2 = 0.0;
#pragma unroll 1
        for (uint32_t r0 = 0; r0 < n_parts; r0 += 128) {   // four independent loads per lane and round
            double q[4];
#pragma unroll
            for (int u = 0; u < 4; u++) q[u] = r0 + u * 32 + lane < n_parts ? rec.part[r0 + u * 32 + lane] : 0.0;
            s2 += (q[0] + q[1]) + (q[2] + q[3]);
        }
        for (int o = 16; o; o >>= 1) s2 += __shfl_xor_sync(FULL, s2, o);
        if (tid == 0) { sm.S = (float)s2; sm.n_live = 0; }
    }
    __syncthreads();
    const float S = sm.S;
    const bool norm = S > 1e-9f;
    float my_p = 0.0f;
    if ((uint32_t)tid < n) {
        const float e = softmax_num(my_x, m, t, sm.exp_tab);   // exact expf
        my_p = norm ? fdiv(e, S) : e;
        sm.key[tid] = ((unsigned long long)f2u(my_p) << 32) | (unsigned long long)(0xffffffffu - my_id);   // p >= 0
    }
    __syncthreads();
    if ((uint32_t)tid < n) {   // rank by id and by (probability descending, id ascending)
        const unsigned long long kj = sm.key[tid];
        uint32_t r_id = 0, r_p = 0;
#pragma unroll 8
        for (uint32_t o = 0; o < n; o++) {   // broadcast loads, independent of one another: requested in batches
            const unsigned long long ko = sm.key[o];
            r_p += ko > kj;
            r_id += (uint32_t)ko > (uint32_t)kj;   // larger ~id = smaller id
        }
        sm.sid[r_id] = my_id; sm.sp[r_id] = my_p; sm.rp[r_p] = my_p; sm.rpos[r_p] = r_id;
    }
    __syncthreads();
    if ((uint32_t)tid < n) {   // top-k: every tie at the k-th probability survives; zeros never matter
        const float thr = (top_k != 0u && top_k <= n) ? sm.rp[top_k - 1] : 0.0f;
        const bool live = sm.rp[tid] >= thr && sm.rp[tid] > 0.0f;
        const bool next_live = (uint32_t)tid + 1 < n && sm.rp[tid + 1] >= thr && sm.rp[tid + 1] > 0.0f;
        if (live && !next_live) sm.n_live = tid + 1;
    }
    __syncthreads();
    if (tid >= 32) return;
    // one warp: top-p walk in ranked order, then total and inverse-CDF pick in id order
    const uint32_t n_live = sm.n_live;
    uint32_t keep = n_live;
    if (!(top_p >= 1.0f) && n_live > 0) {
        warp_prefix(sm.rp, (int)n_live, sm.p);   // sm.p is free once the candidates are ranked
        const int found = warp_find(sm.p, (int)n_live, SEQ_FIND_GE, top_p);
        if (found >= 0) keep = (uint32_t)found + 1;
    }
    for (uint32_t j = keep + lane; j < n; j += 32) sm.sp[sm.rpos[j]] = 0.0f;
    __syncwarp();
    const float total = warp_prefix(sm.sp, (int)n, sm.p);
    int pick = -1;
    if (total > 1e-9f) pick = warp_find(sm.p, (int)n, SEQ_FIND_GT, fmul(u01, total));
    if (lane == 0) {
        uint32_t token = rec.amax;
        int drew = 0;
        if (total > 1e-9f) { token = pick >= 0 ? sm.sid[pick] : V - 1; drew = 1; }
        a.token[row] = token; a.status[row] = rec.status;
        if (a.drew) a.drew[row] = (uint8_t)drew;
        if (a.argmax) a.argmax[row] = rec.amax;
        if (a.row_max) a.row_max[row] = m;
        if (a.sumexp) a.sumexp[row] = S;
        if (a.total) a.total[row] = total;
    }
    if (a.n_kept || a.dump_ids || a.dump_probs) {   // diagnostics: the kept set in id order
        uint32_t done = 0;
        for (uint32_t base = 0; base < n; base += 32) {
            const uint32_t j = base + lane;
            const bool kept = j < n && sm.sp[j] > 0.0f;
            const unsigned mask = __ballot_sync(FULL, kept);
            const uint32_t at = done + __popc(mask & ((1u << lane) - 1u));
            if (kept && at < a.dump_cap) {
                if (a.dump_ids) a.dump_ids[(size_t)row * a.dump_cap + at] = sm.sid[j];
                if (a.dump_probs) a.dump_probs[(size_t)row * a.dump_cap + at] = sm.sp[j];
            }
            done += __popc(mask);
        }
        if (lane == 0 && a.n_kept) a.n_kept[row] = done;
    }
}

cudaError_t launch_finish_small(const RowArgs& a, const FusedLaunch& fl, cudaStream_t stream) {
    finish_small_kernel<<<a.rows, FS_NT, 0, stream>>>(a, fl);
    return cudaGetLastError();
}

cudaError_t configure_finish() {
    return cudaFuncSetAttribute(finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FinishSmem));
}

cudaError_t launch_finish(const RowArgs& a, const FusedLaunch& fl, cudaStream_t stream) {
    finish_kernel<<<a.rows < 128u ? a.rows : 128u, NT, sizeof(FinishSmem), stream>>>(a, fl);
    return cudaGetLastError();
}

}  // namespace pgs
