// Vocabulary-sharded (tensor-parallel) sampling.  The reference has no multi-GPU code; this mode is
// an extension whose semantics are fixed by the CPU oracle (pgo_tp_sample_row):
//
//   every GPU holds columns [rank * V/n, (rank + 1) * V/n) of every row and emits, per row, one
//   fixed-size record: its max m_r, its own sequential f32 sum s_r = sum exp((x - m_r) / t) (same
//   arithmetic as pagoda/src/sampler.rs:92-114 on the shard), its argmax and its `cand` largest
//   logits by (value descending, id ascending) with their global ids;
//   the records of all shards are gathered on every GPU -- by an NCCL all-gather between the two kernels,
//   or by the emitting kernel itself, which stores its records into every peer's gather buffer over
//   NVLink and then raises a per-shard flag there that the peer's merge kernel waits for (bounded) --
//   and merged on every GPU:
//   M = max m_r, S = sum_r s_r * exp((m_r - M) / t) folded in shard order, candidate probability
//   exp((x - M) / t) / S, then the reference's top-p rule, total and inverse-CDF walk over the
//   union of the candidates; greedy rows take the best candidate, lowest id on ties, which is the
//   global argmax.
//
// Draft verification (pagoda-hf/src/qwen3_5.rs:663-755 returns per-position argmax ids; the accept
// rule itself is defined here): accept while argmax(row j) == draft[j].
#include "pgs_finish.cuh"
#include "pgs_tp.cuh"

namespace pgs {


// system-scope flag accesses: the store publishes everything this GPU wrote before it (records in peer
// memory included), the load makes it visible to the reader
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Peer-store exchange: copies this rank's finished records ([rows x rec_bytes], complete when the kernels in
// front of this one in the stream have ended) into slot [shard_rank] of every other rank's gather buffer with
// plain stores into peer memory; the last CTA then raises this shard's flag on every rank.
__global__ void __launch_bounds__(256) tp_push_kernel(const TpArgs a) {
    cudaGridDependencySynchronize();
    const size_t bytes = (size_t)a.rows * a.rec_bytes;
    const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
    if ((a.rec_bytes & 15u) == 0u) {   // every buffer starts on a 256-byte boundary
        const uint4* src = reinterpret_cast<const uint4*>(a.records);
        for (size_t i = i0; i < bytes / 16; i += step) {
            const uint4 v = src[i];
            for (uint32_t p = 0; p < a.n_shards; p++)
                if (p != a.shard_rank) reinterpret_cast<uint4*>(a.peer_records[p])[i] = v;
        }
    } else {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.records);
        for (size_t i = i0; i < bytes / 4; i += step) {
            const uint32_t v = src[i];
            for (uint32_t p = 0; p < a.n_shards; p++)
                if (p != a.shard_rank) reinterpret_cast<uint32_t*>(a.peer_records[p])[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(a.done, 1u) == gridDim.x - 1u) {
        *a.done = 0u;
        __threadfence_system();
        for (uint32_t p = 0; p < a.n_shards; p++) st_release_sys(a.peer_flags[p] + a.shard_rank, a.epoch);
    }
}

constexpr int TP_MT = 256;    // threads of the merge kernel
constexpr int TP_MCAP = TP_MAX_SHARDS * 128;   // candidates of all shards together (cand <= 128)

struct TpMergeSmem {
    FinishArraysT<TP_MCAP> fin;
    unsigned long long exp_tab[32];
    uint32_t cid[TP_MCAP];
    float cx[TP_MCAP];
    float M, S;
    uint32_t amax, n;
    int fault;   // the row's status when it is not ROW_OK
    uint32_t start[TP_MAX_SHARDS + 1];   // where each shard's candidates begin in cid / cx
    TpRecHead hd[TP_MAX_SHARDS];
    int unsorted;
};


__global__ void __launch_bounds__(TP_MT, 4) tp_merge_kernel(const TpArgs a, const TpOut o) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TpMergeSmem& sm = *reinterpret_cast<TpMergeSmem*>(smem_raw);
    const int tid = threadIdx.x;
    const uint32_t row = blockIdx.x;
    const float temp = a.temperature ? a.temperature[row] : 0.0f;
    const float t = fmaxf(temp, 1e-9f);
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    if (a.flags) {   // peer-store exchange: wait (bounded, about a second) until every shard has raised its flag
        if (tid == 0) {
            int late = 0;
            for (uint32_t r = 0; r < a.n_shards && !late; r++) {
                uint32_t spin = 0;
                while ((int32_t)(ld_acquire_sys(a.flags + r) - a.epoch) < 0) {
                    if (++spin > a.wait_polls) { late = 1; break; }
                    __nanosleep(500);
                }
            }
            sm.fault = late;
        }
        __syncthreads();
        if (sm.fault) {
            if (tid == 0) {
                o.token[row] = 0; o.status[row] = ROW_LOAD_TIMEOUT; if (o.drew) o.drew[row] = 0;
                if (a.timeouts) atomicAdd(a.timeouts, 1ull);
            }
            return;
        }
    }
    __syncthreads();
    auto rec = [&](uint32_t r) {
        return reinterpret_cast<const TpRecHead*>(a.records + ((size_t)r * a.rows + row) * a.rec_bytes);
    };
    const uint32_t top_k = a.top_k ? a.top_k[row] : 0u;
    // every record slot of the row is requested at once (one trip to memory): the heads by the first threads, the
    // candidate slots one or two per thread; which of the slots are filled is known once the heads are in
    if ((uint32_t)tid < a.n_shards) sm.hd[tid] = *rec(tid);
    constexpr int SLOTS = (TP_MCAP + TP_MT - 1) / TP_MT;
    float gx[SLOTS];
    uint32_t gid[SLOTS];
#pragma unroll
    for (int u = 0; u < SLOTS; u++) {
        const uint32_t c = (uint32_t)tid + u * TP_MT;
        gx[u] = 0.0f; gid[u] = 0u;
        if (c < a.n_shards * a.cand) {
            const float* rx = reinterpret_cast<const float*>(rec(c / a.cand) + 1);
            gx[u] = rx[c % a.cand];
            gid[u] = reinterpret_cast<const uint32_t*>(rx + a.cand)[c % a.cand];
        }
    }
    __syncthreads();
    if (tid == 0) {
        float M = -INFINITY;
        int fault = (top_k > a.cand) ? ROW_BAD_PARAM : ROW_OK;   // a record holds the shard's `cand` largest, no more
        bool nonfinite = false, dead = false;
        for (uint32_t r = 0; r < a.n_shards; r++) {
            const float mr = sm.hd[r].m;
            const uint32_t st = sm.hd[r].n_status >> 24;
            if (st == (uint32_t)ROW_BAD_PARAM) fault = ROW_BAD_PARAM;
            nonfinite |= st == (uint32_t)ROW_NONFINITE || mr != mr;
            dead |= st == (uint32_t)ROW_DEAD;
            if (mr == mr) M = fmaxf(M, mr);
        }
        // the order of engine.rs:1292-1303: parameters, then sanity, then the grammar's dead state
        if (fault == ROW_OK) fault = nonfinite ? ROW_NONFINITE : dead ? ROW_DEAD : ROW_OK;
        float S = 0.0f;
        uint32_t n = 0, amax = 0;
        float best = -INFINITY;
        bool have = false;
        for (uint32_t r = 0; r < a.n_shards; r++) {
            const TpRecHead& h = sm.hd[r];
            if (fault == ROW_OK && finite_f(h.m)) {
                // shards are in id order, so strict > keeps the lowest id on ties
                if (!have || h.m > best) { best = h.m; amax = h.argmax; have = true; }
                S = fadd(S, fmul(h.s, pgs_expf_tab(fdiv(fsub(h.m, M), t), sm.exp_tab)));
            }
            sm.start[r] = n;
            n += min(h.n_status & 0xffffffu, a.cand);   // a record can never hold more than `cand` entries
        }
        sm.start[a.n_shards] = n;
        sm.M = M; sm.S = S; sm.amax = amax; sm.n = n; sm.fault = fault;
        sm.unsorted = 0; sm.fin.n_live = 0u;
    }
    __syncthreads();
    if (sm.fault) {
        if (tid == 0) { o.token[row] = 0; o.status[row] = sm.fault; if (o.drew) o.drew[row] = 0; }
        return;
    }
    // the union of the candidates, shard after shard
#pragma unroll
    for (int u = 0; u < SLOTS; u++) {
        const uint32_t c = (uint32_t)tid + u * TP_MT;
        if (c < a.n_shards * a.cand) {
            const uint32_t r = c / a.cand, j = c % a.cand;
            if (j < sm.start[r + 1] - sm.start[r]) { sm.cx[sm.start[r] + j] = gx[u]; sm.cid[sm.start[r] + j] = gid[u]; }
        }
    }
    __syncthreads();
    const bool any = finite_f(sm.M);
    if (o.gmax && tid == 0) o.gmax[row] = sm.M;
    if (temp < 1e-5f || !any) {
        if (tid == 0) {
            o.token[row] = sm.amax; o.status[row] = any ? ROW_OK : ROW_EMPTY;
            if (o.drew) o.drew[row] = 0;
            if (o.argmax) o.argmax[row] = sm.amax;
            if (o.gsum) o.gsum[row] = sm.S;
            if (o.total) o.total[row] = 0.0f;
            if (o.n_kept) o.n_kept[row] = 0;
        }
        return;
    }
    RowArgs ra;
    memset(&ra, 0, sizeof ra);
    ra.token = o.token; ra.status = o.status; ra.drew = o.drew; ra.argmax = o.argmax; ra.sumexp = o.gsum;
    ra.total = o.total; ra.n_kept = o.n_kept;
    ra.row_max = nullptr;
    const float top_p = a.top_p ? a.top_p[row] : 1.0f, u01 = a.uniform ? a.uniform[row] : 0.0f;
    // Every shard's candidates arrive sorted by (logit descending, id ascending), and shards follow one another in id
    // order.  So a candidate's rank among all of them is a sum of binary searches, one per shard, and its place in id
    // order needs a count inside its own shard only: no sort.  The searches are by (probability, id); two different
    // logits can round to one probability, which may leave a shard's list out of that order: such a row (looked for
    // below) takes the general ranking instead.
    const uint32_t n = sm.n;
    const bool norm = sm.S > 1e-9f;
    for (uint32_t c = tid; c < n; c += TP_MT) {
        const float e = softmax_num(sm.cx[c], sm.M, t, sm.exp_tab);   // exact expf
        sm.fin.key[c] = ((unsigned long long)f2u(norm ? fdiv(e, sm.S) : e) << 32) | (unsigned long long)(0xffffffffu - sm.cid[c]);
    }
    __syncthreads();
    for (uint32_t c = tid; c + 1 < n; c += TP_MT) {
        uint32_t r = 0;
        while (sm.start[r + 1] <= c) r++;
        if (c + 1 < sm.start[r + 1] && !(sm.fin.key[c] > sm.fin.key[c + 1])) sm.unsorted = 1;
    }
    __syncthreads();
    if (sm.unsorted) {   // CTA-uniform
        cta_finish<TP_MT>(sm.fin, sm.exp_tab, ra, row, a.vocab, sm.cid, sm.cx, n, sm.M, t, sm.S, top_k, top_p, u01, sm.amax, ROW_OK);
        return;
    }
    for (uint32_t c = tid; c < n; c += TP_MT) {
        const unsigned long long kc = sm.fin.key[c];
        uint32_t own = 0;
        while (sm.start[own + 1] <= c) own++;
        uint32_t r_p = 0;
        for (uint32_t r = 0; r < a.n_shards; r++) {   // keys of shard r that come before kc: the list is descending
            uint32_t lo = sm.start[r], hi = sm.start[r + 1];
            const uint32_t base = lo;
            while (lo < hi) {
                const uint32_t mid = (lo + hi) >> 1;
                if (sm.fin.key[mid] > kc) lo = mid + 1; else hi = mid;
            }
            r_p += lo - base;
        }
        uint32_t r_id = sm.start[own];
        const uint32_t idc = sm.cid[c];
        for (uint32_t o2 = sm.start[own]; o2 < sm.start[own + 1]; o2++) r_id += sm.cid[o2] < idc;
        const float pc = u2f((uint32_t)(kc >> 32));
        sm.fin.sid[r_id] = idc; sm.fin.sp[r_id] = pc; sm.fin.rp[r_p] = pc; sm.fin.rpos[r_p] = r_id;
    }
    cta_finish_ranked<TP_MT>(sm.fin, ra, row, a.vocab, n, sm.M, sm.S, top_k, top_p, u01, sm.amax, ROW_OK);
}

__global__ void draft_accept_kernel(const uint32_t* row_argmax, const uint32_t* draft, uint32_t sequences,
                                    uint32_t positions, uint32_t* accepted, uint32_t* next) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= sequences || positions == 0) return;
    uint32_t acc = 0;
    while (acc < positions && row_argmax[s * positions + acc] == draft[s * positions + acc]) acc++;
    accepted[s] = acc;
    next[s] = row_argmax[s * positions + (acc < positions ? acc : positions - 1)];
}

cudaError_t configure_tp() {
    cudaError_t e = cudaFuncSetAttribute(tp_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(TpMergeSmem));
    if (e != cudaSuccess) return e;
    // several rows per SM: most of a row's time is one warp's serial walk
    return cudaFuncSetAttribute(tp_merge_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

cudaError_t launch_tp_push(const TpArgs& a, cudaStream_t stream) {
    const size_t units = ((size_t)a.rows * a.rec_bytes) / 16 + 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((units + 255) / 256 < 64 ? (units + 255) / 256 : 64), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, tp_push_kernel, a);
}

cudaError_t launch_tp_merge(const TpArgs& a, const TpOut& o, cudaStream_t stream) {
    tp_merge_kernel<<<a.rows, TP_MT, sizeof(TpMergeSmem), stream>>>(a, o);
    return cudaGetLastError();
}

cudaError_t launch_draft_accept(const uint32_t* row_argmax, const uint32_t* draft, uint32_t sequences,
                                uint32_t positions, uint32_t* accepted, uint32_t* next, cudaStream_t stream) {
    draft_accept_kernel<<<(sequences + 127) / 128, 128, 0, stream>>>(row_argmax, draft, sequences, positions, accepted,
                                                                     next);
    return cudaGetLastError();
}

}  // namespace pgs
