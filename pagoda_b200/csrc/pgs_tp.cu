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

constexpr int TP_LIST = 1024;

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

struct TpRecHead { float m; float s; uint32_t n; uint32_t argmax; };   // then float x[cand], uint32 id[cand]

struct TpPartialSmem {
    ReduceSmem rs;
    SeqSmem seq;
    SelectSmem sel;
    unsigned long long exp_tab[32];
    float lx[TP_LIST];
    uint32_t lid[TP_LIST];
    uint32_t ln;
};

// Copies the finished record of `row` from this rank's gather buffer into the same slot of every other
// rank's (plain stores into peer memory).  Called by the whole CTA after a barrier.
__device__ __forceinline__ void push_record(const TpArgs& a, uint32_t row) {
    if (!a.done) return;
    const uint32_t words = a.rec_bytes / 4u;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.records + (size_t)row * a.rec_bytes);
    for (uint32_t w = threadIdx.x; w < words; w += NT) {
        const uint32_t v = src[w];
        for (uint32_t p = 0; p < a.n_shards; p++)
            if (p != a.shard_rank) reinterpret_cast<uint32_t*>(a.peer_records[p] + (size_t)row * a.rec_bytes)[w] = v;
    }
}

__global__ void __launch_bounds__(NT, 1) tp_partial_kernel(const TpArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TpPartialSmem& sm = *reinterpret_cast<TpPartialSmem*>(smem_raw);
    const int tid = threadIdx.x;
    const uint32_t n = a.shard_vocab;
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    __syncthreads();
    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const float* x = a.logits + (size_t)row * a.row_stride;
        TpRecHead* head = reinterpret_cast<TpRecHead*>(a.records + (size_t)row * a.rec_bytes);
        float* rx = reinterpret_cast<float*>(head + 1);
        uint32_t* rid = reinterpret_cast<uint32_t*>(rx + a.cand);
        const float temp = a.temperature ? a.temperature[row] : 0.0f;
        // shard max / argmax (lowest id) and sanity
        unsigned long long best = 0ull;
        int nonfinite = 0;
        for (uint32_t i = tid; i < n; i += NT) {
            const float v = x[i];
            nonfinite |= !finite_f(v);
            const unsigned long long k = order_key(v);
            if (k) {
                const unsigned long long c = (k << 32) | (unsigned long long)(0xffffffffu - i);
                best = c > best ? c : best;
            }
        }
        nonfinite = __syncthreads_or(nonfinite);
        best = block_max_u64(best, sm.rs);
        if (nonfinite) {   // the merge reports the row as faulted when any shard saw a non-finite logit
            if (tid == 0) { head->m = NAN; head->s = 0.0f; head->n = 0; head->argmax = 0; }
            __syncthreads();
            push_record(a, row);
            continue;
        }
        const float m = best ? key_to_float((uint32_t)(best >> 32)) : -INFINITY;
        const uint32_t amax = best ? a.shard_lo + (0xffffffffu - (uint32_t)best) : 0u;
        float s = 0.0f;
        if (!(temp < 1e-5f)) {
            const float t = fmaxf(temp, 1e-9f);
            s = seq_scan([&](int i) { return softmax_num(x[i], m, t, sm.exp_tab); }, (int)n, 0.0f, SEQ_SUM, 0.0f,
                         nullptr, sm.seq, sm.rs);
        }
        // the `cand` largest by (value descending, id ascending)
        const uint32_t want = a.cand < n ? a.cand : n;
        const uint32_t kk = radix_select_kth([&](int i) { return order_key(x[i]); }, (int)n, want, sm.sel, sm.rs);
        if (tid == 0) sm.ln = 0;
        __syncthreads();
        for (uint32_t i = tid; i < n; i += NT) {   // strictly above the threshold: fewer than `want`
            if (order_key(x[i]) > kk) {
                const uint32_t at = atomicAdd(&sm.ln, 1u);
                sm.lx[at] = x[i]; sm.lid[at] = i;
            }
        }
        __syncthreads();
        const uint32_t n_gt = sm.ln;
        uint32_t filled = n_gt;
        for (uint32_t base = 0; base < n && filled < want; base += NT) {   // ties, lowest ids first
            const uint32_t i = base + tid;
            const uint32_t tie = (i < n && order_key(x[i]) == kk) ? 1u : 0u;
            uint32_t tot;
            const uint32_t at = filled + block_excl_scan_u32(tie, &tot, sm.rs);
            if (tie && at < want) { sm.lx[at] = x[i]; sm.lid[at] = i; }
            filled = min(want, filled + tot);
        }
        __syncthreads();
        for (uint32_t j = tid; j < want; j += NT) {   // rank-sort the `want` entries
            const float v = sm.lx[j];
            const uint32_t id = sm.lid[j];
            uint32_t r = 0;
            for (uint32_t o = 0; o < want; o++) r += (sm.lx[o] > v) || (sm.lx[o] == v && sm.lid[o] < id);
            rx[r] = v;
            rid[r] = a.shard_lo + id;
        }
        if (tid == 0) { head->m = m; head->s = s; head->n = want; head->argmax = amax; }
        __syncthreads();
        push_record(a, row);
    }
    if (a.done) {   // peer-store exchange: the last CTA of the launch raises this shard's flag on every rank
        __threadfence_system();
        __syncthreads();
        if (tid == 0 && atomicAdd(a.done, 1u) == gridDim.x - 1u) {
            *a.done = 0u;
            __threadfence_system();
            for (uint32_t p = 0; p < a.n_shards; p++) st_release_sys(a.peer_flags[p] + a.shard_rank, a.epoch);
        }
    }
}

struct TpMergeSmem {
    FinishSmem fin;
    uint32_t cid[F_MCAP];
    float cx[F_MCAP];
    float M, S;
    uint32_t amax, n;
    int fault;
};


__global__ void __launch_bounds__(NT, 1) tp_merge_kernel(const TpArgs a, const TpOut o) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TpMergeSmem& sm = *reinterpret_cast<TpMergeSmem*>(smem_raw);
    const int tid = threadIdx.x;
    const uint32_t row = blockIdx.x;
    const float temp = a.temperature ? a.temperature[row] : 0.0f;
    const float t = fmaxf(temp, 1e-9f);
    if (tid < 32) sm.fin.exp_tab[tid] = kExp2TableDev[tid];
    if (a.flags) {   // peer-store exchange: wait (bounded, about a second) until every shard has raised its flag
        if (tid == 0) {
            int late = 0;
            for (uint32_t r = 0; r < a.n_shards && !late; r++) {
                uint32_t spin = 0;
                while ((int32_t)(ld_acquire_sys(a.flags + r) - a.epoch) < 0) {
                    if (++spin > (1u << 21)) { late = 1; break; }
                    __nanosleep(500);
                }
            }
            sm.fault = late;
        }
        __syncthreads();
        if (sm.fault) {
            if (tid == 0) { o.token[row] = 0; o.status[row] = ROW_LOAD_TIMEOUT; if (o.drew) o.drew[row] = 0; }
            return;
        }
    }
    __syncthreads();
    auto rec = [&](uint32_t r) {
        return reinterpret_cast<const TpRecHead*>(a.records + ((size_t)r * a.rows + row) * a.rec_bytes);
    };
    if (tid == 0) {
        float M = -INFINITY;
        int fault = 0;
        for (uint32_t r = 0; r < a.n_shards; r++) {
            const float mr = rec(r)->m;
            if (mr != mr) fault = 1; else M = fmaxf(M, mr);
        }
        float S = 0.0f;
        uint32_t n = 0, amax = 0;
        float best = -INFINITY;
        bool have = false;
        for (uint32_t r = 0; r < a.n_shards && !fault; r++) {
            const TpRecHead* h = rec(r);
            if (finite_f(h->m)) {
                // shards are in id order, so strict > keeps the lowest id on ties
                if (!have || h->m > best) { best = h->m; amax = h->argmax; have = true; }
                S = fadd(S, fmul(h->s, pgs_expf_tab(fdiv(fsub(h->m, M), t), sm.fin.exp_tab)));
            }
            n += min(h->n, a.cand);   // a record can never hold more than `cand` entries
        }
        sm.M = M; sm.S = S; sm.amax = amax; sm.n = n; sm.fault = fault;
    }
    __syncthreads();
    if (sm.fault) {
        if (tid == 0) { o.token[row] = 0; o.status[row] = ROW_NONFINITE; if (o.drew) o.drew[row] = 0; }
        return;
    }
    // gather the union of the candidates
    uint32_t off = 0;
    for (uint32_t r = 0; r < a.n_shards; r++) {
        const TpRecHead* h = rec(r);
        const float* rx = reinterpret_cast<const float*>(h + 1);
        const uint32_t* rid = reinterpret_cast<const uint32_t*>(rx + a.cand);
        const uint32_t hn = min(h->n, a.cand);
        for (uint32_t j = tid; j < hn; j += NT) { sm.cx[off + j] = rx[j]; sm.cid[off + j] = rid[j]; }
        off += hn;
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
    finish_row(sm.fin, ra, row, a.vocab, sm.cid, sm.cx, sm.n, sm.M, t, sm.S, 0u, a.top_p ? a.top_p[row] : 1.0f,
               a.uniform ? a.uniform[row] : 0.0f, sm.amax, ROW_OK);
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
    cudaError_t e = cudaFuncSetAttribute(tp_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(TpPartialSmem));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(tp_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(TpMergeSmem));
}

cudaError_t launch_tp_partial(const TpArgs& a, uint32_t grid, cudaStream_t stream) {
    tp_partial_kernel<<<grid, NT, sizeof(TpPartialSmem), stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_tp_merge(const TpArgs& a, const TpOut& o, cudaStream_t stream) {
    tp_merge_kernel<<<a.rows, NT, sizeof(TpMergeSmem), stream>>>(a, o);
    return cudaGetLastError();
}

cudaError_t launch_draft_accept(const uint32_t* row_argmax, const uint32_t* draft, uint32_t sequences,
                                uint32_t positions, uint32_t* accepted, uint32_t* next, cudaStream_t stream) {
    draft_accept_kernel<<<(sequences + 127) / 128, 128, 0, stream>>>(row_argmax, draft, sequences, positions, accepted,
                                                                     next);
    return cudaGetLastError();
}

}  // namespace pgs
