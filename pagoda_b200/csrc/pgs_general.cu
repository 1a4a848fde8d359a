// General row kernel: one 1024-thread CTA walks one batch row through the whole chain of
// Engine::advance_with_logits (pagoda/src/engine.rs:1286-1314) with its working copy of the row
// in a global-memory scratch slot.  It accepts every shape and parameter combination (any vocab
// size or alignment, top-k off, top-p without top-k, thousands of tied candidates, long
// histories) and is the path rows take when the streaming row kernel cannot serve them.
//
// Order of operations per row, as the reference runs them:
//   sanity (engine.rs:1278-1295) -> repetition* / frequency / presence penalties
//   (engine.rs:1553-1573; * extension) -> grammar bitmask (grammar.rs:73-85) -> EOS fix
//   (engine.rs:1307-1312) -> argmax (sampler.rs:59-70) or temperature softmax, top-k, top-p and
//   the inverse-CDF walk (sampler.rs:28-55, 92-150).
#include "pgs_args.cuh"
#include "pgs_block.cuh"

#include <cuda_bf16.h>

namespace pgs {

struct GeneralSmem {
    ReduceSmem rs;
    SeqSmem seq;
    SelectSmem sel;
    unsigned long long sort_tile[SORT_TILE];
    unsigned long long exp_tab[32];
};

__device__ __forceinline__ float load_logit(const void* base, uint32_t dtype, size_t i) {
    if (dtype == 0) return ((const float*)base)[i];
    return __uint_as_float((uint32_t)((const unsigned short*)base)[i] << 16);
}

__device__ __forceinline__ void write_row(const RowArgs& a, uint32_t row, uint32_t token, int status,
                                          int drew, uint32_t amax, float rmax, float sumexp,
                                          float total, uint32_t n_kept) {
    a.token[row] = token;
    a.status[row] = status;
    if (a.drew) a.drew[row] = (uint8_t)drew;
    if (a.argmax) a.argmax[row] = amax;
    if (a.row_max) a.row_max[row] = rmax;
    if (a.sumexp) a.sumexp[row] = sumexp;
    if (a.total) a.total[row] = total;
    if (a.n_kept) a.n_kept[row] = n_kept;
}

// Vocabulary-sharded mode: the shard's record of one row from its processed logits X (penalties, mask and EOS fix
// applied).  The `tp_cand` largest finite logits by (value descending, id ascending), then the shard's f32
// left-fold sum (which overwrites X).  Called by the whole CTA.
__device__ __forceinline__ void tp_emit_row(const RowArgs& a, GeneralSmem& sm, uint32_t row, float* X, uint32_t V, bool any,
                                            float m, uint32_t amax, float temp, const unsigned long long* tab) {
    const int tid = threadIdx.x;
    if (!any || temp < 1e-5f) {   // greedy rows travel as maximum + argmax alone
        if (tid == 0) tp_write_head(a, row, m, 0.0f, 0u, ROW_OK, amax);
        return;
    }
    float* lx = reinterpret_cast<float*>(sm.sort_tile);
    uint32_t* lid = reinterpret_cast<uint32_t*>(sm.sort_tile) + 1024;
    uint32_t* ln = reinterpret_cast<uint32_t*>(sm.sort_tile) + 2048;
    TpRecHead* head = reinterpret_cast<TpRecHead*>(a.tp_records + (size_t)row * a.tp_rec_bytes);
    float* rx = reinterpret_cast<float*>(head + 1);
    uint32_t* rid = reinterpret_cast<uint32_t*>(rx + a.tp_cand);
    uint32_t fin = 0;
    for (uint32_t i = tid; i < V; i += NT) fin += order_key(X[i]) != 0u;
    uint32_t n_fin;
    block_excl_scan_u32(fin, &n_fin, sm.rs);
    const uint32_t want = a.tp_cand < n_fin ? a.tp_cand : n_fin;   // >= 1: the row has a finite maximum
    const uint32_t kk = radix_select_kth([&](int i) { return order_key(X[i]); }, (int)V, want, sm.sel, sm.rs);
    if (tid == 0) *ln = 0;
    __syncthreads();
    for (uint32_t i = tid; i < V; i += NT) {   // strictly above the threshold: fewer than `want`
        if (order_key(X[i]) > kk) {
            const uint32_t at = atomicAdd(ln, 1u);
            lx[at] = X[i]; lid[at] = i;
        }
    }
    __syncthreads();
    uint32_t filled = *ln;
    for (uint32_t base = 0; base < V && filled < want; base += NT) {   // ties, lowest ids first
        const uint32_t i = base + tid;
        const uint32_t tie = (i < V && order_key(X[i]) == kk) ? 1u : 0u;
        uint32_t tot;
        const uint32_t at = filled + block_excl_scan_u32(tie, &tot, sm.rs);
        if (tie && at < want) { lx[at] = X[i]; lid[at] = i; }
        filled = min(want, filled + tot);
    }
    __syncthreads();
    for (uint32_t j = tid; j < want; j += NT) {   // rank-sort the `want` entries
        const float v = lx[j];
        const uint32_t id = lid[j];
        uint32_t r = 0;
        for (uint32_t o = 0; o < want; o++) r += (lx[o] > v) || (lx[o] == v && lid[o] < id);
        rx[r] = v;
        rid[r] = a.id_base + id;
    }
    const float t = fmaxf(temp, 1e-9f);
    const float s = seq_scan([&](int i) { return softmax_num(X[i], m, t, tab); }, (int)V, 0.0f, SEQ_SUM, 0.0f, nullptr,
                             sm.seq, sm.rs);
    if (tid == 0) tp_write_head(a, row, m, s, want, ROW_OK, amax);
}

__global__ void __launch_bounds__(NT, 1) general_row_kernel(const RowArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    GeneralSmem& sm = *reinterpret_cast<GeneralSmem*>(smem_raw);
    const int tid = threadIdx.x;
    const uint32_t V = a.vocab;
    const uint32_t slot = blockIdx.x;
    if (a.work_rows) cudaGridDependencySynchronize();   // the work-list pass is launched ahead of the end of the kernel that fills the list
    const uint32_t n_work = a.work_rows ? *a.work_count : a.rows;
    if (n_work == 0u) return;   // the usual case of the work-list pass: nothing listed, nothing to reset
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    __syncthreads();
    const unsigned long long* tab = sm.exp_tab;

    for (uint32_t w = blockIdx.x; w < n_work; w += gridDim.x) {
        const uint32_t row = a.work_rows ? a.work_rows[w] : w;
        __syncthreads();
        // ---------------------------------------------------------------- parameters
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
        const bool tp = a.tp_records != nullptr;
        if (bad) {
            if (tid == 0) {
                if (tp) tp_write_head(a, row, -INFINITY, 0.0f, 0u, ROW_BAD_PARAM, 0u);
                else write_row(a, row, 0u, ROW_BAD_PARAM, 0, 0u, -INFINITY, 0.0f, 0.0f, 0u);
            }
            continue;
        }

        // ------------------------------------------------ sanity + upcast + grammar bitmask
        float* X = a.sx + (size_t)slot * a.vocab_pad;
        const char* rowp = (const char*)a.logits + (size_t)row * a.row_stride * (a.dtype == 0 ? 4 : 2);
        int nonfinite = 0;
        if (a.dtype == 0 && (((uintptr_t)rowp & 15) == 0) && (V & 3) == 0) {
            const float4* src = (const float4*)rowp;
            for (uint32_t q = tid; q < V / 4; q += NT) {
                float4 v = src[q];
                nonfinite |= !finite_f(v.x) | !finite_f(v.y) | !finite_f(v.z) | !finite_f(v.w);
                if (mw) {
                    const uint32_t bits = mw[q >> 3] >> ((q & 7) * 4);
                    if (!(bits & 1u)) v.x = -INFINITY;
                    if (!(bits & 2u)) v.y = -INFINITY;
                    if (!(bits & 4u)) v.z = -INFINITY;
                    if (!(bits & 8u)) v.w = -INFINITY;
                }
                ((float4*)X)[q] = v;
            }
        } else {
            for (uint32_t i = tid; i < V; i += NT) {
                float x = load_logit(rowp, a.dtype, i);
                nonfinite |= !finite_f(x);
                if (mw && !((mw[i >> 5] >> (i & 31)) & 1u)) x = -INFINITY;
                X[i] = x;
            }
        }
        nonfinite = __syncthreads_or(nonfinite);
        if (nonfinite) {
            if (tid == 0) {
                if (tp) tp_write_head(a, row, NAN, 0.0f, 0u, ROW_NONFINITE, 0u);
                else write_row(a, row, 0u, ROW_NONFINITE, 0, 0u, -INFINITY, 0.0f, 0.0f, 0u);
                if (a.faulted) atomicAdd(a.faulted, 1ull);
            }
            continue;
        }
        if (gflags & 2u) {
            if (tid == 0) {
                if (tp) tp_write_head(a, row, -INFINITY, 0.0f, 0u, ROW_DEAD, 0u);
                else write_row(a, row, 0u, ROW_DEAD, 0, 0u, -INFINITY, 0.0f, 0.0f, 0u);
            }
            continue;
        }

        // ----------------------------------------------------------------- penalties
        const bool do_fp = !(fabsf(freq) < 1e-6f && fabsf(pres) < 1e-6f);
        const bool do_pres = fabsf(pres) > 1e-6f;
        const bool do_rep = rep != 1.0f;
        if (nh > 0 && (do_fp || do_rep)) {
            uint32_t cap = 64;
            while (cap < 2 * nh) cap <<= 1;   // <= hash_cap because nh <= max_history
            uint32_t* hk = a.sh_key + (size_t)slot * a.hash_cap;
            uint32_t* hc = a.sh_cnt + (size_t)slot * a.hash_cap;
            for (uint32_t s = tid; s < cap; s += NT) { hk[s] = 0xffffffffu; hc[s] = 0u; }
            __syncthreads();
            for (uint32_t j = tid; j < nh; j += NT) {
                const uint32_t id = a.hist_ids[h0 + j] - a.id_base;   // ids below the shard wrap around
                if (id >= V) continue;
                uint32_t s = (id * 2654435761u) & (cap - 1);
                for (uint32_t probe = 0; probe < cap; probe++) {
                    const uint32_t prev = atomicCAS(&hk[s], 0xffffffffu, id);
                    if (prev == 0xffffffffu || prev == id) { atomicAdd(&hc[s], 1u); break; }
                    s = (s + 1) & (cap - 1);
                }
            }
            __syncthreads();
            for (uint32_t s = tid; s < cap; s += NT) {
                const uint32_t id = hk[s];
                if (id == 0xffffffffu) continue;
                float x = X[id];
                if (do_rep) x = x > 0.0f ? fdiv(x, rep) : fmul(x, rep);
                if (do_fp) {
                    x = fsub(x, fmul(freq, (float)hc[s]));
                    if (do_pres) x = fsub(x, pres);
                }
                X[id] = x;
            }
            __syncthreads();
        }
        // ------------------------------------------------------------------- EOS fix
        if (mw && (gflags & 1u) && a.eos >= 0 && (uint32_t)a.eos < V && tid == 0 &&
            !finite_f(X[a.eos]))
            X[a.eos] = 0.0f;
        __syncthreads();

        // --------------------------------------------------------- max / argmax (lowest id)
        unsigned long long best = 0ull;
        for (uint32_t i = tid; i < V; i += NT) {
            const unsigned long long k = order_key(X[i]);
            if (k) {
                const unsigned long long cand = (k << 32) | (unsigned long long)(0xffffffffu - i);
                best = cand > best ? cand : best;
            }
        }
        best = block_max_u64(best, sm.rs);
        const bool any = best != 0ull;
        const float m = any ? key_to_float((uint32_t)(best >> 32)) : -INFINITY;
        const uint32_t amax = any ? 0xffffffffu - (uint32_t)best : 0u;
        const int status = any ? ROW_OK : ROW_EMPTY;
        if (tp) {   // vocabulary-sharded mode: the row ends as this shard's record
            tp_emit_row(a, sm, row, X, V, any, m, amax, temp, tab);
            continue;
        }
        if (temp < 1e-5f) {
            if (tid == 0) write_row(a, row, amax, status, 0, amax, m, 0.0f, 0.0f, 0u);
            continue;
        }

        // ------------------------------- temperature softmax numerators and their f32 fold
        const float t = fmaxf(temp, 1e-9f);
        const float S = seq_scan(
            [&](int i) { const float e = softmax_num(X[i], m, t, tab); X[i] = e; return e; },
            (int)V, 0.0f, SEQ_SUM, 0.0f, nullptr, sm.seq, sm.rs);
        const bool norm = S > 1e-9f;
        auto prob = [&](int i) { const float e = X[i]; return norm ? fdiv(e, S) : e; };
        const bool use_k = top_k != 0u && top_k < V;
        const bool use_p = !(top_p >= 1.0f);
        const bool want_list = use_k || use_p || a.n_kept || a.dump_ids || a.dump_probs;

        uint32_t token = amax, n_kept = 0;
        int drew = 0;
        float total = 0.0f;
        if (!want_list) {
            // plain categorical over the whole vocabulary
            total = seq_scan(prob, (int)V, 0.0f, SEQ_SUM, 0.0f, nullptr, sm.seq, sm.rs);
            if (total > 1e-9f) {
                int found;
                seq_scan(prob, (int)V, 0.0f, SEQ_FIND_GT, fmul(u01, total), &found, sm.seq, sm.rs);
                token = found >= 0 ? (uint32_t)found : V - 1;
                drew = 1;
            }
        } else {
            // top-k threshold on probabilities: ties at the threshold all survive (sampler.rs:124)
            float thr = 0.0f;
            if (use_k) {
                const uint32_t kk = radix_select_kth([&](int i) { return f2u(X[i]); }, (int)V, top_k,
                                                     sm.sel, sm.rs);
                thr = norm ? fdiv(u2f(kk), S) : u2f(kk);
            }
            // ordered compaction of the survivors with non-zero probability
            uint32_t* lid = a.sl_id + (size_t)slot * a.vocab_pad;
            float* lp = a.sl_p + (size_t)slot * a.vocab_pad;
            uint32_t n = 0;
            for (uint32_t base = 0; base < V; base += NT * 4) {
                const uint32_t i0 = base + tid * 4;
                float p[4];
                uint32_t cnt = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    p[j] = (i0 + j < V) ? prob((int)(i0 + j)) : 0.0f;
                    if (!(p[j] > 0.0f && p[j] >= thr)) p[j] = 0.0f;
                    cnt += p[j] > 0.0f;
                }
                uint32_t tot;
                uint32_t at = n + block_excl_scan_u32(cnt, &tot, sm.rs);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (p[j] > 0.0f) { lid[at] = i0 + j; lp[at] = p[j]; at++; }
                n += tot;
            }
            __syncthreads();
            // top-p: walk the candidates by probability descending, id ascending (sampler.rs:134-144)
            if (use_p && n > 0) {
                uint32_t npad = 2;
                while (npad < n) npad <<= 1;
                unsigned long long* keys =
                    npad <= (uint32_t)SORT_TILE ? sm.sort_tile : a.sl_key + (size_t)slot * a.sort_pad;
                for (uint32_t j = tid; j < npad; j += NT)
                    keys[j] = j < n ? ((unsigned long long)(~f2u(lp[j])) << 32) | j : ~0ull;
                bitonic_sort(keys, (int)npad, sm.sort_tile);
                int found;
                seq_scan([&](int j) { return u2f(~(uint32_t)(keys[j] >> 32)); }, (int)n, 0.0f,
                         SEQ_FIND_GE, top_p, &found, sm.seq, sm.rs);
                if (found >= 0)
                    for (uint32_t j = (uint32_t)found + 1 + tid; j < n; j += NT)
                        lp[(uint32_t)keys[j]] = 0.0f;
                __syncthreads();
            }
            total = seq_scan([&](int j) { return lp[j]; }, (int)n, 0.0f, SEQ_SUM, 0.0f, nullptr, sm.seq,
                             sm.rs);
            if (total > 1e-9f) {
                int found;
                seq_scan([&](int j) { return lp[j]; }, (int)n, 0.0f, SEQ_FIND_GT, fmul(u01, total),
                         &found, sm.seq, sm.rs);
                token = found >= 0 ? lid[found] : V - 1;
                drew = 1;
            }
            if (a.n_kept || a.dump_ids || a.dump_probs) {
                for (uint32_t base = 0; base < n; base += NT) {
                    const uint32_t j = base + tid;
                    const uint32_t keep = (j < n && lp[j] > 0.0f) ? 1u : 0u;
                    uint32_t tot;
                    const uint32_t at = n_kept + block_excl_scan_u32(keep, &tot, sm.rs);
                    if (keep && at < a.dump_cap) {
                        if (a.dump_ids) a.dump_ids[(size_t)row * a.dump_cap + at] = lid[j];
                        if (a.dump_probs) a.dump_probs[(size_t)row * a.dump_cap + at] = lp[j];
                    }
                    n_kept += tot;
                }
            }
        }
        if (tid == 0) write_row(a, row, token, status, drew, amax, m, S, total, n_kept);
    }
    // the last CTA to finish a work list empties it for the next step
    if (a.work_rows && tid == 0) {
        __threadfence();
        if (atomicAdd(a.work_count + 1, 1u) == gridDim.x - 1) {
            a.work_count[0] = 0u;
            a.work_count[1] = 0u;
        }
    }
}

size_t general_smem_bytes() { return sizeof(GeneralSmem); }

// once per device, with that device current
cudaError_t configure_general() {
    return cudaFuncSetAttribute(general_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(GeneralSmem));
}

cudaError_t launch_general(const RowArgs& a, uint32_t grid, cudaStream_t stream) {
    if (!a.work_rows) {
        general_row_kernel<<<grid, NT, sizeof(GeneralSmem), stream>>>(a);
        return cudaGetLastError();
    }
    // the work-list pass: programmatic stream serialization, see cudaGridDependencySynchronize() in the kernel
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = sizeof(GeneralSmem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, general_row_kernel, a);
}

}  // namespace pgs

// ------------------------------------------------------------------------------------------
// Entry point for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: a serving process whose memory
// pool already owns the whole device, a plugin loaded into a runtime that forbids allocation
// after start-up, or code that runs where an allocation would synchronise the device at the
// wrong moment.  pgs_sample_batch_static runs the general row kernel above with its per-row
// working storage placed in the fixed array below instead of in buffers owned by a handle, so
// it needs no handle and performs no allocation of any kind (no cudaMalloc / cudaFree, no
// library call that allocates).  The price is a fixed capacity and shared storage:
//   - vocab <= PGS_STATIC_MAX_VOCAB, at most PGS_STATIC_MAX_HISTORY history ids per row (longer
//     rows get PGS_ROW_BAD_PARAM), no grammar tables, every array in device memory;
//   - the array belongs to the device, not to the call: every call on that device uses the same
//     storage and leaves its last rows' working data behind.  Nothing in it has to start at zero
//     (each row rewrites every part of its slot before reading it), but two calls whose kernels
//     overlap on the GPU -- different streams, or different host threads -- race on it;
//   - every GPU that loads the library holds the array (about 10.6 MB) until the process exits.
// The first call on a device looks up the array's device address and raises the kernel's
// shared-memory limit; make that first call outside of any stream capture.
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/pagoda_sampler.h"

namespace pgs {

constexpr uint32_t STATIC_SLOTS = 8;            // rows in flight
constexpr uint32_t STATIC_MAX_VOCAB = 65536;
constexpr uint32_t STATIC_MAX_HISTORY = 1024;
constexpr uint32_t STATIC_HASH_CAP = 2048;      // >= 2 * STATIC_MAX_HISTORY, power of two
constexpr size_t STATIC_BYTES = (size_t)STATIC_SLOTS * STATIC_MAX_VOCAB * (4 + 4 + 4 + 8) +
                                (size_t)STATIC_SLOTS * STATIC_HASH_CAP * 8;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

static void* g_static_addr[64];                 // device address of the array, per device ordinal
static std::mutex g_static_setup;               // two threads making their first call on a device at once
static thread_local char g_static_error[256] = "";

static int static_fail(int code, const char* what, cudaError_t e) {
    snprintf(g_static_error, sizeof g_static_error, "%s%s%s", what, e == cudaSuccess ? "" : ": ",
             e == cudaSuccess ? "" : cudaGetErrorString(e));
    return code;
}

}  // namespace pgs

extern "C" const char* pgs_static_last_error(void) {
    return pgs::g_static_error;
}

extern "C" int pgs_sample_batch_static(int device, const pgs_batch_desc* desc_ptr, void* cuda_stream) {
    using namespace pgs;
    const pgs_batch_desc* d = desc_ptr;
    if (!d || d->struct_size != sizeof(pgs_batch_desc)) return static_fail(-1, "pgs_sample_batch_static: bad descriptor size", cudaSuccess);
    if (device < 0 || device >= 64) return static_fail(-1, "pgs_sample_batch_static: device ordinal out of range", cudaSuccess);
    if (d->rows == 0) return 0;
    if (d->vocab == 0 || d->vocab > STATIC_MAX_VOCAB)
        return static_fail(-4, "pgs_sample_batch_static: vocab exceeds the static capacity of 65536", cudaSuccess);
    if (!d->logits || !d->token || !d->status || d->row_stride < d->vocab || d->logits_dtype > 1)
        return static_fail(-1, "pgs_sample_batch_static: logits, token, status required; row_stride >= vocab", cudaSuccess);
    if (d->logits_mem != 0 || d->aux_mem != 0)
        return static_fail(-1, "pgs_sample_batch_static: every array must be device memory (staging would allocate)",
                           cudaSuccess);
    if (d->mask_table || d->mask_state)
        return static_fail(-1, "pgs_sample_batch_static: grammar tables belong to a handle and are not supported here",
                           cudaSuccess);
    if ((d->hist_offsets == nullptr) != (d->hist_ids == nullptr))
        return static_fail(-1, "pgs_sample_batch_static: hist_offsets and hist_ids must be given together", cudaSuccess);
    if ((d->dump_ids || d->dump_probs) && d->dump_cap == 0)
        return static_fail(-1, "pgs_sample_batch_static: dump arrays given with dump_cap == 0", cudaSuccess);
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_fail(-2, "cudaGetDevice", e);
    if (prev != device && (e = cudaSetDevice(device)) != cudaSuccess) return static_fail(-2, "cudaSetDevice", e);
    int rc = 0;
    void* scratch = nullptr;
    {   // set-up, once per device, with that device current
        std::lock_guard<std::mutex> lk(g_static_setup);
        scratch = g_static_addr[device];
    }
    if (!scratch) {
        std::lock_guard<std::mutex> lk(g_static_setup);
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e == cudaSuccess) e = configure_general();
        if (e != cudaSuccess) rc = static_fail(-2, "pgs_sample_batch_static set-up", e);
        else g_static_addr[device] = scratch = p;
    }
    if (rc == 0) {
        unsigned char* base = static_cast<unsigned char*>(scratch);
        const size_t per = (size_t)STATIC_SLOTS * STATIC_MAX_VOCAB;
        RowArgs a;
        memset(&a, 0, sizeof a);
        a.logits = d->logits; a.dtype = d->logits_dtype; a.rows = d->rows; a.vocab = d->vocab;
        a.row_stride = d->row_stride;
        a.temperature = d->temperature; a.top_k = d->top_k; a.top_p = d->top_p;
        a.freq = d->frequency_penalty; a.pres = d->presence_penalty; a.rep = d->repetition_penalty;
        a.hist_offsets = d->hist_offsets; a.hist_ids = d->hist_ids;
        a.eos = d->eos_token_id; a.uniform = d->uniform;
        a.token = d->token; a.status = d->status; a.drew = d->drew; a.argmax = d->argmax; a.row_max = d->row_max;
        a.sumexp = d->sumexp; a.total = d->total; a.n_kept = d->n_kept;
        a.dump_cap = d->dump_cap; a.dump_ids = d->dump_ids; a.dump_probs = d->dump_probs;
        a.sx = reinterpret_cast<float*>(base);
        a.sl_id = reinterpret_cast<uint32_t*>(base + per * 4);
        a.sl_p = reinterpret_cast<float*>(base + per * 8);
        a.sl_key = reinterpret_cast<unsigned long long*>(base + per * 12);
        a.sh_key = reinterpret_cast<uint32_t*>(base + per * 20);
        a.sh_cnt = reinterpret_cast<uint32_t*>(base + per * 20 + (size_t)STATIC_SLOTS * STATIC_HASH_CAP * 4);
        a.vocab_pad = STATIC_MAX_VOCAB; a.sort_pad = STATIC_MAX_VOCAB; a.hash_cap = STATIC_HASH_CAP;
        a.max_history = STATIC_MAX_HISTORY;
        const uint32_t grid = d->rows < STATIC_SLOTS ? d->rows : STATIC_SLOTS;
        e = launch_general(a, grid, static_cast<cudaStream_t>(cuda_stream));
        if (e != cudaSuccess) rc = static_fail(-2, "pgs_sample_batch_static launch", e);
    }
    if (prev != device && prev >= 0) cudaSetDevice(prev);
    return rc;
}
