// Host side of the C ABI declared in include/pagoda_sampler.h: handle lifecycle, grammar table
// uploads, staging of host-resident batches and kernel launches.  No CPU fallback: every entry
// point either runs the CUDA kernels or returns an error.
#include "../../include/pagoda_sampler.h"

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <vector>

#include "pgs_args.cuh"
#include "pgs_stream.cuh"
#include "pgs_tp.cuh"

namespace pgs {
cudaError_t configure_general();
cudaError_t launch_general(const RowArgs& a, uint32_t grid, cudaStream_t stream);
size_t general_smem_bytes();

size_t stream_smem_bytes();
cudaError_t configure_stream();
cudaError_t stream_ctas_per_sm(int* out);
cudaError_t launch_stream(const RowArgs& a, const StreamLaunch& sl, uint32_t grid, uint32_t csize, cudaStream_t stream);
cudaError_t stream_max_clusters(int csize, int* out);
struct ScoreArgs {
    const float* logits;
    unsigned long long row_stride;
    uint32_t rows, vocab;
    const uint32_t* ids;
    float* out_gather;
    float* out_full;
    int32_t* status;
};
cudaError_t configure_score();
cudaError_t launch_log_softmax(const ScoreArgs& a, uint32_t grid, cudaStream_t stream);
cudaError_t configure_tp();
cudaError_t launch_tp_push(const TpArgs& a, cudaStream_t stream);
cudaError_t launch_tp_merge(const TpArgs& a, const TpOut& o, cudaStream_t stream);
cudaError_t launch_draft_accept(const uint32_t* row_argmax, const uint32_t* draft, uint32_t sequences,
                                uint32_t positions, uint32_t* accepted, uint32_t* next, cudaStream_t stream);
}  // namespace pgs

static thread_local char g_create_error[256] = "";

struct pgs_handle {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t last_stream = nullptr;   // stream of the step before: steps of one handle share its scratch and must not overlap
    cudaEvent_t ev_step = nullptr;
    uint32_t max_rows = 0, max_vocab = 0, max_history = 0;
    uint32_t slots = 0, vocab_pad = 0, sort_pad = 0, hash_cap = 0;
    // scratch slots
    float* sx = nullptr;
    uint32_t* sl_id = nullptr;
    float* sl_p = nullptr;
    unsigned long long* sl_key = nullptr;
    uint32_t* sh_key = nullptr;
    uint32_t* sh_cnt = nullptr;
    // grammar tables
    pgs::TableDir tables_host[pgs::MAX_TABLES];
    pgs::TableDir* tables_dev = nullptr;
    // staging for host-resident batches
    void* logits_stage = nullptr;
    size_t logits_stage_bytes = 0;
    unsigned char* aux_host = nullptr;   // pinned
    unsigned char* aux_dev = nullptr;
    size_t aux_bytes = 0;
    // rows the row kernel hands on to the general kernel (work list)
    uint32_t* work_rows = nullptr;
    uint32_t* work_count = nullptr;   // [2]
    uint32_t* tp_done = nullptr;      // CTAs finished in the current peer-store push
    int exact = 0;
    // streaming row kernel: id -> count slots, shared memory and CTAs per SM, the gate's counter
    uint32_t stream_hash = 0, stream_cohort = 0;
    int max_clusters[4] = {0, 0, 0, 0};   // resident clusters of 1 (unused), 2, 4, 8 CTAs of the row kernel
    int cluster_mode = 1;                 // PGS_CLUSTER=0 turns row sharing off
    size_t stream_smem = 0;
    int stream_ctas = 0;
    uint32_t* p1_done = nullptr;      // device counter: rows that finished their first pass, over all launches
    uint32_t done_total = 0;          // the value that counter has when every launch so far has completed
    unsigned long long* faulted = nullptr;   // device counters: [0] ROW_NONFINITE rows, [1] rows whose exchange wait ran out
    unsigned long long* tp_timeouts = nullptr;   // = faulted + 1
    unsigned long long timeouts_seen = 0;    // value of the second counter at the last pgs_tp_exchange_status
    uint32_t wait_polls = 1u << 21;          // bound of the merge's flag wait (about a second)
    cudaStream_t tp_stream = nullptr;        // stream of the last pgs_tp_merge_wait
    long long* prof = nullptr;        // phase timers of the row kernel (PGS_PROFILE=1)
    pgs_counters counters = {};
    char err[256] = "";
};

static int fail(pgs_handle* h, int code, const char* fmt, ...) {
    char* dst = h ? h->err : g_create_error;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, 256, fmt, ap);
    va_end(ap);
    return code;
}

#define PGS_CUDA(h, call)                                                                  \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            cudaGetLastError(); /* a reported error must not resurface at the next launch */ \
            return fail(h, e_ == cudaErrorMemoryAllocation ? PGS_ERR_NOMEM : PGS_ERR_CUDA, \
                        "%s: %s", #call, cudaGetErrorString(e_));                          \
        }                                                                                  \
    } while (0)

namespace {
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        int cur = -1;
        cudaGetDevice(&cur);
        if (prev >= 0 && prev != cur) cudaSetDevice(prev);
    }
};

uint32_t pow2_at_least(uint32_t v, uint32_t lo) {
    uint32_t p = lo;
    while (p < v) p <<= 1;
    return p;
}
}  // namespace

extern "C" const char* pgs_last_error(const pgs_handle* h) { return h ? h->err : g_create_error; }

static int destroy_impl(pgs_handle* h) {
    DeviceGuard g(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    for (int t = 0; t < pgs::MAX_TABLES; t++) {
        if (h->tables_host[t].live) {
            cudaFree((void*)h->tables_host[t].words);
            cudaFree((void*)h->tables_host[t].flags);
        }
    }
    cudaFree(h->sx); cudaFree(h->sl_id); cudaFree(h->sl_p); cudaFree(h->sl_key);
    cudaFree(h->sh_key); cudaFree(h->sh_cnt); cudaFree(h->tables_dev);
    cudaFree(h->logits_stage); cudaFree(h->aux_dev); cudaFree(h->work_rows); cudaFree(h->work_count); cudaFree(h->tp_done); cudaFree(h->prof);
    cudaFree(h->p1_done); cudaFree(h->faulted);
    if (h->aux_host) cudaFreeHost(h->aux_host);
    if (h->ev_step) cudaEventDestroy(h->ev_step);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    return PGS_OK;
}

extern "C" int pgs_create(int device, uint32_t max_rows, uint32_t max_vocab, uint32_t max_history,
                          pgs_handle** out) {
    if (!out) return fail(nullptr, PGS_ERR_INVALID, "pgs_create: out is NULL");
    *out = nullptr;
    if (max_rows == 0 || max_vocab == 0 || max_vocab > (1u << 24) || max_history > (1u << 22))
        return fail(nullptr, PGS_ERR_INVALID,
                    "pgs_create: need 1 <= max_rows, 1 <= max_vocab <= 2^24, max_history <= 2^22");
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev == 0)
        return fail(nullptr, PGS_ERR_CUDA, "pgs_create: no CUDA device (%s); this library has no CPU path",
                    cudaGetErrorString(e));
    if (device < 0 || device >= n_dev)
        return fail(nullptr, PGS_ERR_INVALID, "pgs_create: device %d out of range (0..%d)", device, n_dev - 1);
    pgs_handle* h = new (std::nothrow) pgs_handle();
    if (!h) return fail(nullptr, PGS_ERR_NOMEM, "pgs_create: out of host memory");
    h->device = device;
    memset(h->tables_host, 0, sizeof h->tables_host);
    DeviceGuard g(device);
    int rc = [&]() -> int {
        cudaDeviceProp prop;
        PGS_CUDA(nullptr, cudaGetDeviceProperties(&prop, device));
        if (prop.major < 10)
            return fail(nullptr, PGS_ERR_CUDA, "pgs_create: device %d is sm_%d%d; this library is built for sm_100a",
                        device, prop.major, prop.minor);
        h->sm_count = prop.multiProcessorCount;
        PGS_CUDA(nullptr, cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking));
        PGS_CUDA(nullptr, cudaEventCreateWithFlags(&h->ev_step, cudaEventDisableTiming));
        h->last_stream = h->stream;
        PGS_CUDA(nullptr, pgs::configure_general());
        PGS_CUDA(nullptr, pgs::configure_tp());
        PGS_CUDA(nullptr, pgs::configure_score());
        PGS_CUDA(nullptr, cudaMalloc(&h->work_rows, (size_t)max_rows * sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMalloc(&h->work_count, 2 * sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMemsetAsync(h->work_count, 0, 2 * sizeof(uint32_t), h->stream));
        PGS_CUDA(nullptr, cudaMalloc(&h->tp_done, sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMemsetAsync(h->tp_done, 0, sizeof(uint32_t), h->stream));
        PGS_CUDA(nullptr, cudaMalloc(&h->p1_done, sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMemsetAsync(h->p1_done, 0, sizeof(uint32_t), h->stream));
        PGS_CUDA(nullptr, cudaMalloc(&h->faulted, 2 * sizeof(unsigned long long)));
        PGS_CUDA(nullptr, cudaMemsetAsync(h->faulted, 0, 2 * sizeof(unsigned long long), h->stream));
        h->tp_timeouts = h->faulted + 1;
        h->stream_hash = pow2_at_least(2 * (max_history ? max_history : 1), 64);
        if (h->stream_hash > (uint32_t)pgs::S_MAX_HASH) h->stream_hash = pgs::S_MAX_HASH;   // longer histories take the general kernel
        h->stream_smem = pgs::stream_smem_bytes();
        PGS_CUDA(nullptr, pgs::configure_stream());
        PGS_CUDA(nullptr, pgs::stream_ctas_per_sm(&h->stream_ctas));
        if (h->stream_ctas < 1) return fail(nullptr, PGS_ERR_CUDA, "pgs_create: the row kernel does not fit an SM (%zu bytes of shared memory)", h->stream_smem);
        // rows that may be in their first pass at once: no limit by default (measured on 256 x 151936: a limit of
        // about an SM count keeps pass 2 in L2 but leaves half the threads of every SM waiting at the gate)
        h->stream_cohort = 0xffffffffu;
        if (const char* ev = getenv("PGS_COHORT")) { if (atoi(ev) > 0) h->stream_cohort = (uint32_t)atoi(ev); }
        if (const char* ev = getenv("PGS_CLUSTER")) h->cluster_mode = atoi(ev);
        for (int i = 1; i < 4; i++) {
            if (pgs::stream_max_clusters(1 << i, &h->max_clusters[i]) != cudaSuccess) { cudaGetLastError(); h->max_clusters[i] = 0; }
        }
        if (const char* ev = getenv("PGS_EXACT")) h->exact = atoi(ev);
        if (const char* ev = getenv("PGS_PROFILE")) {
            if (atoi(ev)) {
                PGS_CUDA(nullptr, cudaMalloc(&h->prof, 1024 * 16 * sizeof(long long)));
                PGS_CUDA(nullptr, cudaMemsetAsync(h->prof, 0, 1024 * 16 * sizeof(long long), h->stream));
            }
        }
        h->max_rows = max_rows; h->max_vocab = max_vocab; h->max_history = max_history;
        h->slots = max_rows < (uint32_t)h->sm_count ? max_rows : (uint32_t)h->sm_count;
        h->vocab_pad = (max_vocab + 31u) & ~31u;
        h->sort_pad = pow2_at_least(max_vocab, 2);
        h->hash_cap = pow2_at_least(2 * (max_history ? max_history : 1), 64);
        const size_t s = h->slots;
        PGS_CUDA(nullptr, cudaMalloc(&h->sx, s * h->vocab_pad * sizeof(float)));
        PGS_CUDA(nullptr, cudaMalloc(&h->sl_id, s * h->vocab_pad * sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMalloc(&h->sl_p, s * h->vocab_pad * sizeof(float)));
        PGS_CUDA(nullptr, cudaMalloc(&h->sl_key, s * h->sort_pad * sizeof(unsigned long long)));
        PGS_CUDA(nullptr, cudaMalloc(&h->sh_key, s * h->hash_cap * sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMalloc(&h->sh_cnt, s * h->hash_cap * sizeof(uint32_t)));
        PGS_CUDA(nullptr, cudaMalloc(&h->tables_dev, sizeof h->tables_host));
        PGS_CUDA(nullptr, cudaMemsetAsync(h->tables_dev, 0, sizeof h->tables_host, h->stream));
        // aux staging: per-row parameter and output arrays of a host-resident batch
        h->aux_bytes = (size_t)max_rows * 128 + (size_t)max_rows * max_history * 4 + 4096;
        PGS_CUDA(nullptr, cudaMalloc(&h->aux_dev, h->aux_bytes));
        PGS_CUDA(nullptr, cudaMallocHost(&h->aux_host, h->aux_bytes));
        PGS_CUDA(nullptr, cudaStreamSynchronize(h->stream));
        return PGS_OK;
    }();
    if (rc != PGS_OK) {
        destroy_impl(h);
        return rc;
    }
    *out = h;
    return PGS_OK;
}

extern "C" int pgs_destroy(pgs_handle* h) {
    if (!h) return PGS_OK;
    return destroy_impl(h);
}

extern "C" void* pgs_stream(pgs_handle* h) { return h ? (void*)h->stream : nullptr; }

extern "C" int pgs_get_counters(const pgs_handle* h, pgs_counters* out) {
    if (!h || !out) return PGS_ERR_INVALID;
    *out = h->counters;
    // faulted rows are counted on the device by the kernels that find them
    DeviceGuard g(h->device);
    unsigned long long f = 0;
    cudaError_t e = cudaStreamSynchronize(h->stream);
    if (e == cudaSuccess && h->last_stream != h->stream) e = cudaStreamSynchronize(h->last_stream);
    if (e == cudaSuccess) e = cudaMemcpy(&f, h->faulted, sizeof f, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { cudaGetLastError(); return PGS_ERR_CUDA; }
    out->rows_faulted = f;
    return PGS_OK;
}

extern "C" int pgs_mask_table_upload(pgs_handle* h, uint32_t n_states, uint32_t words_per_state,
                                     const uint32_t* host_words, const uint8_t* state_flags,
                                     int32_t* table_id) {
    if (!h) return PGS_ERR_INVALID;
    if (!host_words || !table_id || n_states == 0 || words_per_state == 0)
        return fail(h, PGS_ERR_INVALID, "pgs_mask_table_upload: empty table or NULL argument");
    int t = -1;
    for (int i = 0; i < pgs::MAX_TABLES; i++)
        if (!h->tables_host[i].live) { t = i; break; }
    if (t < 0) return fail(h, PGS_ERR_LIMIT, "pgs_mask_table_upload: all %d table slots in use", pgs::MAX_TABLES);
    DeviceGuard g(h->device);
    uint32_t* words = nullptr;
    uint8_t* flags = nullptr;
    const size_t wbytes = (size_t)n_states * words_per_state * sizeof(uint32_t);
    PGS_CUDA(h, cudaMalloc(&words, wbytes));
    cudaError_t e = cudaMalloc(&flags, n_states);
    if (e != cudaSuccess) { cudaFree(words); return fail(h, PGS_ERR_NOMEM, "cudaMalloc(flags): %s", cudaGetErrorString(e)); }
    std::vector<uint8_t> zero;
    if (!state_flags) { zero.assign(n_states, 0); state_flags = zero.data(); }
    pgs::TableDir d;
    d.words = words; d.flags = flags; d.words_per_state = words_per_state; d.n_states = n_states;
    d.live = 1; d.pad = 0;
    e = cudaMemcpyAsync(words, host_words, wbytes, cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(flags, state_flags, n_states, cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h->tables_dev + t, &d, sizeof d, cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    if (e != cudaSuccess) {
        cudaFree(words); cudaFree(flags);
        return fail(h, PGS_ERR_CUDA, "pgs_mask_table_upload: %s", cudaGetErrorString(e));
    }
    h->tables_host[t] = d;
    *table_id = t;
    return PGS_OK;
}

extern "C" int pgs_mask_table_free(pgs_handle* h, int32_t table_id) {
    if (!h) return PGS_ERR_INVALID;
    if (table_id < 0 || table_id >= pgs::MAX_TABLES || !h->tables_host[table_id].live)
        return fail(h, PGS_ERR_INVALID, "pgs_mask_table_free: table %d is not live", table_id);
    DeviceGuard g(h->device);
    pgs::TableDir d = h->tables_host[table_id];
    pgs::TableDir dead;
    memset(&dead, 0, sizeof dead);
    PGS_CUDA(h, cudaMemcpyAsync(h->tables_dev + table_id, &dead, sizeof dead, cudaMemcpyHostToDevice, h->stream));
    PGS_CUDA(h, cudaStreamSynchronize(h->stream));
    cudaFree((void*)d.words);
    cudaFree((void*)d.flags);
    h->tables_host[table_id] = dead;
    return PGS_OK;
}

// ------------------------------------------------------------------------------ batches

namespace {

// One step: the streaming row kernel serves every row it can and lists the others, which the general kernel then
// processes.  In exact mode every row takes the
// general kernel.
int launch_step(pgs_handle* h, pgs::RowArgs& a, cudaStream_t stream) {
    const uint32_t rows = a.rows;
    const uint32_t grid = rows < h->slots ? rows : h->slots;
    a.faulted = h->faulted;
    // Every step of a handle uses the same scratch, lists and counters: a step on another stream than the one before
    // waits for that one to finish on the device.
    if (stream != h->last_stream) {
        PGS_CUDA(h, cudaEventRecord(h->ev_step, h->last_stream));
        PGS_CUDA(h, cudaStreamWaitEvent(stream, h->ev_step, 0));
        h->last_stream = stream;
    }
    if (h->exact || a.vocab > (uint32_t)pgs::S_MAX_VOCAB) {
        PGS_CUDA(h, pgs::launch_general(a, grid, stream));
        h->counters.kernel_launches += 1;
        return PGS_OK;
    }
    pgs::StreamLaunch sl;
    sl.hash_slots = h->stream_hash; sl.cohort = h->stream_cohort;
    sl.done_base = h->done_total; sl.gate_polls = 1u << 16;   // x 200 ns: gives up after about 13 ms
    sl.p1_done = h->p1_done;
    sl.work_rows = h->work_rows; sl.work_count = h->work_count;
    sl.prof = h->prof;
    const uint32_t resident = (uint32_t)h->stream_ctas * (uint32_t)h->sm_count;
    // Small batches: the CTAs of a cluster share every row, with the largest cluster size that still has all rows
    // resident at once (a row alone on one CTA is bound by latency, not by bandwidth).
    uint32_t csize = 1;
    if (h->cluster_mode && !a.tp_records)
        for (int i = 3; i >= 2; i--)   // (pairs do not pay: two CTAs per row with half the rows' CTAs measured slower)
            if (h->max_clusters[i] > 0 && rows <= (uint32_t)h->max_clusters[i]) { csize = 1u << i; break; }
    PGS_CUDA(h, pgs::launch_stream(a, sl, csize > 1 ? rows : (rows < resident ? rows : resident), csize, stream));
    h->done_total += rows;
    // The list is usually empty.  The pass over it is set up while the row kernel still runs (programmatic stream
    // serialization) and returns at once when it finds nothing listed.
    pgs::RowArgs wl = a;
    wl.work_rows = h->work_rows;
    wl.work_count = h->work_count;
    PGS_CUDA(h, pgs::launch_general(wl, grid < 32u ? grid : 32u, stream));
    h->counters.kernel_launches += 2;
    return PGS_OK;
}

struct AuxPlan {
    pgs_handle* h;
    size_t used = 0;
    bool overflow = false;
    // (host destination, offset, bytes) of every output to copy back
    struct Out { void* dst; size_t off, bytes; };
    std::vector<Out> outs;
    size_t out_lo = 0, out_hi = 0;

    size_t reserve(size_t bytes) {
        size_t off = (used + 15) & ~size_t(15);
        if (off + bytes > h->aux_bytes) { overflow = true; return 0; }
        used = off + bytes;
        return off;
    }
    template <class T> const T* in(const T* host, size_t n) {
        if (!host) return nullptr;
        size_t off = reserve(n * sizeof(T));
        if (overflow) return nullptr;
        memcpy(h->aux_host + off, host, n * sizeof(T));
        return (const T*)(h->aux_dev + off);
    }
    template <class T> T* out(T* host, size_t n) {
        if (!host) return nullptr;
        size_t off = reserve(n * sizeof(T));
        if (overflow) return nullptr;
        outs.push_back({host, off, n * sizeof(T)});
        return (T*)(h->aux_dev + off);
    }
};

int validate(pgs_handle* h, const pgs_batch_desc* d) {
    if (!d) return fail(h, PGS_ERR_INVALID, "desc is NULL");
    if (d->struct_size != sizeof(pgs_batch_desc))
        return fail(h, PGS_ERR_INVALID, "desc.struct_size %u != %zu (ABI mismatch)", d->struct_size,
                    sizeof(pgs_batch_desc));
    if (d->rows == 0) return PGS_OK;
    if (d->rows > h->max_rows || d->vocab > h->max_vocab)
        return fail(h, PGS_ERR_LIMIT, "batch %u x %u exceeds the handle's %u x %u", d->rows, d->vocab,
                    h->max_rows, h->max_vocab);
    if (d->vocab == 0 || !d->logits || !d->token || !d->status)
        return fail(h, PGS_ERR_INVALID, "vocab, logits, token and status are required");
    if (d->row_stride < d->vocab) return fail(h, PGS_ERR_INVALID, "row_stride < vocab");
    if (d->logits_dtype > PGS_BF16 || d->logits_mem > PGS_MEM_HOST || d->aux_mem > PGS_MEM_HOST)
        return fail(h, PGS_ERR_INVALID, "bad dtype / memory kind");
    if (d->hist_ids && !d->hist_offsets)
        return fail(h, PGS_ERR_INVALID, "hist_ids given without hist_offsets");
    // Offsets without ids: only host arrays can be checked for "every row is empty"; device offsets
    // cannot be read here, so there the pair must come together.
    if (d->hist_offsets && !d->hist_ids && (d->aux_mem != PGS_MEM_HOST || d->hist_offsets[d->rows] != 0))
        return fail(h, PGS_ERR_INVALID, "hist_offsets given without hist_ids");
    if ((d->dump_ids || d->dump_probs) && d->dump_cap == 0)
        return fail(h, PGS_ERR_INVALID, "dump arrays given with dump_cap == 0");
    return PGS_OK;
}

int run_batch(pgs_handle* h, const pgs_batch_desc* d, cudaStream_t stream, bool wait) {
    int rc = validate(h, d);
    if (rc != PGS_OK) return rc;
    if (d->rows == 0) return PGS_OK;
    DeviceGuard g(h->device);
    const uint32_t rows = d->rows;
    const size_t esz = d->logits_dtype == PGS_F32 ? 4 : 2;
    pgs::RowArgs a;
    memset(&a, 0, sizeof a);
    a.dtype = d->logits_dtype; a.rows = rows; a.vocab = d->vocab; a.eos = d->eos_token_id;
    a.tables = h->tables_dev;
    a.sx = h->sx; a.sl_id = h->sl_id; a.sl_p = h->sl_p; a.sl_key = h->sl_key;
    a.sh_key = h->sh_key; a.sh_cnt = h->sh_cnt;
    a.vocab_pad = h->vocab_pad; a.sort_pad = h->sort_pad; a.hash_cap = h->hash_cap;
    a.max_history = h->max_history;
    a.dump_cap = d->dump_cap;

    // logits
    if (d->logits_mem == PGS_MEM_HOST) {
        const size_t need = (size_t)rows * d->vocab * esz;
        if (need > h->logits_stage_bytes) {
            if (h->logits_stage) { cudaStreamSynchronize(stream); cudaFree(h->logits_stage); h->logits_stage = nullptr; }
            const size_t full = (size_t)h->max_rows * h->max_vocab * 4;
            PGS_CUDA(h, cudaMalloc(&h->logits_stage, full));
            h->logits_stage_bytes = full;
        }
        PGS_CUDA(h, cudaMemcpy2DAsync(h->logits_stage, (size_t)d->vocab * esz, d->logits,
                                      (size_t)d->row_stride * esz, (size_t)d->vocab * esz, rows,
                                      cudaMemcpyHostToDevice, stream));
        a.logits = h->logits_stage;
        a.row_stride = d->vocab;
    } else {
        a.logits = d->logits;
        a.row_stride = d->row_stride;
    }

    AuxPlan plan{h};
    uint64_t hist_total = 0, masked_rows = 0;
    if (d->aux_mem == PGS_MEM_HOST) {
        if (d->hist_offsets) {
            hist_total = d->hist_offsets[rows];
            for (uint32_t r = 0; r < rows; r++) {
                if (d->hist_offsets[r + 1] < d->hist_offsets[r])
                    return fail(h, PGS_ERR_INVALID, "hist_offsets must be non-decreasing");
                if (d->hist_offsets[r + 1] - d->hist_offsets[r] > h->max_history)
                    return fail(h, PGS_ERR_LIMIT, "row %u has %u history ids; the handle allows %u", r,
                                d->hist_offsets[r + 1] - d->hist_offsets[r], h->max_history);
            }
        }
        if (d->mask_table)
            for (uint32_t r = 0; r < rows; r++) masked_rows += d->mask_table[r] >= 0;
        a.temperature = plan.in(d->temperature, rows);
        a.top_k = plan.in(d->top_k, rows);
        a.top_p = plan.in(d->top_p, rows);
        a.freq = plan.in(d->frequency_penalty, rows);
        a.pres = plan.in(d->presence_penalty, rows);
        a.rep = plan.in(d->repetition_penalty, rows);
        a.hist_offsets = plan.in(d->hist_offsets, (size_t)rows + 1);
        a.hist_ids = hist_total ? plan.in(d->hist_ids, hist_total) : nullptr;
        a.mask_table = plan.in(d->mask_table, rows);
        a.mask_state = plan.in(d->mask_state, rows);
        a.uniform = plan.in(d->uniform, rows);
        const size_t in_bytes = plan.used;
        plan.out_lo = (plan.used + 15) & ~size_t(15);
        a.token = plan.out(d->token, rows);
        a.status = plan.out(d->status, rows);
        a.drew = plan.out(d->drew, rows);
        a.argmax = plan.out(d->argmax, rows);
        a.row_max = plan.out(d->row_max, rows);
        a.sumexp = plan.out(d->sumexp, rows);
        a.total = plan.out(d->total, rows);
        a.n_kept = plan.out(d->n_kept, rows);
        plan.out_hi = plan.used;
        if (plan.overflow)
            return fail(h, PGS_ERR_LIMIT, "per-row arrays exceed the staging buffer sized at creation");
        // the candidate dump can be large; it gets its own device buffer per call
        uint32_t* dump_ids_dev = nullptr;
        float* dump_probs_dev = nullptr;
        const size_t dump_n = (size_t)rows * d->dump_cap;
        if (d->dump_ids) PGS_CUDA(h, cudaMalloc(&dump_ids_dev, dump_n * 4));
        if (d->dump_probs) PGS_CUDA(h, cudaMalloc(&dump_probs_dev, dump_n * 4));
        a.dump_ids = dump_ids_dev; a.dump_probs = dump_probs_dev;
        PGS_CUDA(h, cudaMemcpyAsync(h->aux_dev, h->aux_host, in_bytes, cudaMemcpyHostToDevice, stream));
        rc = launch_step(h, a, stream);
        if (rc != PGS_OK) { cudaFree(dump_ids_dev); cudaFree(dump_probs_dev); return rc; }
        PGS_CUDA(h, cudaMemcpyAsync(h->aux_host + plan.out_lo, h->aux_dev + plan.out_lo,
                                    plan.out_hi - plan.out_lo, cudaMemcpyDeviceToHost, stream));
        if (dump_ids_dev) PGS_CUDA(h, cudaMemcpyAsync(d->dump_ids, dump_ids_dev, dump_n * 4, cudaMemcpyDeviceToHost, stream));
        if (dump_probs_dev) PGS_CUDA(h, cudaMemcpyAsync(d->dump_probs, dump_probs_dev, dump_n * 4, cudaMemcpyDeviceToHost, stream));
        cudaError_t e = cudaStreamSynchronize(stream);
        cudaFree(dump_ids_dev); cudaFree(dump_probs_dev);
        if (e != cudaSuccess) return fail(h, PGS_ERR_CUDA, "kernel or copy failed: %s", cudaGetErrorString(e));
        for (const auto& o : plan.outs) memcpy(o.dst, h->aux_host + o.off, o.bytes);
    } else {
        a.temperature = d->temperature; a.top_k = d->top_k; a.top_p = d->top_p;
        a.freq = d->frequency_penalty; a.pres = d->presence_penalty; a.rep = d->repetition_penalty;
        a.hist_offsets = d->hist_offsets; a.hist_ids = d->hist_ids;
        a.mask_table = d->mask_table; a.mask_state = d->mask_state; a.uniform = d->uniform;
        a.token = d->token; a.status = d->status; a.drew = d->drew; a.argmax = d->argmax;
        a.row_max = d->row_max; a.sumexp = d->sumexp; a.total = d->total; a.n_kept = d->n_kept;
        a.dump_ids = d->dump_ids; a.dump_probs = d->dump_probs;
        rc = launch_step(h, a, stream);
        if (rc != PGS_OK) return rc;
        if (wait) {
            cudaError_t e = cudaStreamSynchronize(stream);
            if (e != cudaSuccess) return fail(h, PGS_ERR_CUDA, "kernel failed: %s", cudaGetErrorString(e));
        }
    }
    h->counters.calls += 1;
    h->counters.rows += rows;
    h->counters.bytes += (uint64_t)rows * (d->vocab * esz + 64) + hist_total * 4 + masked_rows * (d->vocab / 8);
    return PGS_OK;
}

}  // namespace

// Phase timers of the row kernel (clock ticks, [ctas x 16]); only with PGS_PROFILE=1.
extern "C" PGS_API int pgs_debug_read_profile(pgs_handle* h, long long* out, uint32_t n_ctas) {
    if (!h || !h->prof || n_ctas > 1024) return PGS_ERR_INVALID;
    DeviceGuard g(h->device);
    PGS_CUDA(h, cudaStreamSynchronize(h->stream));
    PGS_CUDA(h, cudaMemcpy(out, h->prof, (size_t)n_ctas * 16 * sizeof(long long), cudaMemcpyDeviceToHost));
    PGS_CUDA(h, cudaMemset(h->prof, 0, 1024 * 16 * sizeof(long long)));
    return PGS_OK;
}

extern "C" int pgs_set_exact(pgs_handle* h, int on) {
    if (!h) return PGS_ERR_INVALID;
    h->exact = on ? 1 : 0;
    return PGS_OK;
}

extern "C" int pgs_sample_batch(pgs_handle* h, const pgs_batch_desc* desc) {
    if (!h) return PGS_ERR_INVALID;
    return run_batch(h, desc, h->stream, true);
}

extern "C" int pgs_sample_batch_async(pgs_handle* h, const pgs_batch_desc* desc, void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    if (desc && (desc->logits_mem != PGS_MEM_DEVICE || desc->aux_mem != PGS_MEM_DEVICE))
        return fail(h, PGS_ERR_INVALID, "pgs_sample_batch_async needs every array in device memory");
    return run_batch(h, desc, cuda_stream ? (cudaStream_t)cuda_stream : h->stream, false);
}

// ------------------------------------------------------------------- vocabulary-sharded mode

extern "C" size_t pgs_tp_record_bytes(uint32_t cand) { return 16 + (size_t)cand * 8; }

static int tp_args(pgs_handle* h, const pgs_tp_desc* d, pgs::TpArgs* a) {
    if (!d || d->struct_size != sizeof(pgs_tp_desc)) return fail(h, PGS_ERR_INVALID, "bad pgs_tp_desc");
    if (d->n_shards == 0 || d->n_shards > 8 || d->shard_rank >= d->n_shards || d->vocab % d->n_shards)
        return fail(h, PGS_ERR_INVALID, "need 1 <= n_shards <= 8, rank < n_shards, vocab divisible by n_shards");
    if (d->cand == 0 || d->cand > 128) return fail(h, PGS_ERR_INVALID, "cand must be in 1..128");
    if (d->rows == 0 || d->rows > h->max_rows) return fail(h, PGS_ERR_LIMIT, "%u rows exceed the handle's %u", d->rows, h->max_rows);
    a->shard_vocab = d->vocab / d->n_shards;
    if (a->shard_vocab > h->max_vocab) return fail(h, PGS_ERR_LIMIT, "shard width %u exceeds the handle's vocab %u", a->shard_vocab, h->max_vocab);
    if (d->row_stride < a->shard_vocab) return fail(h, PGS_ERR_INVALID, "row_stride < shard width");
    a->logits = d->logits; a->row_stride = d->row_stride; a->rows = d->rows; a->vocab = d->vocab;
    a->shard_lo = d->shard_rank * a->shard_vocab; a->n_shards = d->n_shards; a->cand = d->cand;
    a->temperature = d->temperature; a->top_p = d->top_p; a->uniform = d->uniform; a->top_k = d->top_k;
    a->wait_polls = h->wait_polls; a->timeouts = h->tp_timeouts;
    a->rec_bytes = (uint32_t)pgs_tp_record_bytes(d->cand);
    memset(a->peer_records, 0, sizeof a->peer_records);
    memset(a->peer_flags, 0, sizeof a->peer_flags);
    a->flags = nullptr; a->done = nullptr; a->epoch = 0; a->shard_rank = d->shard_rank;
    return PGS_OK;
}

// The emitting half is the batch step itself over this rank's columns, with records in place of tokens: the same
// kernels, checks, penalties, mask and EOS fix; history ids and eos_token_id are global ids.
static int tp_emit(pgs_handle* h, const pgs_tp_desc* d, const pgs::TpArgs& t, unsigned char* records, cudaStream_t stream) {
    if ((d->hist_offsets == nullptr) != (d->hist_ids == nullptr))
        return fail(h, PGS_ERR_INVALID, "hist_offsets and hist_ids must be given together");
    if (((uintptr_t)records & 15u) != 0) return fail(h, PGS_ERR_INVALID, "the record buffer must be 16-byte aligned");
    pgs::RowArgs a;
    memset(&a, 0, sizeof a);
    a.logits = d->logits; a.dtype = 0; a.rows = d->rows; a.vocab = t.shard_vocab; a.row_stride = d->row_stride;
    a.temperature = d->temperature;
    a.freq = d->frequency_penalty; a.pres = d->presence_penalty; a.rep = d->repetition_penalty;
    a.hist_offsets = d->hist_offsets; a.hist_ids = d->hist_ids;
    a.mask_table = d->mask_table; a.mask_state = d->mask_state; a.tables = h->tables_dev;
    const int64_t eos_local = (int64_t)d->eos_token_id - (int64_t)t.shard_lo;
    a.eos = (d->eos_token_id >= 0 && eos_local >= 0 && eos_local < (int64_t)t.shard_vocab) ? (int32_t)eos_local : -1;
    a.sx = h->sx; a.sl_id = h->sl_id; a.sl_p = h->sl_p; a.sl_key = h->sl_key;
    a.sh_key = h->sh_key; a.sh_cnt = h->sh_cnt;
    a.vocab_pad = h->vocab_pad; a.sort_pad = h->sort_pad; a.hash_cap = h->hash_cap;
    a.max_history = h->max_history;
    a.tp_records = records; a.tp_rec_bytes = t.rec_bytes; a.tp_cand = t.cand; a.id_base = t.shard_lo;
    return launch_step(h, a, stream);
}

extern "C" int pgs_tp_partial(pgs_handle* h, const pgs_tp_desc* d, void* records_out, void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    pgs::TpArgs a;
    int rc = tp_args(h, d, &a);
    if (rc != PGS_OK) return rc;
    if (!d->logits || !records_out) return fail(h, PGS_ERR_INVALID, "logits and records_out are required");
    DeviceGuard g(h->device);
    return tp_emit(h, d, a, (unsigned char*)records_out, cuda_stream ? (cudaStream_t)cuda_stream : h->stream);
}

extern "C" int pgs_tp_merge(pgs_handle* h, const pgs_tp_desc* d, const void* records_all, const pgs_tp_out* out,
                            void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    pgs::TpArgs a;
    int rc = tp_args(h, d, &a);
    if (rc != PGS_OK) return rc;
    if (!records_all || !out || !out->token || !out->status)
        return fail(h, PGS_ERR_INVALID, "records_all, out->token and out->status are required");
    DeviceGuard g(h->device);
    a.records = (unsigned char*)records_all;
    pgs::TpOut o{out->token, out->status, out->drew, out->argmax, out->gmax, out->gsum, out->total, out->n_kept};
    PGS_CUDA(h, pgs::launch_tp_merge(a, o, cuda_stream ? (cudaStream_t)cuda_stream : h->stream));
    h->counters.kernel_launches += 1;
    h->counters.rows += a.rows;
    return PGS_OK;
}

extern "C" int pgs_peer_alloc(pgs_handle* h, size_t bytes, void** dev_ptr, unsigned char ipc_handle_out[64]) {
    if (!h || !dev_ptr || !ipc_handle_out || bytes == 0) return PGS_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the IPC handle is exchanged as 64 bytes");
    DeviceGuard g(h->device);
    void* p = nullptr;
    PGS_CUDA(h, cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t ih;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&ih, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(h, PGS_ERR_CUDA, "pgs_peer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(ipc_handle_out, &ih, sizeof ih);
    *dev_ptr = p;
    return PGS_OK;
}

extern "C" int pgs_peer_open(pgs_handle* h, const unsigned char ipc_handle[64], void** dev_ptr) {
    if (!h || !dev_ptr || !ipc_handle) return PGS_ERR_INVALID;
    DeviceGuard g(h->device);
    cudaIpcMemHandle_t ih;
    memcpy(&ih, ipc_handle, sizeof ih);
    void* p = nullptr;
    PGS_CUDA(h, cudaIpcOpenMemHandle(&p, ih, cudaIpcMemLazyEnablePeerAccess));
    // prove that this device reaches the mapping before any kernel is pointed at it
    uint32_t probe = 0;
    const cudaError_t e = cudaMemcpy(&probe, p, sizeof probe, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        cudaIpcCloseMemHandle(p);
        return fail(h, PGS_ERR_CUDA, "pgs_peer_open: the mapped buffer is not readable from device %d: %s", h->device,
                    cudaGetErrorString(e));
    }
    *dev_ptr = p;
    return PGS_OK;
}

extern "C" int pgs_peer_close(pgs_handle* h, void* dev_ptr) {
    if (!h || !dev_ptr) return PGS_ERR_INVALID;
    DeviceGuard g(h->device);
    PGS_CUDA(h, cudaIpcCloseMemHandle(dev_ptr));
    return PGS_OK;
}

extern "C" int pgs_peer_free(pgs_handle* h, void* dev_ptr) {
    if (!h || !dev_ptr) return PGS_ERR_INVALID;
    DeviceGuard g(h->device);
    PGS_CUDA(h, cudaFree(dev_ptr));
    return PGS_OK;
}

extern "C" int pgs_tp_partial_push(pgs_handle* h, const pgs_tp_desc* d, void* const* peer_records,
                                   uint32_t* const* peer_flags, uint32_t epoch, void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    pgs::TpArgs a;
    int rc = tp_args(h, d, &a);
    if (rc != PGS_OK) return rc;
    if (!d->logits || !peer_records || !peer_flags) return fail(h, PGS_ERR_INVALID, "logits, peer_records and peer_flags are required");
    for (uint32_t p = 0; p < d->n_shards; p++) {
        if (!peer_records[p] || !peer_flags[p]) return fail(h, PGS_ERR_INVALID, "peer %u: NULL gather buffer or flag array", p);
        // this shard's block inside rank p's [n_shards][rows][record] buffer
        a.peer_records[p] = (unsigned char*)peer_records[p] + (size_t)d->shard_rank * a.rows * a.rec_bytes;
        a.peer_flags[p] = peer_flags[p];
    }
    DeviceGuard g(h->device);
    // every buffer must be device memory this GPU can reach: its own, or a peer's with peer access enabled
    // (enabled here when it is not yet; an IPC mapping alone does not do that for this device)
    for (uint32_t p = 0; p < d->n_shards; p++) {
        const void* ptrs[2] = {peer_records[p], peer_flags[p]};
        for (const void* ptr : ptrs) {
            cudaPointerAttributes at;
            PGS_CUDA(h, cudaPointerGetAttributes(&at, ptr));
            if (at.type != cudaMemoryTypeDevice) return fail(h, PGS_ERR_INVALID, "peer %u: not device memory", p);
            if (at.device == h->device) continue;
            int can = 0;
            PGS_CUDA(h, cudaDeviceCanAccessPeer(&can, h->device, at.device));
            if (!can) return fail(h, PGS_ERR_INVALID, "device %d cannot access memory of device %d", h->device, at.device);
            const cudaError_t e = cudaDeviceEnablePeerAccess(at.device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) return fail(h, PGS_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d): %s", at.device, cudaGetErrorString(e));
        }
    }
    a.records = a.peer_records[d->shard_rank];   // built in this rank's own buffer, then copied out
    a.done = h->tp_done;                         // zero between launches
    a.epoch = epoch;
    cudaStream_t stream = cuda_stream ? (cudaStream_t)cuda_stream : h->stream;
    rc = tp_emit(h, d, a, a.records, stream);
    if (rc != PGS_OK) return rc;
    PGS_CUDA(h, pgs::launch_tp_push(a, stream));
    h->counters.kernel_launches += 1;
    return PGS_OK;
}

extern "C" int pgs_tp_merge_wait(pgs_handle* h, const pgs_tp_desc* d, const void* records_all, const uint32_t* flags,
                                 uint32_t epoch, const pgs_tp_out* out, void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    pgs::TpArgs a;
    int rc = tp_args(h, d, &a);
    if (rc != PGS_OK) return rc;
    if (!records_all || !flags || !out || !out->token || !out->status)
        return fail(h, PGS_ERR_INVALID, "records_all, flags, out->token and out->status are required");
    DeviceGuard g(h->device);
    a.records = (unsigned char*)records_all;
    a.flags = (uint32_t*)flags;
    a.epoch = epoch;
    pgs::TpOut o{out->token, out->status, out->drew, out->argmax, out->gmax, out->gsum, out->total, out->n_kept};
    h->tp_stream = cuda_stream ? (cudaStream_t)cuda_stream : h->stream;
    PGS_CUDA(h, pgs::launch_tp_merge(a, o, h->tp_stream));
    h->counters.kernel_launches += 1;
    h->counters.rows += a.rows;
    return PGS_OK;
}

extern "C" int pgs_set_wait_limit(pgs_handle* h, uint32_t polls) {
    if (!h) return PGS_ERR_INVALID;
    if (polls == 0) return fail(h, PGS_ERR_INVALID, "pgs_set_wait_limit: at least one poll");
    h->wait_polls = polls;
    return PGS_OK;
}

extern "C" int pgs_tp_exchange_status(pgs_handle* h) {
    if (!h) return PGS_ERR_INVALID;
    DeviceGuard g(h->device);
    unsigned long long n = 0;
    cudaError_t e = cudaStreamSynchronize(h->tp_stream ? h->tp_stream : h->stream);
    if (e == cudaSuccess) e = cudaMemcpy(&n, h->tp_timeouts, sizeof n, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(h, PGS_ERR_CUDA, "pgs_tp_exchange_status: %s", cudaGetErrorString(e));
    const unsigned long long fresh = n - h->timeouts_seen;
    h->timeouts_seen = n;
    if (fresh) return fail(h, PGS_ERR_TIMEOUT, "%llu rows gave up waiting for a shard's records", fresh);
    return PGS_OK;
}

extern "C" int pgs_draft_accept(pgs_handle* h, const uint32_t* row_argmax, const uint32_t* draft, uint32_t sequences,
                                uint32_t positions, uint32_t* accepted, uint32_t* next, void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    if (!row_argmax || !draft || !accepted || !next || positions == 0)
        return fail(h, PGS_ERR_INVALID, "pgs_draft_accept: NULL argument or zero positions");
    if (sequences == 0) return PGS_OK;
    DeviceGuard g(h->device);
    PGS_CUDA(h, pgs::launch_draft_accept(row_argmax, draft, sequences, positions, accepted, next,
                                         cuda_stream ? (cudaStream_t)cuda_stream : h->stream));
    h->counters.kernel_launches += 1;
    return PGS_OK;
}

// ------------------------------------------------------------------------------ scoring

extern "C" int pgs_log_softmax(pgs_handle* h, const float* logits, uint32_t rows, uint32_t vocab, uint64_t row_stride,
                               const uint32_t* ids, float* out_gather, float* out_full, int32_t* status,
                               void* cuda_stream) {
    if (!h) return PGS_ERR_INVALID;
    if (!logits || vocab == 0 || row_stride < vocab || (!out_full && !(ids && out_gather)))
        return fail(h, PGS_ERR_INVALID, "pgs_log_softmax: need logits, row_stride >= vocab and an output");
    if (rows == 0) return PGS_OK;
    DeviceGuard g(h->device);
    pgs::ScoreArgs a{logits, row_stride, rows, vocab, ids, out_gather, out_full, status};
    const uint32_t grid = rows < (uint32_t)h->sm_count ? rows : (uint32_t)h->sm_count;
    PGS_CUDA(h, pgs::launch_log_softmax(a, grid, cuda_stream ? (cudaStream_t)cuda_stream : h->stream));
    h->counters.kernel_launches += 1;
    return PGS_OK;
}
