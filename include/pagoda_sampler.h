/*
 * pagoda_sampler.h -- C ABI of the B200 (sm_100a) backend for pagoda's per-step
 * logits -> token chain.
 *
 * The reference runs this chain on the host, one sequence at a time, inside
 * Engine::advance_with_logits (pagoda/src/engine.rs:1286-1327): sanity check ->
 * penalties -> grammar mask -> EOS fix -> Sampler::sample.  The reference has no
 * FFI today; these entry points are what a `pagoda-sampler-sys` crate would bind so
 * that the per-sequence loop at pagoda/src/engine.rs:511-544 becomes one batched
 * call.  Every function returns an int: 0 on success, a negative pgs_error
 * otherwise; nothing throws or aborts across the boundary.  There is no CPU
 * fallback: without a CUDA device pgs_create fails.
 *
 * Plain pointers and sizes only.  All calls on one handle must come from one thread
 * at a time (the reference samples on its single actor thread,
 * pagoda/src/engine.rs:1396); a handle may move between threads.
 */
#ifndef PAGODA_SAMPLER_H
#define PAGODA_SAMPLER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PGS_ABI_VERSION 1

#if defined(__GNUC__)
#define PGS_API __attribute__((visibility("default")))
#else
#define PGS_API
#endif

typedef struct pgs_handle pgs_handle;

enum pgs_error {
    PGS_OK = 0,
    PGS_ERR_INVALID = -1,  /* bad argument (message in pgs_last_error) */
    PGS_ERR_CUDA = -2,     /* a CUDA call failed */
    PGS_ERR_NOMEM = -3,
    PGS_ERR_LIMIT = -4,    /* rows / vocab / history beyond what pgs_create was sized for */
    PGS_ERR_TIMEOUT = -5   /* a bounded device-side wait ran out (peer exchange; pgs_tp_exchange_status) */
};

/* Per-row outcome.  Maps onto the reference's per-request finish reasons so that a
 * bad row never affects its batch-mates (pagoda/tests/fault_tests.rs:63-82). */
enum pgs_row_status {
    PGS_ROW_OK = 0,
    PGS_ROW_NONFINITE = 1, /* logits_sane failed (engine.rs:1278-1295) -> FinishReason::Fault */
    PGS_ROW_DEAD = 2,      /* grammar state is a dead end (engine.rs:1299-1303) -> Stop, no token */
    PGS_ROW_EMPTY = 3,     /* nothing finite left after masking; token 0, as sampler.rs:59-70 returns */
    PGS_ROW_BAD_PARAM = 4, /* non-finite parameter, bad mask table/state, history too long */
    PGS_ROW_LOAD_TIMEOUT = 5 /* a bounded wait for another shard's records ran out; nothing sampled */
};

enum pgs_mem { PGS_MEM_DEVICE = 0, PGS_MEM_HOST = 1 };
enum pgs_dtype { PGS_F32 = 0, PGS_BF16 = 1 };

/* Replaces Sampler::new / Engine's ownership of the sampler (sampler.rs:16-18,
 * engine.rs:96,202).  Sizes the device workspace once; later calls never allocate
 * unless a host-resident batch first needs its staging buffer. */
PGS_API int pgs_create(int device_ordinal, uint32_t max_rows, uint32_t max_vocab,
               uint32_t max_history_per_row, pgs_handle **out);
PGS_API int pgs_destroy(pgs_handle *h);
/* Message for the last failing call on this handle (or on creation when h == NULL). */
PGS_API const char *pgs_last_error(const pgs_handle *h);

/* Grammar bitmask tables.  Replaces the per-step allowed-byte vector that
 * Grammar::allowed_bytes builds and mask_logits applies (grammar.rs:52-65, :73-85):
 * the host tabulates its grammar into states, uploads one bitmask of
 * `words_per_state` u32 words per state once, and then names (table, state) per row.
 * Token i is kept iff bit (i & 31) of word (i >> 5) is set.  state_flags (may be NULL):
 * bit 0 = the partial output is already complete (drives the EOS fix of
 * engine.rs:1307-1312), bit 1 = dead end. */
PGS_API int pgs_mask_table_upload(pgs_handle *h, uint32_t n_states, uint32_t words_per_state,
                          const uint32_t *host_words, const uint8_t *state_flags,
                          int32_t *table_id);
PGS_API int pgs_mask_table_free(pgs_handle *h, int32_t table_id);

/* ---- host-side grammar state machines (no CUDA involved) ------------------------------------
 * Replace Grammar::regex / Grammar::json / allowed_bytes / is_complete (grammar.rs:32-66,
 * :458-575, :613-733).  A grammar is tabulated once into mask states (state 0 = dead end); the
 * table goes to the device through pgs_mask_table_upload and each sequence keeps a small host
 * state that is advanced by the bytes it emits, instead of re-running the grammar over the whole
 * output at every step (engine.rs:1297-1313).  Byte-level tokenizers only, as the reference
 * requires (engine.rs:986-987): token id = first_byte_id + byte. */
typedef struct pgs_grammar pgs_grammar;
typedef struct pgs_gstate pgs_gstate;
PGS_API int pgs_grammar_regex(const char *pattern, pgs_grammar **out, char *err, size_t err_len);
PGS_API int pgs_grammar_json(pgs_grammar **out);
PGS_API void pgs_grammar_free(pgs_grammar *g);
PGS_API uint32_t pgs_grammar_n_states(const pgs_grammar *g);
/* words_out: [n_states x ceil(vocab/32)], flags_out: [n_states] -- the arguments of pgs_mask_table_upload */
PGS_API int pgs_grammar_build_table(const pgs_grammar *g, uint32_t vocab, uint32_t first_byte_id,
                                    uint32_t *words_out, uint8_t *flags_out);
PGS_API int pgs_grammar_state_new(const pgs_grammar *g, pgs_gstate **out);
PGS_API int pgs_grammar_state_reset(const pgs_grammar *g, pgs_gstate *s);
PGS_API void pgs_grammar_state_free(pgs_gstate *s);
/* feed the bytes of the newly generated token(s) */
PGS_API int pgs_grammar_advance(const pgs_grammar *g, pgs_gstate *s, const uint8_t *bytes, size_t n);
/* the row's mask_state for the next step */
PGS_API uint32_t pgs_grammar_mask_state(const pgs_grammar *g, const pgs_gstate *s);
/* allowed bytes (256 flags), completeness and deadness of a table state */
PGS_API int pgs_grammar_state_info(const pgs_grammar *g, uint32_t state, uint8_t *allowed256, int *complete,
                                   int *dead);

/* One decode step for a batch of rows.  Per-row arrays may be NULL (defaults in
 * brackets, the reference's SamplingParams::default(), spec.rs:90-105). */
typedef struct pgs_batch_desc {
    uint32_t struct_size;         /* sizeof(pgs_batch_desc) */
    uint32_t rows;
    uint32_t vocab;
    uint32_t logits_dtype;        /* pgs_dtype; bf16 is upcast exactly, then the same math */
    uint64_t row_stride;          /* elements between consecutive rows (>= vocab) */
    const void *logits;           /* [rows x row_stride], read only */
    uint32_t logits_mem;          /* pgs_mem: where `logits` lives */
    uint32_t aux_mem;             /* pgs_mem: where every other array below lives */

    const float *temperature;     /* [0.0] below 1e-5 -> greedy (sampler.rs:29) */
    const uint32_t *top_k;        /* [0] 0 or >= vocab disables (sampler.rs:117) */
    const float *top_p;           /* [1.0] >= 1 disables (sampler.rs:131) */
    const float *frequency_penalty; /* [0.0] engine.rs:1553-1573 */
    const float *presence_penalty;  /* [0.0] */
    const float *repetition_penalty;/* [1.0] extension: logit > 0 ? logit / r : logit * r */
    const uint32_t *hist_offsets; /* CSR over generated token ids, rows + 1 entries (NULL = none) */
    const uint32_t *hist_ids;     /* ids >= vocab are skipped (engine.rs:1562) */
    const int32_t *mask_table;    /* per row table id, < 0 = no grammar (NULL = none) */
    const int32_t *mask_state;    /* per row state inside that table */
    int32_t eos_token_id;         /* < 0: none */
    uint32_t reserved0;
    const float *uniform;         /* per row rng.next_f32() (rng.rs:28-30); only read for rows that draw */

    uint32_t *token;              /* out, required */
    int32_t *status;              /* out, required: pgs_row_status */
    uint8_t *drew;                /* out, optional: 1 iff the row consumed its uniform (sampler.rs:43-46) */

    /* optional diagnostics for parity checks (NULL to skip) */
    uint32_t *argmax;             /* argmax of the processed logits, lowest id on ties */
    float *row_max;               /* max over finite processed logits */
    float *sumexp;                /* the f32 left-fold sum of temperature_softmax */
    float *total;                 /* sample_categorical's total */
    uint32_t *n_kept;             /* entries with probability > 0 after top-k / top-p */
    uint32_t dump_cap;            /* per row capacity of the two arrays below */
    uint32_t reserved1;
    uint32_t *dump_ids;           /* [rows x dump_cap] kept ids, ascending */
    float *dump_probs;            /* [rows x dump_cap] their probabilities */
} pgs_batch_desc;

/* Replaces the loop body apply_penalties -> mask_logits -> Sampler::sample
 * (engine.rs:1296-1314) for every row at once.  Returns after the outputs are
 * readable by the host. */
PGS_API int pgs_sample_batch(pgs_handle *h, const pgs_batch_desc *desc);
/* Same, enqueued on `cuda_stream` (a cudaStream_t; NULL = the handle's own stream)
 * without waiting.  Every array must be device memory.
 * Steps of one handle share its per-row working storage, so the library orders them on the GPU:
 * when a step is enqueued on a different stream than the handle's previous step, the new stream
 * first waits (cudaStreamWaitEvent) for the previous step's last kernel.  The caller only has to
 * keep to one host thread per handle at a time, and to keep a stream alive until the steps it
 * carried have finished.  Steps on different handles are independent. */
PGS_API int pgs_sample_batch_async(pgs_handle *h, const pgs_batch_desc *desc, void *cuda_stream);

/* Allocation-free variant of pgs_sample_batch_async.  It has no counterpart in the reference
 * (whose sampler works on host vectors and never touches device memory); it exists for callers
 * that may not allocate device memory once they are running -- a server whose memory pool owns
 * the whole GPU, a plugin inside a runtime that forbids allocation after start-up.  It needs no
 * handle and calls no allocator: the rows' working storage is a fixed array inside the library
 * (about 10.6 MB on every GPU that loads it).  Limits: vocab <= 65536, at most 1024 history ids
 * per row (longer rows report PGS_ROW_BAD_PARAM), no grammar tables, every array of the
 * descriptor in device memory; beyond them the call fails with PGS_ERR_LIMIT / PGS_ERR_INVALID
 * and a message in pgs_static_last_error().  Results are those of the general (bit-exact)
 * kernel.  All calls on one device share the array: calls whose kernels may overlap on the GPU
 * (different streams or host threads) race and must be serialised by the caller.  hist_offsets
 * and hist_ids must be given together or not at all.  The first call on each device does a
 * one-time set-up (guarded by a mutex, so two threads may make it at once) and should be made
 * outside any stream capture.
 * Only enqueues work on `cuda_stream` (a cudaStream_t; NULL = the default stream). */
PGS_API int pgs_sample_batch_static(int device_ordinal, const pgs_batch_desc *desc, void *cuda_stream);
PGS_API const char *pgs_static_last_error(void);

/* Fidelity switch.  By default rows run in the streaming row kernel: every decision follows the
 * reference, candidate probabilities use the exact expf, and the f32 left-fold sum of
 * temperature_softmax (sampler.rs:99-113) agrees with the reference's to about 1e-6 relative,
 * so a top-p or CDF decision can differ only when it sits that close to its boundary.  With
 * `on` != 0 every row takes the general kernel, which reproduces that sum -- and therefore
 * every token id -- bit for bit, at a fraction of the speed.  (Environment: PGS_EXACT=1.) */
PGS_API int pgs_set_exact(pgs_handle *h, int on);

/* ---- vocabulary-sharded sampling (extension; the reference has no multi-GPU code) ----------
 * Rank r of n holds columns [r * vocab/n, (r+1) * vocab/n) of every row.  pgs_tp_partial emits one
 * record of pgs_tp_record_bytes(cand) bytes per row (shard max, shard sum, argmax, the `cand`
 * largest logits with global ids); the caller all-gathers the records of all ranks into
 * [n_shards][rows][record] (NCCL over NVLink) and pgs_tp_merge turns them into tokens with the
 * same softmax / top-p / inverse-CDF rule as Sampler::sample (sampler.rs:28-55) restricted to
 * the union of the candidates.  All pointers are device memory; both calls only enqueue work
 * on `cuda_stream` (NULL = the handle's stream). */
typedef struct pgs_tp_desc {
    uint32_t struct_size;
    uint32_t rows;
    uint32_t vocab;               /* full vocabulary; must be a multiple of n_shards */
    uint32_t n_shards, shard_rank;
    uint32_t cand;                /* candidates per shard, 1..128 */
    uint64_t row_stride;          /* elements between rows of the shard */
    const float *logits;          /* [rows x row_stride] f32, this rank's columns */
    const float *temperature;     /* per row; NULL = greedy */
    const float *top_p;           /* per row; NULL = 1.0 (merge) */
    const float *uniform;         /* per row (merge) */
    const uint32_t *top_k;        /* per row, 0 = off; NULL = off (merge).  Must not exceed cand: the row gets
                                   * PGS_ROW_BAD_PARAM otherwise.  Ties at the k-th probability survive as in
                                   * sampler.rs:116-128, as far as the records hold them. */
    /* The rest of the chain of engine.rs:1296-1313, applied by the emitting half to its own columns before
     * anything else, exactly as pgs_sample_batch applies it to whole rows.  Ids are GLOBAL token ids. */
    const float *frequency_penalty, *presence_penalty, *repetition_penalty;   /* per row; NULL = off */
    const uint32_t *hist_offsets; /* [rows + 1] CSR; NULL = no history */
    const uint32_t *hist_ids;     /* generated ids of every row, global */
    const int32_t *mask_table;    /* per row: table id or -1; NULL = no grammar.  A table used here holds THIS
                                   * SHARD's bits: bit j of a state's words is column shard_rank * vocab/n_shards + j
                                   * (words_per_state * 32 >= vocab / n_shards). */
    const int32_t *mask_state;    /* per row: state inside the table */
    int32_t eos_token_id;         /* global id; -1 = none.  Only the shard that owns it applies the EOS fix. */
    int32_t reserved0;
} pgs_tp_desc;
PGS_API size_t pgs_tp_record_bytes(uint32_t cand);
PGS_API int pgs_tp_partial(pgs_handle *h, const pgs_tp_desc *desc, void *records_out, void *cuda_stream);
typedef struct pgs_tp_out {
    uint32_t *token; int32_t *status; uint8_t *drew;   /* token and status required */
    uint32_t *argmax; float *gmax; float *gsum; float *total; uint32_t *n_kept; /* optional */
} pgs_tp_out;
PGS_API int pgs_tp_merge(pgs_handle *h, const pgs_tp_desc *desc, const void *records_all,
                         const pgs_tp_out *out, void *cuda_stream);
/* The same exchange without a collective between the two kernels (no reference counterpart): the emitting
 * kernel stores each finished record into slot [shard_rank][row] of EVERY rank's gather buffer -- peer
 * memory over NVLink, mapped by the caller (CUDA IPC or symmetric memory) -- and, when its last row is out,
 * raises flag [shard_rank] in every rank's flag array to `epoch` (system-scope release).  pgs_tp_merge_wait
 * is pgs_tp_merge preceded by a bounded wait (about one second unless pgs_set_wait_limit says otherwise) for all
 * n_shards flags of this rank to reach `epoch`; when a shard never answers, the rows get status
 * PGS_ROW_LOAD_TIMEOUT instead of a hang, and the next pgs_tp_exchange_status returns PGS_ERR_TIMEOUT.
 *   peer_records[p]  rank p's gather buffer, [n_shards][rows][pgs_tp_record_bytes(cand)], p = 0..n_shards-1
 *   peer_flags[p]    rank p's flag array, [n_shards] uint32, zero before the first step
 *   epoch            1, 2, 3, ... one per step, the same on every rank
 * Both pointer arrays live in host memory.  Buffers and flags must be double-buffered by the caller
 * (epoch parity): a rank may start step k+1 while a peer still merges step k, never step k+2.  Run at most
 * one push per handle at a time. */
/* Buffers for that exchange.  pgs_peer_alloc: zeroed device memory on the handle's device plus the 64-byte
 * CUDA IPC handle a peer process needs to map it.  pgs_peer_open: maps a peer's buffer into this process
 * for the handle's device (peer access is enabled on the way) and proves the mapping with a 4-byte copy, so
 * that an unreachable peer is an error code here and not a fault in a kernel later.  Close what was opened
 * and free what was allocated before pgs_destroy. */
PGS_API int pgs_peer_alloc(pgs_handle *h, size_t bytes, void **dev_ptr, unsigned char ipc_handle_out[64]);
PGS_API int pgs_peer_open(pgs_handle *h, const unsigned char ipc_handle[64], void **dev_ptr);
PGS_API int pgs_peer_close(pgs_handle *h, void *dev_ptr);
PGS_API int pgs_peer_free(pgs_handle *h, void *dev_ptr);
PGS_API int pgs_tp_partial_push(pgs_handle *h, const pgs_tp_desc *desc, void *const *peer_records,
                                uint32_t *const *peer_flags, uint32_t epoch, void *cuda_stream);
PGS_API int pgs_tp_merge_wait(pgs_handle *h, const pgs_tp_desc *desc, const void *records_all,
                              const uint32_t *flags, uint32_t epoch, const pgs_tp_out *out, void *cuda_stream);
/* Bound of pgs_tp_merge_wait's wait, in polls of about half a microsecond each (default 2^21: about a second).
 * A serving loop that would rather drop a step than stall sets it to a few thousand. */
PGS_API int pgs_set_wait_limit(pgs_handle *h, uint32_t polls);
/* Failure detection for the exchange: waits for the stream of the last pgs_tp_merge_wait and returns
 * PGS_ERR_TIMEOUT when rows gave up waiting since the previous call of this function (a peer that never
 * answered), PGS_OK otherwise.  The handle stays usable either way. */
PGS_API int pgs_tp_exchange_status(pgs_handle *h);

/* Draft verification over per-position argmax ids (pagoda-hf/src/qwen3_5.rs:663-755 produces
 * them; the reference leaves the accept rule open): accepted[s] = length of the longest prefix
 * with row_argmax[s][j] == draft[s][j]; next[s] = the argmax at the first mismatch, or of the
 * last position when everything is accepted.  Device pointers. */
PGS_API int pgs_draft_accept(pgs_handle *h, const uint32_t *row_argmax, const uint32_t *draft,
                             uint32_t sequences, uint32_t positions, uint32_t *accepted,
                             uint32_t *next, void *cuda_stream);

/* Replaces sampler::log_softmax + the gather of Engine::score (sampler.rs:73-87,
 * engine.rs:1066-1090): per row out = ln(exp(x - max)) - max(ln(sum), f32::MIN_POSITIVE) with the
 * reference's f32 left-fold sum.  `ids` (one token id per row) selects what out_gather[row]
 * receives; out_full ([rows x vocab], may be NULL) receives the whole vector.  Device pointers;
 * only enqueues work on `cuda_stream` (NULL = the handle's stream).  Rows holding a non-finite
 * logit get status PGS_ROW_NONFINITE and NaN. */
PGS_API int pgs_log_softmax(pgs_handle *h, const float *logits, uint32_t rows, uint32_t vocab,
                            uint64_t row_stride, const uint32_t *ids, float *out_gather, float *out_full,
                            int32_t *status, void *cuda_stream);

/* Counters since creation (for the engine's /stats): rows sampled, rows faulted, algorithmic
 * bytes touched. */
typedef struct pgs_counters {
    uint64_t calls, rows, rows_faulted, bytes;
    uint64_t kernel_launches;
} pgs_counters;
PGS_API int pgs_get_counters(const pgs_handle *h, pgs_counters *out);

/* Phase timers of the streaming row kernel, a diagnostic: only handles created with PGS_PROFILE=1 in the
 * environment keep them.  out[cta * 16 + slot] receives the cycles thread 0 of CTA `cta` spent in each phase since
 * the last read (summed over its rows), then the timers are cleared.  Slots: 0 gate + row barrier, 1 history
 * indexed, 2 first pass, 6 reductions + argmax, 7 top-k bound, 3 fold table, 4 second pass, 5 finish.
 * n_ctas <= 1024.
 * Synchronises the handle's stream. */
PGS_API int pgs_debug_read_profile(pgs_handle *h, long long *out, uint32_t n_ctas);

/* The handle's stream as a cudaStream_t, for callers that time or order work on it. */
PGS_API void *pgs_stream(pgs_handle *h);

#ifdef __cplusplus
}
#endif
#endif
