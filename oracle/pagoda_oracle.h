/*
 * CPU oracle for the logits -> token chain of quantz8a/pagoda.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * Rust sampler chain, written to be the checker for the CUDA path.  It is
 * never linked into, imported by, or called from the shipped library; only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark load it.
 *
 * Parity status: pinned against every known-answer test the reference holds
 * for this path (sampler.rs tests, engine.rs penalty tests, grammar.rs tests);
 * the reference itself is Rust and cannot be compiled in this environment.
 * Extensions that have no reference counterpart (repetition penalty, bf16
 * logits, arbitrary-token bitmasks, vocabulary-sharded merge, draft
 * acceptance) are "parity unpinned": this file defines them.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#ifndef PAGODA_ORACLE_H
#define PAGODA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Row status, same numbering as the device library (include/pagoda_sampler.h). */
enum {
    PGO_ROW_OK = 0,
    PGO_ROW_NONFINITE = 1, /* logits_sane failed -> FinishReason::Fault */
    PGO_ROW_DEAD = 2,      /* grammar dead end -> FinishReason::Stop, nothing sampled */
    PGO_ROW_EMPTY = 3,     /* nothing finite left after masking; token 0 as the reference returns */
    PGO_ROW_BAD_PARAM = 4  /* a parameter outside of what the call supports (sharded mode: top_k > cand) */
};

/* ---- rng.rs:7-31 ---- */
typedef struct { uint64_t s; } pgo_rng;
void pgo_rng_new(pgo_rng *r, uint64_t seed);
uint64_t pgo_rng_next_u64(pgo_rng *r);
double pgo_rng_next_f64(pgo_rng *r);
float pgo_rng_next_f32(pgo_rng *r);

/* ---- sampler.rs ---- */
uint32_t pgo_argmax(const float *xs, size_t n);                 /* :59-70 */
void pgo_log_softmax(const float *xs, size_t n, float *out);    /* :73-87 */
void pgo_temperature_softmax(float *xs, size_t n, float temp);  /* :92-114 */
void pgo_apply_top_k(float *xs, size_t n, uint64_t k);          /* :116-128 */
void pgo_apply_top_p(float *xs, size_t n, float p);             /* :130-150 */
/* :40-55; `u` is what rng.next_f32() would return; *drew = 1 iff the draw is consumed */
uint32_t pgo_sample_categorical(const float *probs, size_t n, float u, int *drew);
/* :28-37 */
uint32_t pgo_sample(const float *logits, size_t n, float temperature, uint64_t top_k,
                    float top_p, float u, int *drew);

/* ---- engine.rs ---- */
int pgo_logits_sane(const float *logits, size_t n, size_t vocab);          /* :1278-1280 */
void pgo_apply_penalties(float *logits, size_t n, const uint32_t *output, size_t n_out,
                         float freq, float pres);                           /* :1553-1573 */
/* extension (no reference counterpart): for every distinct id < n in `output`,
 * logit > 0 -> logit / rep, else logit * rep.  Runs before frequency/presence. */
void pgo_apply_repetition(float *logits, size_t n, const uint32_t *output, size_t n_out,
                          float rep);

/* ---- grammar.rs:73-85 ---- */
void pgo_mask_logits_bytes(const uint8_t *allowed, size_t n_allowed, float *logits, size_t n);
/* device form of the same rule: keep token i iff bit (i & 31) of words[i >> 5] is set */
void pgo_mask_logits_bits(const uint32_t *words, float *logits, size_t n);

/* ---- one row of Engine::advance_with_logits (engine.rs:1286-1314) ---- */
typedef struct {
    float temperature;
    float top_p;
    uint32_t top_k;      /* 0 = disabled (usize::MAX in the reference); >= vocab is a no-op too */
    float freq, pres, rep;
    const uint32_t *history; uint32_t n_history;
    const uint32_t *mask_words;   /* NULL = no grammar on this row */
    int grammar_dead;             /* allowed_bytes() == None */
    int grammar_complete;         /* is_complete() */
    int32_t eos_id;               /* < 0: none */
    float uniform;
} pgo_row_params;

typedef struct {
    uint32_t token;
    int32_t status;
    int32_t drew;
    uint32_t argmax;     /* argmax of the processed logits */
    float row_max;       /* max over finite processed logits (-inf if none) */
    float sumexp;        /* the sequential f32 sum of temperature_softmax (0 for greedy rows) */
    float total;         /* sample_categorical's total */
    uint32_t n_kept;     /* entries with probability > 0 after top-k/top-p */
    /* relative distance of the closest decision (top-k threshold gap, top-p
     * boundary, CDF boundary) from flipping; 1.0 when no decision was taken */
    float margin;
    /* the same, one per decision: gap between the top-k threshold and the next smaller distinct
     * probability; distance of the top-p cumulative sums around the cut from p; distance of
     * u * total from the CDF steps around the drawn token */
    float margin_k, margin_p, margin_cdf;
} pgo_row_out;

/* `logits` is read only; `work` must hold 2*n floats; `probs_out` (may be NULL) receives
 * the final probability vector that sample_categorical walked. */
void pgo_sample_row(const float *logits, size_t n, const pgo_row_params *p,
                    pgo_row_out *out, float *work, float *probs_out);

/* Whole batch with the rows spread over `n_threads` host threads (1 = the
 * reference's own serial loop, engine.rs:511-544).  Arrays are per row;
 * hist_offsets has rows+1 entries; mask_rows[r] points at that row's words or NULL. */
typedef struct {
    const float *logits; size_t rows, vocab, row_stride;
    const float *temperature, *top_p; const uint32_t *top_k;
    const float *freq, *pres, *rep;
    const uint32_t *hist_offsets, *hist_ids;
    const uint32_t *const *mask_rows; const uint8_t *row_flags; /* bit0 complete, bit1 dead */
    int32_t eos_id;
    const float *uniform;
} pgo_batch;
void pgo_sample_batch(const pgo_batch *b, pgo_row_out *out, int n_threads);

/* bf16 -> f32 exact upcast (extension) */
void pgo_bf16_to_f32(const uint16_t *in, float *out, size_t n);

/* ---- vocabulary-sharded merge (extension; semantics defined here) ----
 * The row is split into n_shards equal column ranges.  Each shard contributes its
 * max m_r, its own sequential sum s_r = sum exp((x - m_r)/t) and its top `cand`
 * entries (value desc, id asc).  Merge: M = max m_r; S = sum_r s_r*exp((m_r - M)/t)
 * folded in shard order; candidate probability exp((x - M)/t)/S; then top-k (p->top_k <= cand,
 * else PGO_ROW_BAD_PARAM), top-p, total and the CDF walk exactly as the single-device chain does,
 * over the candidate set.  Sanity, penalties, grammar mask and EOS fix run first, as in
 * pgo_sample_row; records hold finite logits only, and a shard without any contributes nothing. */
typedef struct {
    uint32_t token; int32_t status; int32_t drew; uint32_t argmax;
    float gmax, gsum, total; uint32_t n_kept; float margin;
} pgo_tp_out;
void pgo_tp_sample_row(const float *logits, size_t n, uint32_t n_shards, uint32_t cand,
                       const pgo_row_params *p, pgo_tp_out *out);
/* draft verification: accept while argmax(row j) == draft[j]; returns accepted count,
 * *next = argmax at the first mismatch, or of the last row when all are accepted */
uint32_t pgo_draft_accept(const uint32_t *row_argmax, const uint32_t *draft, uint32_t n,
                          uint32_t *next);

/* ---- grammar.rs: byte regex (:93-576) and JSON prefix scanner (:582-1016) ---- */
typedef struct pgo_regex pgo_regex;
pgo_regex *pgo_regex_new(const char *pattern, char *err, size_t err_len); /* NULL on error */
void pgo_regex_free(pgo_regex *re);
int pgo_regex_is_complete(const pgo_regex *re, const uint8_t *text, size_t n);
/* returns -1 when dead (None), else the number of allowed bytes written to out[256] */
int pgo_regex_allowed_bytes(const pgo_regex *re, const uint8_t *text, size_t n, uint8_t *out);
int pgo_json_is_complete(const uint8_t *text, size_t n);
int pgo_json_allowed_bytes(const uint8_t *text, size_t n, uint8_t *out);

#ifdef __cplusplus
}
#endif
#endif
