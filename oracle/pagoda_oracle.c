/*
 * CPU oracle: sampler chain, penalties, mask and RNG of quantz8a/pagoda restated in C.
 * TEST INFRASTRUCTURE ONLY -- see pagoda_oracle.h.  Build with
 *   gcc -O2 -fno-fast-math -ffp-contract=off
 * so that every float operation rounds once, exactly as the reference's scalar Rust does.
 * Every sum is a left fold in index order (Rust's `iter().sum()` and explicit `+=` loops).
 */
#include "pagoda_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define PGO_EPS 1e-9f /* sampler.rs:8 */

/* ------------------------------------------------------------------ rng.rs */

void pgo_rng_new(pgo_rng *r, uint64_t seed) { r->s = seed + 0x9e3779b97f4a7c15ULL; } /* :10-13 */

uint64_t pgo_rng_next_u64(pgo_rng *r) { /* :15-21 */
    r->s += 0x9e3779b97f4a7c15ULL;
    uint64_t z = r->s;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

double pgo_rng_next_f64(pgo_rng *r) { /* :24-26 */
    return (double)(pgo_rng_next_u64(r) >> 11) * (1.0 / (double)(1ULL << 53));
}

float pgo_rng_next_f32(pgo_rng *r) { return (float)pgo_rng_next_f64(r); } /* :28-30 */

/* -------------------------------------------------------------- sampler.rs */

static int finite_f(float x) { return isfinite(x); }

uint32_t pgo_argmax(const float *xs, size_t n) { /* :59-70: largest finite, strict >, 0 if none */
    size_t best = 0;
    float best_v = -INFINITY;
    for (size_t i = 0; i < n; i++) {
        if (finite_f(xs[i]) && xs[i] > best_v) {
            best_v = xs[i];
            best = i;
        }
    }
    return (uint32_t)best;
}

void pgo_log_softmax(const float *xs, size_t n, float *out) { /* :73-87 */
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++) max = fmaxf(max, xs[i]); /* f32::max ignores NaN like fmaxf */
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float e = expf(xs[i] - max);
        out[i] = e;
        sum += e;
    }
    float log_sum = fmaxf(logf(sum), 1.17549435e-38f); /* .max(f32::MIN_POSITIVE) */
    for (size_t i = 0; i < n; i++) out[i] = logf(out[i]) - log_sum;
}

void pgo_temperature_softmax(float *xs, size_t n, float temp) { /* :92-114 */
    float t = fmaxf(temp, PGO_EPS);
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++)
        if (finite_f(xs[i])) max = fmaxf(max, xs[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        if (finite_f(xs[i])) {
            float e = expf((xs[i] - max) / t);
            xs[i] = e;
            sum += e;
        } else {
            xs[i] = 0.0f;
        }
    }
    if (sum > PGO_EPS)
        for (size_t i = 0; i < n; i++) xs[i] /= sum;
}

static int cmp_desc_f(const void *a, const void *b) {
    float x = *(const float *)a, y = *(const float *)b;
    return (x < y) - (x > y);
}

void pgo_apply_top_k(float *xs, size_t n, uint64_t k) { /* :116-128 */
    if (k == 0 || k >= n) return;
    float *sorted = (float *)malloc(n * sizeof(float));
    memcpy(sorted, xs, n * sizeof(float));
    qsort(sorted, n, sizeof(float), cmp_desc_f); /* values only: any correct sort gives sorted[k-1] */
    float threshold = sorted[k - 1];
    free(sorted);
    for (size_t i = 0; i < n; i++)
        if (xs[i] < threshold) xs[i] = 0.0f;
}

/* stable merge sort of indices by probability descending (Rust's sort_by is stable, so equal
 * probabilities stay in ascending id order) */
static void sort_idx_desc(const float *xs, uint32_t *idx, uint32_t *tmp, size_t n) {
    for (size_t w = 1; w < n; w *= 2) {
        for (size_t lo = 0; lo < n; lo += 2 * w) {
            size_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            size_t a = lo, b = mid, o = lo;
            while (a < mid && b < hi) tmp[o++] = (xs[idx[b]] > xs[idx[a]]) ? idx[b++] : idx[a++];
            while (a < mid) tmp[o++] = idx[a++];
            while (b < hi) tmp[o++] = idx[b++];
        }
        memcpy(idx, tmp, n * sizeof(uint32_t));
    }
}

/* shared by pgo_apply_top_p and the margin bookkeeping: returns the number of kept entries
 * and, through cum_before/cum_at, the running sum just before and at the boundary entry */
static size_t top_p_core(float *xs, size_t n, float p, float *cum_before, float *cum_at) {
    uint32_t *idx = (uint32_t *)malloc(2 * n * sizeof(uint32_t));
    uint8_t *keep = (uint8_t *)calloc(n, 1);
    for (size_t i = 0; i < n; i++) idx[i] = (uint32_t)i;
    sort_idx_desc(xs, idx, idx + n, n);
    float cum = 0.0f, prev = 0.0f;
    size_t kept = 0;
    int hit = 0;
    for (size_t j = 0; j < n; j++) {
        prev = cum;
        cum += xs[idx[j]];
        keep[idx[j]] = 1;
        kept++;
        if (cum >= p) { hit = 1; break; }
    }
    if (cum_before) *cum_before = hit ? prev : -1.0f;
    if (cum_at) *cum_at = hit ? cum : -1.0f;
    for (size_t i = 0; i < n; i++)
        if (!keep[i]) xs[i] = 0.0f;
    free(idx);
    free(keep);
    return kept;
}

void pgo_apply_top_p(float *xs, size_t n, float p) { /* :130-150 */
    if (p >= 1.0f - PGO_EPS) return; /* 1.0f - 1e-9f == 1.0f */
    top_p_core(xs, n, p, NULL, NULL);
}

uint32_t pgo_sample_categorical(const float *probs, size_t n, float u01, int *drew) { /* :40-55 */
    float total = 0.0f;
    for (size_t i = 0; i < n; i++) total += probs[i];
    if (total <= PGO_EPS) {
        if (drew) *drew = 0;
        return pgo_argmax(probs, n);
    }
    if (drew) *drew = 1;
    float u = u01 * total;
    float acc = 0.0f;
    for (size_t i = 0; i < n; i++) {
        acc += probs[i];
        if (u < acc) return (uint32_t)i;
    }
    return (uint32_t)(n - 1);
}

uint32_t pgo_sample(const float *logits, size_t n, float temperature, uint64_t top_k, float top_p,
                    float u, int *drew) { /* :28-37 */
    if (temperature < 1e-5f) {
        if (drew) *drew = 0;
        return pgo_argmax(logits, n);
    }
    float *probs = (float *)malloc(n * sizeof(float));
    memcpy(probs, logits, n * sizeof(float));
    pgo_temperature_softmax(probs, n, temperature);
    pgo_apply_top_k(probs, n, top_k);
    pgo_apply_top_p(probs, n, top_p);
    uint32_t tok = pgo_sample_categorical(probs, n, u, drew);
    free(probs);
    return tok;
}

/* --------------------------------------------------------------- engine.rs */

int pgo_logits_sane(const float *logits, size_t n, size_t vocab) { /* :1278-1280 */
    if (n != vocab) return 0;
    for (size_t i = 0; i < n; i++)
        if (!finite_f(logits[i])) return 0;
    return 1;
}

/* The reference counts ids with a HashMap and then walks its entries (engine.rs:1557-1572).
 * Each distinct id is touched exactly once per penalty, so the iteration order does not
 * matter; an open-addressing table gives the same result. */
typedef struct { uint32_t *key; uint32_t *cnt; size_t cap; } id_counts;

static void id_counts_build(id_counts *h, const uint32_t *ids, size_t n) {
    size_t cap = 16;
    while (cap < 2 * n + 1) cap *= 2;
    h->cap = cap;
    h->key = (uint32_t *)malloc(cap * sizeof(uint32_t));
    h->cnt = (uint32_t *)calloc(cap, sizeof(uint32_t));
    for (size_t i = 0; i < n; i++) {
        size_t s = (ids[i] * 2654435761u) & (cap - 1);
        while (h->cnt[s] && h->key[s] != ids[i]) s = (s + 1) & (cap - 1);
        h->key[s] = ids[i];
        h->cnt[s]++;
    }
}
static void id_counts_free(id_counts *h) { free(h->key); free(h->cnt); }

void pgo_apply_penalties(float *logits, size_t n, const uint32_t *output, size_t n_out, float freq,
                         float pres) { /* :1553-1573 */
    if (fabsf(freq) < 1e-6f && fabsf(pres) < 1e-6f) return;
    id_counts h;
    id_counts_build(&h, output, n_out);
    for (size_t s = 0; s < h.cap; s++)
        if (h.cnt[s] && h.key[s] < n) logits[h.key[s]] -= freq * (float)h.cnt[s];
    if (fabsf(pres) > 1e-6f)
        for (size_t s = 0; s < h.cap; s++)
            if (h.cnt[s] && h.key[s] < n) logits[h.key[s]] -= pres;
    id_counts_free(&h);
}

void pgo_apply_repetition(float *logits, size_t n, const uint32_t *output, size_t n_out, float rep) {
    if (rep == 1.0f) return;
    id_counts h;
    id_counts_build(&h, output, n_out);
    for (size_t s = 0; s < h.cap; s++) {
        if (!h.cnt[s] || h.key[s] >= n) continue;
        float x = logits[h.key[s]];
        logits[h.key[s]] = x > 0.0f ? x / rep : x * rep;
    }
    id_counts_free(&h);
}

/* -------------------------------------------------------- grammar.rs:73-85 */

void pgo_mask_logits_bytes(const uint8_t *allowed, size_t n_allowed, float *logits, size_t n) {
    uint8_t keep[256];
    memset(keep, 0, sizeof keep);
    for (size_t i = 0; i < n_allowed; i++) keep[allowed[i]] = 1;
    for (size_t i = 0; i < n; i++) {
        size_t byte_idx = i - 3; /* wrapping_sub(FIRST_BYTE_ID) */
        int ok = byte_idx < 256 && keep[byte_idx];
        if (!ok) logits[i] = -INFINITY;
    }
}

void pgo_mask_logits_bits(const uint32_t *words, float *logits, size_t n) {
    for (size_t i = 0; i < n; i++)
        if (!((words[i >> 5] >> (i & 31)) & 1u)) logits[i] = -INFINITY;
}

void pgo_bf16_to_f32(const uint16_t *in, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        uint32_t b = (uint32_t)in[i] << 16;
        memcpy(&out[i], &b, 4);
    }
}

/* ------------------------------------------- one row, engine.rs:1286-1314 */

static float rel_gap(float a, float b) {
    float d = fabsf(a - b), s = fmaxf(fabsf(a), fabsf(b));
    return s > 0.0f ? d / s : 1.0f;
}

void pgo_sample_row(const float *logits_in, size_t n, const pgo_row_params *p, pgo_row_out *out,
                    float *work, float *probs_out) {
    float *logits = work, *probs = work + n;
    memset(out, 0, sizeof *out);
    out->margin = out->margin_k = out->margin_p = out->margin_cdf = 1.0f;
    out->row_max = -INFINITY;
    /* :1292-1295 sanity before anything else */
    if (!pgo_logits_sane(logits_in, n, n)) {
        out->status = PGO_ROW_NONFINITE;
        return;
    }
    memcpy(logits, logits_in, n * sizeof(float));
    /* :1296 penalties (the repetition extension slots in first) */
    pgo_apply_repetition(logits, n, p->history, p->n_history, p->rep);
    pgo_apply_penalties(logits, n, p->history, p->n_history, p->freq, p->pres);
    /* :1297-1313 grammar */
    if (p->mask_words || p->grammar_dead) {
        if (p->grammar_dead) {
            out->status = PGO_ROW_DEAD;
            return;
        }
        pgo_mask_logits_bits(p->mask_words, logits, n);
        if (p->grammar_complete && p->eos_id >= 0 && (size_t)p->eos_id < n &&
            !finite_f(logits[p->eos_id]))
            logits[p->eos_id] = 0.0f;
    }
    int any = 0;
    for (size_t i = 0; i < n; i++)
        if (finite_f(logits[i])) { any = 1; out->row_max = fmaxf(out->row_max, logits[i]); }
    out->argmax = pgo_argmax(logits, n);
    if (!any) out->status = PGO_ROW_EMPTY;
    /* :1314 -> sampler.rs:28-37 */
    if (p->temperature < 1e-5f) {
        out->token = out->argmax;
        return;
    }
    memcpy(probs, logits, n * sizeof(float));
    {   /* temperature_softmax, restated inline so the sum can be reported */
        float t = fmaxf(p->temperature, PGO_EPS), max = out->row_max, sum = 0.0f;
        for (size_t i = 0; i < n; i++) {
            if (finite_f(probs[i])) {
                float e = expf((probs[i] - max) / t);
                probs[i] = e;
                sum += e;
            } else probs[i] = 0.0f;
        }
        if (sum > PGO_EPS)
            for (size_t i = 0; i < n; i++) probs[i] /= sum;
        out->sumexp = sum;
    }
    if (p->top_k != 0 && (size_t)p->top_k < n) {
        float *sorted = (float *)malloc(n * sizeof(float));
        memcpy(sorted, probs, n * sizeof(float));
        qsort(sorted, n, sizeof(float), cmp_desc_f);
        float threshold = sorted[p->top_k - 1];
        /* margin: gap to the next smaller distinct probability */
        size_t j = p->top_k;
        while (j < n && sorted[j] == threshold) j++;
        if (j < n && threshold > 0.0f) out->margin_k = rel_gap(threshold, sorted[j]);
        free(sorted);
        for (size_t i = 0; i < n; i++)
            if (probs[i] < threshold) probs[i] = 0.0f;
    }
    if (!(p->top_p >= 1.0f - PGO_EPS)) {
        float before, at;
        top_p_core(probs, n, p->top_p, &before, &at);
        if (at >= 0.0f) out->margin_p = fminf(rel_gap(at, p->top_p), rel_gap(before, p->top_p));
    }
    for (size_t i = 0; i < n; i++) out->n_kept += probs[i] > 0.0f;
    {   /* sample_categorical with margin bookkeeping */
        float total = 0.0f;
        for (size_t i = 0; i < n; i++) total += probs[i];
        out->total = total;
        if (total <= PGO_EPS) {
            out->token = pgo_argmax(probs, n);
        } else {
            out->drew = 1;
            float u = p->uniform * total, acc = 0.0f, prev = 0.0f;
            uint32_t tok = (uint32_t)(n - 1);
            int hit = 0;
            for (size_t i = 0; i < n; i++) {
                prev = acc;
                acc += probs[i];
                if (u < acc) { tok = (uint32_t)i; hit = 1; break; }
            }
            out->token = tok;
            if (hit) out->margin_cdf = fminf(fabsf(acc - u) / total, fabsf(u - prev) / total + (prev == 0.0f ? 1.0f : 0.0f));
            else out->margin_cdf = fabsf(u - acc) / total;
        }
    }
    out->margin = fminf(out->margin_k, fminf(out->margin_p, out->margin_cdf));
    if (probs_out) memcpy(probs_out, probs, n * sizeof(float));
}

typedef struct { const pgo_batch *b; pgo_row_out *out; size_t lo, hi; } batch_job;

static void *batch_worker(void *arg) {
    batch_job *j = (batch_job *)arg;
    const pgo_batch *b = j->b;
    float *work = (float *)malloc(2 * b->vocab * sizeof(float));
    for (size_t r = j->lo; r < j->hi; r++) {
        pgo_row_params p;
        memset(&p, 0, sizeof p);
        p.temperature = b->temperature ? b->temperature[r] : 0.0f;
        p.top_p = b->top_p ? b->top_p[r] : 1.0f;
        p.top_k = b->top_k ? b->top_k[r] : 0;
        p.freq = b->freq ? b->freq[r] : 0.0f;
        p.pres = b->pres ? b->pres[r] : 0.0f;
        p.rep = b->rep ? b->rep[r] : 1.0f;
        if (b->hist_offsets) {
            p.history = b->hist_ids + b->hist_offsets[r];
            p.n_history = b->hist_offsets[r + 1] - b->hist_offsets[r];
        }
        p.mask_words = b->mask_rows ? b->mask_rows[r] : NULL;
        p.grammar_complete = b->row_flags ? (b->row_flags[r] & 1) : 0;
        p.grammar_dead = b->row_flags ? ((b->row_flags[r] >> 1) & 1) : 0;
        p.eos_id = b->eos_id;
        p.uniform = b->uniform ? b->uniform[r] : 0.0f;
        pgo_sample_row(b->logits + r * b->row_stride, b->vocab, &p, &j->out[r], work, NULL);
    }
    free(work);
    return NULL;
}

void pgo_sample_batch(const pgo_batch *b, pgo_row_out *out, int n_threads) {
    if (n_threads < 1) n_threads = 1;
    if ((size_t)n_threads > b->rows) n_threads = b->rows ? (int)b->rows : 1;
    batch_job *jobs = (batch_job *)malloc(n_threads * sizeof(batch_job));
    pthread_t *th = (pthread_t *)malloc(n_threads * sizeof(pthread_t));
    for (int t = 0; t < n_threads; t++) {
        jobs[t].b = b;
        jobs[t].out = out;
        jobs[t].lo = b->rows * t / n_threads;
        jobs[t].hi = b->rows * (t + 1) / n_threads;
        if (n_threads == 1) batch_worker(&jobs[t]);
        else pthread_create(&th[t], NULL, batch_worker, &jobs[t]);
    }
    if (n_threads > 1)
        for (int t = 0; t < n_threads; t++) pthread_join(th[t], NULL);
    free(jobs);
    free(th);
}

/* ---------------------------------------- vocabulary-sharded merge (extension) */

typedef struct { float v; uint32_t id; } cand_t;
static int cmp_cand(const void *a, const void *b) {
    const cand_t *x = (const cand_t *)a, *y = (const cand_t *)b;
    if (x->v != y->v) return (x->v < y->v) - (x->v > y->v);
    return (x->id > y->id) - (x->id < y->id);
}

void pgo_tp_sample_row(const float *logits_in, size_t n, uint32_t n_shards, uint32_t cand,
                       const pgo_row_params *p, pgo_tp_out *out) {
    memset(out, 0, sizeof *out);
    out->margin = 1.0f;
    out->gmax = -INFINITY;
    /* the chain in front of the sampler is that of pgo_sample_row: every step touches one logit at a
     * time, so running it on the whole row equals running it shard by shard */
    if (p->top_k > cand) { out->status = PGO_ROW_BAD_PARAM; return; }
    if (!pgo_logits_sane(logits_in, n, n)) { out->status = PGO_ROW_NONFINITE; return; }
    float *logits = (float *)malloc(n * sizeof(float));
    memcpy(logits, logits_in, n * sizeof(float));
    pgo_apply_repetition(logits, n, p->history, p->n_history, p->rep);
    pgo_apply_penalties(logits, n, p->history, p->n_history, p->freq, p->pres);
    if (p->mask_words || p->grammar_dead) {
        if (p->grammar_dead) { out->status = PGO_ROW_DEAD; free(logits); return; }
        pgo_mask_logits_bits(p->mask_words, logits, n);
        if (p->grammar_complete && p->eos_id >= 0 && (size_t)p->eos_id < n && !finite_f(logits[p->eos_id]))
            logits[p->eos_id] = 0.0f;
    }
    size_t per = n / n_shards;
    float temperature = p->temperature;
    float t = fmaxf(temperature, PGO_EPS);
    int greedy = temperature < 1e-5f;
    float *m = (float *)malloc(n_shards * sizeof(float)), *s = (float *)malloc(n_shards * sizeof(float));
    cand_t *all = (cand_t *)malloc(per * sizeof(cand_t));
    cand_t *keep = (cand_t *)malloc((size_t)n_shards * cand * sizeof(cand_t));
    size_t n_keep = 0;
    float M = -INFINITY, best = -INFINITY;
    int have = 0;
    for (uint32_t r = 0; r < n_shards; r++) {
        size_t lo = r * per, hi = lo + per, n_fin = 0;
        float mr = -INFINITY;
        for (size_t i = lo; i < hi; i++)
            if (finite_f(logits[i])) { mr = fmaxf(mr, logits[i]); all[n_fin].v = logits[i]; all[n_fin].id = (uint32_t)i; n_fin++; }
        float sr = 0.0f;
        if (!greedy)   /* non-finite entries contribute zero, as in temperature_softmax */
            for (size_t i = lo; i < hi; i++)
                if (finite_f(logits[i])) sr += expf((logits[i] - mr) / t);
        m[r] = mr; s[r] = sr;
        M = fmaxf(M, mr);
        if (n_fin) {   /* shard argmax: largest value, lowest id; shards come in id order */
            float bv = all[0].v; uint32_t bi = all[0].id;
            for (size_t j = 1; j < n_fin; j++) if (all[j].v > bv) { bv = all[j].v; bi = all[j].id; }
            if (!have || bv > best) { best = bv; out->argmax = bi; have = 1; }
        }
        if (!greedy) {
            qsort(all, n_fin, sizeof(cand_t), cmp_cand);
            size_t take = cand < n_fin ? cand : n_fin;
            memcpy(keep + n_keep, all, take * sizeof(cand_t));
            n_keep += take;
        }
    }
    out->gmax = M;
    if (!have) out->status = PGO_ROW_EMPTY;
    if (greedy || !have) { out->token = out->argmax; free(logits); free(m); free(s); free(all); free(keep); return; }
    float S = 0.0f;
    for (uint32_t r = 0; r < n_shards; r++)
        if (finite_f(m[r])) S += s[r] * expf((m[r] - M) / t);
    out->gsum = S;
    float *probs = (float *)calloc(n, sizeof(float));
    for (size_t j = 0; j < n_keep; j++) {
        float e = expf((keep[j].v - M) / t);
        probs[keep[j].id] = S > PGO_EPS ? e / S : e;
    }
    if (p->top_k != 0 && (size_t)p->top_k <= n_keep) {   /* apply_top_k over the union (ties survive) */
        float *sorted = (float *)malloc(n_keep * sizeof(float));
        for (size_t j = 0; j < n_keep; j++) sorted[j] = probs[keep[j].id];
        qsort(sorted, n_keep, sizeof(float), cmp_desc_f);
        float threshold = sorted[p->top_k - 1];
        size_t j = p->top_k;
        while (j < n_keep && sorted[j] == threshold) j++;
        if (j < n_keep && threshold > 0.0f) out->margin = fminf(out->margin, rel_gap(threshold, sorted[j]));
        free(sorted);
        for (size_t q = 0; q < n_keep; q++)
            if (probs[keep[q].id] < threshold) probs[keep[q].id] = 0.0f;
    }
    if (!(p->top_p >= 1.0f - PGO_EPS)) {
        float before, at;
        top_p_core(probs, n, p->top_p, &before, &at);
        if (at >= 0.0f) {
            out->margin = fminf(out->margin, rel_gap(at, p->top_p));
            out->margin = fminf(out->margin, rel_gap(before, p->top_p));
        }
    }
    for (size_t i = 0; i < n; i++) out->n_kept += probs[i] > 0.0f;
    float total = 0.0f;
    for (size_t i = 0; i < n; i++) total += probs[i];
    out->total = total;
    if (total <= PGO_EPS) {
        out->token = out->argmax;
    } else {
        out->drew = 1;
        float uu = p->uniform * total, acc = 0.0f, prev = 0.0f;
        uint32_t tok = (uint32_t)(n - 1);
        int hit = 0;
        for (size_t i = 0; i < n; i++) {
            prev = acc; acc += probs[i];
            if (uu < acc) { tok = (uint32_t)i; hit = 1; break; }
        }
        out->token = tok;
        if (hit) {
            out->margin = fminf(out->margin, fabsf(acc - uu) / total);
            out->margin = fminf(out->margin, fabsf(uu - prev) / total + (prev == 0.0f ? 1.0f : 0.0f));
        } else out->margin = fminf(out->margin, fabsf(uu - acc) / total);
    }
    free(probs); free(logits); free(m); free(s); free(all); free(keep);
}

uint32_t pgo_draft_accept(const uint32_t *row_argmax, const uint32_t *draft, uint32_t n,
                          uint32_t *next) {
    uint32_t a = 0;
    while (a < n && row_argmax[a] == draft[a]) a++;
    *next = row_argmax[a < n ? a : n - 1];
    return a;
}
