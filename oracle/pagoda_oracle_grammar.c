/*
 * CPU oracle, grammar half: the byte regex (Thompson NFA re-run from scratch on every
 * query) and the JSON prefix scanner of quantz8a/pagoda, restated in C.
 * TEST INFRASTRUCTURE ONLY -- see pagoda_oracle.h.
 *
 * The restatement keeps the reference's observable quirks, because the shipped host code
 * (DFA tabulation) is checked against it:
 *   - state ids are handed out in the same order, since the `{m}` repetition copies the id
 *     range [start, end] of a fragment (grammar.rs:206-233) and therefore only duplicates
 *     fragments whose states are contiguous (a group closed by `|`, `*`, `+` or `?` is not);
 *   - `{m,n}` checks n but expands exactly m copies, and `{0}` still leaves one copy
 *     (grammar.rs:298-323, 343-350);
 *   - `^` and `$` are skipped and the next atom is parsed in their place (grammar.rs:372-375);
 *   - a JSON number that ends the input in its integer, fraction-digit or exponent-digit
 *     phase counts as finished (grammar.rs:825-831).
 */
#include "pagoda_oracle.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ NFA */

typedef struct { int16_t c; /* -1 = epsilon */ uint32_t to; } edge_t;
typedef struct { edge_t *e; uint32_t n, cap; } edges_t;

struct pgo_regex {
    edges_t *st;
    uint8_t *accept;
    uint32_t n, cap;
    uint32_t start;
};

typedef struct { uint32_t s, e; } frag_t;

static uint32_t nfa_fresh(pgo_regex *b) { /* grammar.rs:120-124 */
    if (b->n == b->cap) {
        b->cap = b->cap ? 2 * b->cap : 64;
        b->st = (edges_t *)realloc(b->st, b->cap * sizeof(edges_t));
        b->accept = (uint8_t *)realloc(b->accept, b->cap);
    }
    memset(&b->st[b->n], 0, sizeof(edges_t));
    b->accept[b->n] = 0;
    return b->n++;
}

static void nfa_edge(pgo_regex *b, uint32_t from, int16_t c, uint32_t to) {
    edges_t *s = &b->st[from];
    if (s->n == s->cap) {
        s->cap = s->cap ? 2 * s->cap : 4;
        s->e = (edge_t *)realloc(s->e, s->cap * sizeof(edge_t));
    }
    s->e[s->n].c = c;
    s->e[s->n].to = to;
    s->n++;
}

static frag_t frag_set(pgo_regex *b, const uint8_t set[256]) { /* :134-159 */
    frag_t f;
    f.s = nfa_fresh(b);
    f.e = nfa_fresh(b);
    for (int c = 0; c < 256; c++)
        if (set[c]) nfa_edge(b, f.s, (int16_t)c, f.e);
    return f;
}

static frag_t frag_char(pgo_regex *b, uint8_t c) {
    uint8_t set[256];
    memset(set, 0, sizeof set);
    set[c] = 1;
    return frag_set(b, set);
}

static frag_t frag_concat(pgo_regex *b, frag_t x, frag_t y) { /* :161-164 */
    nfa_edge(b, x.e, -1, y.s);
    frag_t f = { x.s, y.e };
    return f;
}

/* alt / star / plus / opt: two fresh states after the operand(s), wired as :166-202 */
static frag_t frag_wrap(pgo_regex *b, frag_t x, const frag_t *y, int skip, int loop) {
    frag_t f;
    f.s = nfa_fresh(b);
    f.e = nfa_fresh(b);
    nfa_edge(b, f.s, -1, x.s);
    if (y) nfa_edge(b, f.s, -1, y->s);
    if (skip) nfa_edge(b, f.s, -1, f.e);
    if (loop) nfa_edge(b, x.e, -1, x.s);
    nfa_edge(b, x.e, -1, f.e);
    if (y) nfa_edge(b, y->e, -1, f.e);
    return f;
}

/* :206-233: duplicate the states whose ids lie in [f.s, f.e], keeping only edges that stay
 * inside that id range */
static frag_t frag_copy(pgo_regex *b, frag_t f) {
    uint32_t lo = f.s, hi = f.e, span = hi - lo + 1, off = b->n;
    for (uint32_t i = 0; i < span; i++) nfa_fresh(b);
    for (uint32_t i = 0; i < span; i++) {
        edges_t src = b->st[lo + i]; /* edge storage of the source does not move below */
        for (uint32_t j = 0; j < src.n; j++) {
            uint32_t to = src.e[j].to;
            if (to >= lo && to <= hi) nfa_edge(b, off + i, src.e[j].c, to - lo + off);
        }
        b->accept[off + i] = b->accept[lo + i];
    }
    frag_t r = { off, off + span - 1 };
    return r;
}

typedef struct { const uint8_t *p; size_t n, pos; const char *err; } parser_t;

static int pk(const parser_t *ps) { return ps->pos < ps->n ? ps->p[ps->pos] : -1; }
static int pk1(const parser_t *ps) { return ps->pos + 1 < ps->n ? ps->p[ps->pos + 1] : -1; }
static int bump(parser_t *ps) { int c = pk(ps); if (c >= 0) ps->pos++; return c; }

static uint8_t unescape(uint8_t c) { /* :448-456 */
    switch (c) {
    case 'n': return '\n';
    case 't': return '\t';
    case 'r': return '\r';
    case '0': return 0;
    default: return c;
    }
}

static int parse_alt(parser_t *ps, pgo_regex *b, frag_t *out);

static int parse_class(parser_t *ps, pgo_regex *b, frag_t *out) { /* :390-445 */
    uint8_t set[256];
    memset(set, 0, sizeof set);
    int negated = 0, first = 1;
    if (pk(ps) == '^') { negated = 1; ps->pos++; }
    for (;;) {
        int c = pk(ps);
        if (c < 0) { ps->err = "unclosed character class"; return 0; }
        if (c == ']' && !first) { ps->pos++; break; }
        first = 0;
        ps->pos++;
        uint8_t lo;
        if (c == '\\') {
            int e = bump(ps);
            if (e < 0) { ps->err = "bad escape in class"; return 0; }
            lo = unescape((uint8_t)e);
        } else lo = (uint8_t)c;
        set[lo] = 1;
        if (pk(ps) == '-' && pk1(ps) >= 0 && pk1(ps) != ']') {
            ps->pos++;
            int hr = bump(ps);
            if (hr < 0) { ps->err = "bad range"; return 0; }
            uint8_t hi;
            if (hr == '\\') {
                int e = bump(ps);
                if (e < 0) { ps->err = "bad escape in range"; return 0; }
                hi = unescape((uint8_t)e);
            } else hi = (uint8_t)hr;
            if (hi < lo) { ps->err = "character range is descending"; return 0; }
            for (int v = lo; v <= hi; v++) set[v] = 1;
        }
    }
    if (negated)
        for (int v = 0; v < 256; v++) set[v] = !set[v];
    *out = frag_set(b, set);
    return 1;
}

static int parse_atom(parser_t *ps, pgo_regex *b, frag_t *out) { /* :352-388 */
    for (;;) {
        int c = pk(ps);
        if (c < 0) { ps->err = "unexpected end of pattern"; return 0; }
        if (c == '(') {
            ps->pos++;
            if (!parse_alt(ps, b, out)) return 0;
            if (bump(ps) == ')') return 1;
            ps->err = "unclosed group";
            return 0;
        }
        if (c == '[') { ps->pos++; return parse_class(ps, b, out); }
        if (c == '.') {
            uint8_t set[256];
            memset(set, 1, sizeof set);
            ps->pos++;
            *out = frag_set(b, set);
            return 1;
        }
        if (c == '^' || c == '$') { ps->pos++; continue; } /* skipped; next atom takes its place */
        if (c == '\\') {
            ps->pos++;
            int e = bump(ps);
            if (e < 0) { ps->err = "dangling escape"; return 0; }
            *out = frag_char(b, unescape((uint8_t)e));
            return 1;
        }
        ps->pos++;
        *out = frag_char(b, (uint8_t)c);
        return 1;
    }
}

/* digits -> count; 0 = ok, 1 = empty, 2 = does not fit a usize */
static int take_count(parser_t *ps, uint64_t *v) {
    size_t begin = ps->pos;
    uint64_t acc = 0;
    int overflow = 0;
    while (pk(ps) >= '0' && pk(ps) <= '9') {
        uint64_t d = (uint64_t)(pk(ps) - '0');
        if (acc > (UINT64_MAX - d) / 10) overflow = 1; else acc = acc * 10 + d;
        ps->pos++;
    }
    if (ps->pos == begin) return 1;
    *v = acc;
    return overflow ? 2 : 0;
}

static int parse_repeat(parser_t *ps, pgo_regex *b, frag_t *out) { /* :282-328 */
    frag_t f;
    if (!parse_atom(ps, b, &f)) return 0;
    for (;;) {
        int c = pk(ps);
        if (c == '*') { ps->pos++; f = frag_wrap(b, f, NULL, 1, 1); }
        else if (c == '+') { ps->pos++; f = frag_wrap(b, f, NULL, 0, 1); }
        else if (c == '?') { ps->pos++; f = frag_wrap(b, f, NULL, 1, 0); }
        else if (c == '{') {
            ps->pos++;
            uint64_t lo = 0, hi = 0;
            int r = take_count(ps, &lo);
            if (r == 1) { ps->err = "missing repetition count"; return 0; }
            if (r == 2) { ps->err = "bad repetition count"; return 0; }
            if (pk(ps) == ',') {
                ps->pos++;
                r = take_count(ps, &hi);
                if (r == 1) { ps->err = "missing max repetition count"; return 0; }
                if (r == 2) { ps->err = "bad max repetition count"; return 0; }
            } else hi = lo;
            if (pk(ps) != '}') { ps->err = "unclosed repetition"; return 0; }
            ps->pos++;
            if (hi < lo) { ps->err = "descending repetition bounds"; return 0; }
            frag_t acc = f; /* exactly `lo` copies; the upper bound is not expanded */
            for (uint64_t i = 1; i < lo; i++) acc = frag_concat(b, acc, frag_copy(b, f));
            f = acc;
        } else break;
    }
    *out = f;
    return 1;
}

static int parse_concat(parser_t *ps, pgo_regex *b, frag_t *out) { /* :268-280 */
    frag_t l;
    if (!parse_repeat(ps, b, &l)) return 0;
    for (;;) {
        int c = pk(ps);
        if (c < 0 || c == ')' || c == '|') break;
        frag_t r;
        if (!parse_repeat(ps, b, &r)) return 0;
        l = frag_concat(b, l, r);
    }
    *out = l;
    return 1;
}

static int parse_alt(parser_t *ps, pgo_regex *b, frag_t *out) { /* :258-266 */
    frag_t l;
    if (!parse_concat(ps, b, &l)) return 0;
    while (pk(ps) == '|') {
        ps->pos++;
        frag_t r;
        if (!parse_concat(ps, b, &r)) return 0;
        l = frag_wrap(b, l, &r, 0, 0);
    }
    *out = l;
    return 1;
}

void pgo_regex_free(pgo_regex *re) {
    if (!re) return;
    for (uint32_t i = 0; i < re->n; i++) free(re->st[i].e);
    free(re->st);
    free(re->accept);
    free(re);
}

pgo_regex *pgo_regex_new(const char *pattern, char *err, size_t err_len) { /* :459-480 */
    pgo_regex *re = (pgo_regex *)calloc(1, sizeof *re);
    parser_t ps = { (const uint8_t *)pattern, strlen(pattern), 0, NULL };
    frag_t f;
    if (!parse_alt(&ps, re, &f)) {
        if (err && err_len) snprintf(err, err_len, "%s", ps.err ? ps.err : "error");
        pgo_regex_free(re);
        return NULL;
    }
    if (ps.pos != ps.n) {
        if (err && err_len)
            snprintf(err, err_len, "unexpected byte '%c' at position %zu", ps.p[ps.pos], ps.pos);
        pgo_regex_free(re);
        return NULL;
    }
    re->accept[f.e] = 1;
    re->start = f.s;
    return re;
}

/* :482-500 epsilon closure of `seeds` into the state set `set` (a byte per state) */
static void eps_closure(const pgo_regex *re, const uint32_t *seeds, uint32_t n_seeds, uint8_t *set) {
    uint32_t *stack = (uint32_t *)malloc(sizeof(uint32_t) * (re->n * 4 + n_seeds + 16));
    uint32_t sp = 0, cap = re->n * 4 + n_seeds + 16;
    memset(set, 0, re->n);
    for (uint32_t i = 0; i < n_seeds; i++) stack[sp++] = seeds[i];
    while (sp) {
        uint32_t s = stack[--sp];
        if (set[s]) continue;
        set[s] = 1;
        for (uint32_t j = 0; j < re->st[s].n; j++)
            if (re->st[s].e[j].c < 0) {
                if (sp == cap) { cap *= 2; stack = (uint32_t *)realloc(stack, cap * sizeof(uint32_t)); }
                stack[sp++] = re->st[s].e[j].to;
            }
    }
    free(stack);
}

/* :502-514 then closure; returns whether the new set is non-empty */
static int step_set(const pgo_regex *re, const uint8_t *cur, uint8_t byte, uint8_t *next) {
    uint32_t cap = 64, n = 0;
    uint32_t *seeds = (uint32_t *)malloc(cap * sizeof(uint32_t));
    for (uint32_t s = 0; s < re->n; s++) {
        if (!cur[s]) continue;
        for (uint32_t j = 0; j < re->st[s].n; j++)
            if (re->st[s].e[j].c == (int16_t)byte) {
                if (n == cap) { cap *= 2; seeds = (uint32_t *)realloc(seeds, cap * sizeof(uint32_t)); }
                seeds[n++] = re->st[s].e[j].to;
            }
    }
    eps_closure(re, seeds, n, next);
    free(seeds);
    for (uint32_t s = 0; s < re->n; s++)
        if (next[s]) return 1;
    return 0;
}

/* :516-526: returns 0 when the set died */
static int run_text(const pgo_regex *re, const uint8_t *text, size_t n, uint8_t *cur) {
    uint8_t *next = (uint8_t *)malloc(re->n);
    eps_closure(re, &re->start, 1, cur);
    int alive = 1;
    for (size_t i = 0; i < n && alive; i++) {
        alive = step_set(re, cur, text[i], next);
        memcpy(cur, next, re->n);
    }
    free(next);
    return alive;
}

/* :529-552 */
static void can_reach_accept(const pgo_regex *re, uint8_t *reach) {
    memset(reach, 0, re->n);
    int changed = 1;
    for (uint32_t s = 0; s < re->n; s++) reach[s] = re->accept[s];
    while (changed) {
        changed = 0;
        for (uint32_t s = 0; s < re->n; s++) {
            if (reach[s]) continue;
            for (uint32_t j = 0; j < re->st[s].n; j++)
                if (reach[re->st[s].e[j].to]) { reach[s] = 1; changed = 1; break; }
        }
    }
}

int pgo_regex_is_complete(const pgo_regex *re, const uint8_t *text, size_t n) { /* :554-556 */
    uint8_t *cur = (uint8_t *)malloc(re->n);
    int ok = 0;
    if (run_text(re, text, n, cur))
        for (uint32_t s = 0; s < re->n; s++) ok |= cur[s] && re->accept[s];
    free(cur);
    return ok;
}

int pgo_regex_allowed_bytes(const pgo_regex *re, const uint8_t *text, size_t n, uint8_t *out) {
    /* :558-575 */
    uint8_t *cur = (uint8_t *)malloc(re->n), *reach = (uint8_t *)malloc(re->n),
            *next = (uint8_t *)malloc(re->n);
    int count = -1;
    if (run_text(re, text, n, cur)) {
        can_reach_accept(re, reach);
        int live = 0;
        for (uint32_t s = 0; s < re->n; s++) live |= cur[s] && reach[s];
        if (live) {
            count = 0;
            for (int b = 0; b < 256; b++) {
                step_set(re, cur, (uint8_t)b, next);
                int ok = 0;
                for (uint32_t s = 0; s < re->n; s++) ok |= next[s] && reach[s];
                if (ok) out[count++] = (uint8_t)b;
            }
        }
    }
    free(cur); free(reach); free(next);
    return count;
}

/* ------------------------------------------------ JSON prefix scanner (:582-1016) */

enum { F_VALUE, F_OBJECT, F_COLON, F_AFTER_MEMBER, F_ARRAY, F_ARRAY_COMMA };
enum { SC_COMPLETE, SC_PREFIX, SC_DEAD };
enum { ST_CONTINUE, ST_DEAD, ST_EOF };
enum { N_ZERO, N_INT, N_FRAC_DOT, N_FRAC_DIGITS, N_EXP_E, N_EXP_SIGN, N_EXP_DIGITS };

typedef struct { const uint8_t *b; size_t n, i; uint8_t *stack; size_t sp, cap; } jscan;

static void set_bytes(uint8_t m[256], const char *s) { for (; *s; s++) m[(uint8_t)*s] = 1; }
static int is_ws(uint8_t c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r'; }
static int is_hex(uint8_t c) {
    return (c >= '0' && c <= '9') || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F');
}
static int is_digit(uint8_t c) { return c >= '0' && c <= '9'; }

static void push(jscan *s, uint8_t f) {
    if (s->sp == s->cap) { s->cap = s->cap ? 2 * s->cap : 32; s->stack = (uint8_t *)realloc(s->stack, s->cap); }
    s->stack[s->sp++] = f;
}
static void skip_ws(jscan *s) { while (s->i < s->n && is_ws(s->b[s->i])) s->i++; }

static void finish_value(jscan *s) { /* :750-757 */
    s->sp--;
    if (s->sp) {
        if (s->stack[s->sp - 1] == F_OBJECT) s->stack[s->sp - 1] = F_AFTER_MEMBER;
        else if (s->stack[s->sp - 1] == F_ARRAY) s->stack[s->sp - 1] = F_ARRAY_COMMA;
    }
}
static void finish_container(jscan *s) { s->sp--; finish_value(s); } /* :759-762 */

static void value_starts(uint8_t m[256]) { set_bytes(m, "{\"tf n0123456789[-"); } /* :966-972 */

static void prefix_allowed(int top, uint8_t m[256]) { /* :974-987 */
    switch (top) {
    case F_VALUE: value_starts(m); break;
    case F_OBJECT: set_bytes(m, "\"}"); break;
    case F_COLON: set_bytes(m, ":"); break;
    case F_AFTER_MEMBER: set_bytes(m, ",}"); break;
    case F_ARRAY: value_starts(m); set_bytes(m, "]"); break;
    default: set_bytes(m, ",]"); break;
    }
    set_bytes(m, " \t\n\r");
}

static int scan_string(jscan *s, uint8_t m[256]) { /* :764-800 */
    for (;;) {
        if (s->i == s->n) { for (int c = 0x20; c < 256; c++) m[c] = 1; return ST_EOF; }
        uint8_t c = s->b[s->i];
        if (c == '"') { s->i++; return ST_CONTINUE; }
        if (c == '\\') {
            s->i++;
            if (s->i == s->n) { set_bytes(m, "\"\\/bfnrtu"); return ST_EOF; }
            uint8_t e = s->b[s->i++];
            if (e == 'u') {
                for (int k = 0; k < 4; k++) {
                    if (s->i == s->n) { set_bytes(m, "0123456789abcdefABCDEF"); return ST_EOF; }
                    if (!is_hex(s->b[s->i])) return ST_DEAD;
                    s->i++;
                }
            } else if (!strchr("\"\\/bfnrt", e) || e == 0) return ST_DEAD;
        } else if (c < 0x20) return ST_DEAD;
        else s->i++;
    }
}

static int scan_number(jscan *s, uint8_t m[256]) { /* :802-901 */
    if (s->b[s->i] == '-') s->i++;
    if (s->i == s->n) { set_bytes(m, "0123456789"); return ST_EOF; }
    int phase;
    if (s->b[s->i] == '0') { s->i++; phase = N_ZERO; }
    else if (s->b[s->i] >= '1' && s->b[s->i] <= '9') { s->i++; phase = N_INT; }
    else return ST_DEAD;
    for (;;) {
        if (s->i == s->n) {
            switch (phase) {
            case N_ZERO: case N_INT: case N_FRAC_DIGITS: case N_EXP_DIGITS: return ST_CONTINUE;
            case N_EXP_E: set_bytes(m, "0123456789+-"); return ST_EOF;
            default: set_bytes(m, "0123456789"); return ST_EOF; /* FracDot, ExpSign */
            }
        }
        uint8_t c = s->b[s->i];
        switch (phase) {
        case N_ZERO:
            if (c == '.') { s->i++; phase = N_FRAC_DOT; }
            else if (c == 'e' || c == 'E') { s->i++; phase = N_EXP_E; }
            else return ST_CONTINUE;
            break;
        case N_INT:
            if (is_digit(c)) s->i++;
            else if (c == '.') { s->i++; phase = N_FRAC_DOT; }
            else if (c == 'e' || c == 'E') { s->i++; phase = N_EXP_E; }
            else return ST_CONTINUE;
            break;
        case N_FRAC_DOT:
            if (is_digit(c)) { s->i++; phase = N_FRAC_DIGITS; } else return ST_DEAD;
            break;
        case N_FRAC_DIGITS:
            if (is_digit(c)) s->i++;
            else if (c == 'e' || c == 'E') { s->i++; phase = N_EXP_E; }
            else return ST_CONTINUE;
            break;
        case N_EXP_E:
            if (c == '+' || c == '-') { s->i++; phase = N_EXP_SIGN; }
            else if (is_digit(c)) { s->i++; phase = N_EXP_DIGITS; }
            else return ST_DEAD;
            break;
        case N_EXP_SIGN:
            if (is_digit(c)) { s->i++; phase = N_EXP_DIGITS; } else return ST_DEAD;
            break;
        default:
            if (is_digit(c)) s->i++; else return ST_CONTINUE;
        }
    }
}

static int match_literal(jscan *s, const char *lit, uint8_t m[256]) { /* :903-914 */
    for (; *lit; lit++) {
        if (s->i == s->n) { m[(uint8_t)*lit] = 1; return ST_EOF; }
        if (s->b[s->i] != (uint8_t)*lit) return ST_DEAD;
        s->i++;
    }
    return ST_CONTINUE;
}

static int json_scan(const uint8_t *b, size_t n, uint8_t m[256]) { /* :625-733 */
    jscan s = { b, n, 0, NULL, 0, 0 };
    int result = -1;
    memset(m, 0, 256);
    push(&s, F_VALUE);
    while (result < 0) {
        if (!s.sp) {
            skip_ws(&s);
            result = s.i == s.n ? SC_COMPLETE : SC_DEAD;
            break;
        }
        int top = s.stack[s.sp - 1];
        skip_ws(&s);
        if (s.i == s.n) { prefix_allowed(top, m); result = SC_PREFIX; break; }
        uint8_t c = s.b[s.i];
        int st = ST_CONTINUE, is_value_scan = 0;
        switch (top) {
        case F_VALUE:
            is_value_scan = 1;
            if (c == '{') { s.i++; push(&s, F_OBJECT); is_value_scan = 0; }
            else if (c == '[') { s.i++; push(&s, F_ARRAY); is_value_scan = 0; }
            else if (c == '"') { s.i++; st = scan_string(&s, m); }
            else if (c == '-' || is_digit(c)) st = scan_number(&s, m);
            else if (c == 't') st = match_literal(&s, "true", m);
            else if (c == 'f') st = match_literal(&s, "false", m);
            else if (c == 'n') st = match_literal(&s, "null", m);
            else st = ST_DEAD;
            if (is_value_scan && st == ST_CONTINUE) finish_value(&s);
            break;
        case F_OBJECT:
            if (c == '"') { s.i++; st = scan_string(&s, m); if (st == ST_CONTINUE) push(&s, F_COLON); }
            else if (c == '}') { s.i++; finish_container(&s); }
            else st = ST_DEAD;
            break;
        case F_COLON:
            if (c == ':') { s.i++; s.stack[s.sp - 1] = F_VALUE; } else st = ST_DEAD;
            break;
        case F_AFTER_MEMBER:
            if (c == ',') { s.i++; s.stack[s.sp - 1] = F_OBJECT; }
            else if (c == '}') { s.i++; finish_container(&s); }
            else st = ST_DEAD;
            break;
        case F_ARRAY:
            if (c == ']') { s.i++; finish_container(&s); } else push(&s, F_VALUE);
            break;
        default:
            if (c == ',') { s.i++; s.stack[s.sp - 1] = F_ARRAY; }
            else if (c == ']') { s.i++; finish_container(&s); }
            else st = ST_DEAD;
        }
        if (st == ST_DEAD) result = SC_DEAD;
        else if (st == ST_EOF) result = SC_PREFIX;
    }
    free(s.stack);
    return result;
}

int pgo_json_is_complete(const uint8_t *text, size_t n) { /* :621-623 */
    uint8_t m[256];
    return json_scan(text, n, m) == SC_COMPLETE;
}

int pgo_json_allowed_bytes(const uint8_t *text, size_t n, uint8_t *out) { /* :613-619 */
    uint8_t m[256];
    int r = json_scan(text, n, m);
    if (r == SC_DEAD) return -1;
    if (r == SC_COMPLETE) return 0;
    int count = 0;
    for (int c = 0; c < 256; c++)
        if (m[c]) out[count++] = (uint8_t)c;
    return count;
}
