// Host side of constrained decoding: grammars tabulated into finite mask states.
//
// The reference recomputes the legal next bytes from scratch at every step: the regex re-runs its
// Thompson NFA over the whole decoded output and rebuilds reachability (pagoda/src/grammar.rs:516-575)
// and the JSON grammar rescans the whole string (grammar.rs:625-733).  Here each grammar is turned
// into a table once -- one allowed-token bitmask per state -- that lives on the device, and the
// per-row state is advanced on the host one byte at a time:
//
//   regex: subset construction over the same NFA (same state numbering, same `{m}` id-range copy,
//          see grammar.rs:206-233) gives a DFA; a state is a reachable epsilon-closed NFA set.
//   JSON:  the scanner's stack is unbounded, but the mask it returns depends only on where the
//          scan stops: one of 6 frame masks, string / escape / hex continuations, digit sets of
//          an open number, the next letter of a literal, "complete" or "dead" -- 19 classes.
//          The host keeps the real pushdown state and maps it to its class.
//
// State 0 of every table is the dead state (allowed_bytes() == None); flags bit 0 = complete,
// bit 1 = dead, as pgs_mask_table_upload expects.  No CUDA in this file.
#include "../../include/pagoda_sampler.h"

#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

namespace {

typedef std::vector<uint8_t> ByteSet;   // 256 flags

// ------------------------------------------------------------------------------- regex -> NFA
struct Edge { int c; uint32_t to; };   // c < 0: epsilon
struct Nfa {
    std::vector<std::vector<Edge>> st;
    std::vector<uint8_t> accept;
    uint32_t start = 0;
    uint32_t fresh() { st.emplace_back(); accept.push_back(0); return (uint32_t)st.size() - 1; }
};
struct Frag { uint32_t s, e; };

struct RegexParser {
    const std::string& p;
    size_t pos = 0;
    Nfa& n;
    std::string err;
    RegexParser(const std::string& pat, Nfa& nfa) : p(pat), n(nfa) {}
    int peek(size_t k = 0) const { return pos + k < p.size() ? (uint8_t)p[pos + k] : -1; }
    int bump() { int c = peek(); if (c >= 0) pos++; return c; }
    static uint8_t unesc(int c) { return c == 'n' ? '\n' : c == 't' ? '\t' : c == 'r' ? '\r' : c == '0' ? 0 : (uint8_t)c; }

    Frag set_frag(const ByteSet& set) {
        Frag f{n.fresh(), 0};
        f.e = n.fresh();
        for (int c = 0; c < 256; c++) if (set[c]) n.st[f.s].push_back({c, f.e});
        return f;
    }
    Frag concat(Frag a, Frag b) { n.st[a.e].push_back({-1, b.s}); return {a.s, b.e}; }
    // alternation / star / plus / optional all add two fresh states after their operands
    Frag wrap(Frag a, const Frag* b, bool skip, bool loop) {
        Frag f{n.fresh(), 0};
        f.e = n.fresh();
        n.st[f.s].push_back({-1, a.s});
        if (b) n.st[f.s].push_back({-1, b->s});
        if (skip) n.st[f.s].push_back({-1, f.e});
        if (loop) n.st[a.e].push_back({-1, a.s});
        n.st[a.e].push_back({-1, f.e});
        if (b) n.st[b->e].push_back({-1, f.e});
        return f;
    }
    // `{m}` duplicates the id range [f.s, f.e] and keeps only the edges that stay inside it
    Frag copy(Frag f) {
        const uint32_t lo = f.s, hi = f.e, span = hi - lo + 1, off = (uint32_t)n.st.size();
        for (uint32_t i = 0; i < span; i++) n.fresh();
        for (uint32_t i = 0; i < span; i++) {
            for (const Edge& e : n.st[lo + i])
                if (e.to >= lo && e.to <= hi) n.st[off + i].push_back({e.c, e.to - lo + off});
            n.accept[off + i] = n.accept[lo + i];
        }
        return {off, off + span - 1};
    }
    bool count(unsigned long long* v, int* why) {   // why: 1 empty, 2 overflow
        size_t b = pos;
        unsigned long long acc = 0;
        bool ovf = false;
        while (peek() >= '0' && peek() <= '9') {
            unsigned d = (unsigned)(peek() - '0');
            if (acc > (~0ull - d) / 10) ovf = true; else acc = acc * 10 + d;
            pos++;
        }
        if (pos == b) { *why = 1; return false; }
        if (ovf) { *why = 2; return false; }
        *v = acc;
        return true;
    }
    bool cls(Frag* out) {
        ByteSet set(256, 0);
        bool neg = false, first = true;
        if (peek() == '^') { neg = true; pos++; }
        for (;;) {
            int c = peek();
            if (c < 0) { err = "unclosed character class"; return false; }
            if (c == ']' && !first) { pos++; break; }
            first = false;
            pos++;
            uint8_t lo;
            if (c == '\\') { int e = bump(); if (e < 0) { err = "bad escape in class"; return false; } lo = unesc(e); }
            else lo = (uint8_t)c;
            set[lo] = 1;
            if (peek() == '-' && peek(1) >= 0 && peek(1) != ']') {
                pos++;
                int hr = bump();
                uint8_t hi;
                if (hr == '\\') { int e = bump(); if (e < 0) { err = "bad escape in range"; return false; } hi = unesc(e); }
                else hi = (uint8_t)hr;
                if (hi < lo) { err = "character range is descending"; return false; }
                for (int v = lo; v <= hi; v++) set[v] = 1;
            }
        }
        if (neg) for (auto& v : set) v = !v;
        *out = set_frag(set);
        return true;
    }
    bool atom(Frag* out) {
        for (;;) {
            int c = peek();
            if (c < 0) { err = "unexpected end of pattern"; return false; }
            if (c == '(') {
                pos++;
                if (!alt(out)) return false;
                if (bump() == ')') return true;
                err = "unclosed group";
                return false;
            }
            if (c == '[') { pos++; return cls(out); }
            if (c == '.') { pos++; *out = set_frag(ByteSet(256, 1)); return true; }
            if (c == '^' || c == '$') { pos++; continue; }   // anchors are skipped, the next atom takes their place
            ByteSet one(256, 0);
            if (c == '\\') {
                pos++;
                int e = bump();
                if (e < 0) { err = "dangling escape"; return false; }
                one[unesc(e)] = 1;
            } else { pos++; one[c] = 1; }
            *out = set_frag(one);
            return true;
        }
    }
    bool repeat(Frag* out) {
        Frag f;
        if (!atom(&f)) return false;
        for (;;) {
            int c = peek();
            if (c == '*') { pos++; f = wrap(f, nullptr, true, true); }
            else if (c == '+') { pos++; f = wrap(f, nullptr, false, true); }
            else if (c == '?') { pos++; f = wrap(f, nullptr, true, false); }
            else if (c == '{') {
                pos++;
                unsigned long long lo = 0, hi = 0;
                int why = 0;
                if (!count(&lo, &why)) { err = why == 1 ? "missing repetition count" : "bad repetition count"; return false; }
                if (peek() == ',') {
                    pos++;
                    if (!count(&hi, &why)) { err = why == 1 ? "missing max repetition count" : "bad max repetition count"; return false; }
                } else hi = lo;
                if (peek() != '}') { err = "unclosed repetition"; return false; }
                pos++;
                if (hi < lo) { err = "descending repetition bounds"; return false; }
                if (lo > 100000) { err = "repetition count too large to tabulate"; return false; }
                Frag acc = f;   // exactly `lo` copies (the upper bound is parsed but not expanded)
                for (unsigned long long i = 1; i < lo; i++) acc = concat(acc, copy(f));
                f = acc;
            } else break;
        }
        *out = f;
        return true;
    }
    bool seq(Frag* out) {
        Frag l;
        if (!repeat(&l)) return false;
        for (;;) {
            int c = peek();
            if (c < 0 || c == ')' || c == '|') break;
            Frag r;
            if (!repeat(&r)) return false;
            l = concat(l, r);
        }
        *out = l;
        return true;
    }
    bool alt(Frag* out) {
        Frag l;
        if (!seq(&l)) return false;
        while (peek() == '|') {
            pos++;
            Frag r;
            if (!seq(&r)) return false;
            l = wrap(l, &r, false, false);
        }
        *out = l;
        return true;
    }
};

// ------------------------------------------------------------------------------- table states
struct MaskState {
    ByteSet allowed;          // 256 flags
    bool complete = false, dead = false;
    std::vector<uint32_t> next;   // regex only: DFA transition per byte (0 = dead)
};

enum JsonFrame : uint8_t { J_VALUE, J_OBJECT, J_COLON, J_AFTER_MEMBER, J_ARRAY, J_ARRAY_COMMA };
enum JsonMode : uint8_t { M_FRAME, M_STRING, M_ESCAPE, M_HEX, M_NUM_SIGN, M_NUMBER, M_LITERAL, M_DEAD };
enum NumPhase : uint8_t { N_ZERO, N_INT, N_FRAC_DOT, N_FRAC_DIGITS, N_EXP_E, N_EXP_SIGN, N_EXP_DIGITS };

// JSON mask classes (table states)
enum JsonClass : uint32_t {
    C_DEAD = 0, C_COMPLETE, C_VALUE, C_OBJECT, C_COLON, C_AFTER_MEMBER, C_ARRAY, C_ARRAY_COMMA, C_STRING, C_ESCAPE,
    C_HEX, C_DIGITS, C_EXP_E, C_LIT_R, C_LIT_U, C_LIT_E, C_LIT_A, C_LIT_L, C_LIT_S, C_COUNT
};

void set_bytes(ByteSet& m, const char* s) { for (; *s; s++) m[(uint8_t)*s] = 1; }

}  // namespace

struct pgs_grammar {
    bool is_json = false;
    std::vector<MaskState> states;   // states[0] is dead
    uint32_t start = 0;
};

// Host-side per-row state.  Regex: `dfa` only.  JSON: the scanner's pushdown state.
struct pgs_gstate {
    uint32_t dfa = 0;
    std::vector<uint8_t> stack;
    uint8_t mode = M_FRAME, phase = 0, hex_left = 0, lit_pos = 0;
    const char* lit = nullptr;
};

namespace {

bool is_ws(uint8_t c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r'; }
bool is_digit(uint8_t c) { return c >= '0' && c <= '9'; }
bool is_hex(uint8_t c) { return is_digit(c) || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F'); }

void json_finish_value(std::vector<uint8_t>& st) {
    st.pop_back();
    if (!st.empty()) {
        if (st.back() == J_OBJECT) st.back() = J_AFTER_MEMBER;
        else if (st.back() == J_ARRAY) st.back() = J_ARRAY_COMMA;
    }
}

// a string just closed: a key (top frame is Object) is followed by a colon, anything else was a value
void json_string_closed(pgs_gstate& s) {
    if (!s.stack.empty() && s.stack.back() == J_OBJECT) s.stack.push_back(J_COLON);
    else json_finish_value(s.stack);
    s.mode = M_FRAME;
}

void json_frame_byte(pgs_gstate& s, uint8_t c);

// one byte while inside a number; a byte that cannot continue it ends the value and is re-read
void json_number_byte(pgs_gstate& s, uint8_t c) {
    auto done = [&]() { json_finish_value(s.stack); s.mode = M_FRAME; json_frame_byte(s, c); };
    switch (s.phase) {
    case N_ZERO:
        if (c == '.') s.phase = N_FRAC_DOT; else if (c == 'e' || c == 'E') s.phase = N_EXP_E; else done();
        break;
    case N_INT:
        if (is_digit(c)) {} else if (c == '.') s.phase = N_FRAC_DOT; else if (c == 'e' || c == 'E') s.phase = N_EXP_E;
        else done();
        break;
    case N_FRAC_DOT: if (is_digit(c)) s.phase = N_FRAC_DIGITS; else s.mode = M_DEAD; break;
    case N_FRAC_DIGITS:
        if (is_digit(c)) {} else if (c == 'e' || c == 'E') s.phase = N_EXP_E; else done();
        break;
    case N_EXP_E:
        if (c == '+' || c == '-') s.phase = N_EXP_SIGN; else if (is_digit(c)) s.phase = N_EXP_DIGITS; else s.mode = M_DEAD;
        break;
    case N_EXP_SIGN: if (is_digit(c)) s.phase = N_EXP_DIGITS; else s.mode = M_DEAD; break;
    default: if (!is_digit(c)) done();
    }
}

void json_frame_byte(pgs_gstate& s, uint8_t c) {
    for (;;) {
        if (is_ws(c)) return;                       // whitespace is skipped before every token
        if (s.stack.empty()) { s.mode = M_DEAD; return; }   // content after a complete value
        switch (s.stack.back()) {
        case J_VALUE:
            if (c == '{') s.stack.push_back(J_OBJECT);
            else if (c == '[') s.stack.push_back(J_ARRAY);
            else if (c == '"') s.mode = M_STRING;
            else if (c == '-') s.mode = M_NUM_SIGN;
            else if (c == '0') { s.mode = M_NUMBER; s.phase = N_ZERO; }
            else if (is_digit(c)) { s.mode = M_NUMBER; s.phase = N_INT; }
            else if (c == 't') { s.mode = M_LITERAL; s.lit = "true"; s.lit_pos = 1; }
            else if (c == 'f') { s.mode = M_LITERAL; s.lit = "false"; s.lit_pos = 1; }
            else if (c == 'n') { s.mode = M_LITERAL; s.lit = "null"; s.lit_pos = 1; }
            else s.mode = M_DEAD;
            return;
        case J_OBJECT:
            if (c == '"') s.mode = M_STRING;
            else if (c == '}') { s.stack.pop_back(); json_finish_value(s.stack); }
            else s.mode = M_DEAD;
            return;
        case J_COLON:
            if (c == ':') s.stack.back() = J_VALUE; else s.mode = M_DEAD;
            return;
        case J_AFTER_MEMBER:
            if (c == ',') s.stack.back() = J_OBJECT;
            else if (c == '}') { s.stack.pop_back(); json_finish_value(s.stack); }
            else s.mode = M_DEAD;
            return;
        case J_ARRAY:
            if (c == ']') { s.stack.pop_back(); json_finish_value(s.stack); return; }
            s.stack.push_back(J_VALUE);   // an element starts here: read the same byte as a value
            continue;
        default:   // J_ARRAY_COMMA
            if (c == ',') s.stack.back() = J_ARRAY;
            else if (c == ']') { s.stack.pop_back(); json_finish_value(s.stack); }
            else s.mode = M_DEAD;
            return;
        }
    }
}

void json_advance(pgs_gstate& s, uint8_t c) {
    switch (s.mode) {
    case M_DEAD: return;
    case M_FRAME: json_frame_byte(s, c); return;
    case M_STRING:
        if (c == '"') json_string_closed(s);
        else if (c == '\\') s.mode = M_ESCAPE;
        else if (c < 0x20) s.mode = M_DEAD;
        return;
    case M_ESCAPE:
        if (c == 'u') { s.mode = M_HEX; s.hex_left = 4; }
        else if (c != 0 && strchr("\"\\/bfnrt", c)) s.mode = M_STRING;
        else s.mode = M_DEAD;
        return;
    case M_HEX:
        if (!is_hex(c)) { s.mode = M_DEAD; return; }
        if (--s.hex_left == 0) s.mode = M_STRING;
        return;
    case M_NUM_SIGN:
        if (c == '0') { s.mode = M_NUMBER; s.phase = N_ZERO; }
        else if (c >= '1' && c <= '9') { s.mode = M_NUMBER; s.phase = N_INT; }
        else s.mode = M_DEAD;
        return;
    case M_NUMBER: json_number_byte(s, c); return;
    default:   // M_LITERAL
        if ((uint8_t)s.lit[s.lit_pos] != c) { s.mode = M_DEAD; return; }
        if (s.lit[++s.lit_pos] == 0) { json_finish_value(s.stack); s.mode = M_FRAME; }
    }
}

uint32_t frame_class(const std::vector<uint8_t>& st) {
    if (st.empty()) return C_COMPLETE;
    switch (st.back()) {
    case J_VALUE: return C_VALUE;
    case J_OBJECT: return C_OBJECT;
    case J_COLON: return C_COLON;
    case J_AFTER_MEMBER: return C_AFTER_MEMBER;
    case J_ARRAY: return C_ARRAY;
    default: return C_ARRAY_COMMA;
    }
}

// the class of the mask the scanner would return if the input ended in this state
uint32_t json_class(const pgs_gstate& s) {
    switch (s.mode) {
    case M_DEAD: return C_DEAD;
    case M_FRAME: return frame_class(s.stack);
    case M_STRING: return C_STRING;
    case M_ESCAPE: return C_ESCAPE;
    case M_HEX: return C_HEX;
    case M_NUM_SIGN: return C_DIGITS;
    case M_NUMBER:
        if (s.phase == N_FRAC_DOT || s.phase == N_EXP_SIGN) return C_DIGITS;
        if (s.phase == N_EXP_E) return C_EXP_E;
        {   // a number that ends the input in any other phase counts as finished
            std::vector<uint8_t> st = s.stack;
            json_finish_value(st);
            return frame_class(st);
        }
    default:
        switch (s.lit[s.lit_pos]) {
        case 'r': return C_LIT_R;
        case 'u': return C_LIT_U;
        case 'e': return C_LIT_E;
        case 'a': return C_LIT_A;
        case 'l': return C_LIT_L;
        default: return C_LIT_S;
        }
    }
}

void json_build(pgs_grammar& g) {
    g.is_json = true;
    g.states.assign(C_COUNT, MaskState());
    for (auto& s : g.states) s.allowed.assign(256, 0);
    g.states[C_DEAD].dead = true;
    g.states[C_COMPLETE].complete = true;
    const char* value_starts = "{\"tf n0123456789[-";
    const char* ws = " \t\n\r";
    auto frame = [&](uint32_t c, const char* a, const char* b) { set_bytes(g.states[c].allowed, a); set_bytes(g.states[c].allowed, b); set_bytes(g.states[c].allowed, ws); };
    frame(C_VALUE, value_starts, "");
    frame(C_OBJECT, "\"}", "");
    frame(C_COLON, ":", "");
    frame(C_AFTER_MEMBER, ",}", "");
    frame(C_ARRAY, value_starts, "]");
    frame(C_ARRAY_COMMA, ",]", "");
    for (int c = 0x20; c < 256; c++) g.states[C_STRING].allowed[c] = 1;
    set_bytes(g.states[C_ESCAPE].allowed, "\"\\/bfnrtu");
    set_bytes(g.states[C_HEX].allowed, "0123456789abcdefABCDEF");
    set_bytes(g.states[C_DIGITS].allowed, "0123456789");
    set_bytes(g.states[C_EXP_E].allowed, "0123456789+-");
    const char letters[] = "rueals";
    for (int i = 0; i < 6; i++) g.states[C_LIT_R + i].allowed[(uint8_t)letters[i]] = 1;
}

// subset construction; returns false when the DFA would exceed `limit` states
bool regex_build(pgs_grammar& g, const Nfa& nfa, uint32_t limit, std::string& err) {
    const uint32_t N = (uint32_t)nfa.st.size();
    // which NFA states can still reach an accepting one
    std::vector<uint8_t> reach(nfa.accept);
    for (bool changed = true; changed;) {
        changed = false;
        for (uint32_t s = 0; s < N; s++)
            if (!reach[s])
                for (const Edge& e : nfa.st[s])
                    if (reach[e.to]) { reach[s] = 1; changed = true; break; }
    }
    auto closure = [&](std::vector<uint32_t> seeds) {
        std::vector<uint8_t> seen(N, 0);
        std::vector<uint32_t> out;
        while (!seeds.empty()) {
            uint32_t s = seeds.back();
            seeds.pop_back();
            if (seen[s]) continue;
            seen[s] = 1;
            out.push_back(s);
            for (const Edge& e : nfa.st[s]) if (e.c < 0) seeds.push_back(e.to);
        }
        std::vector<uint32_t> sorted;
        for (uint32_t s = 0; s < N; s++) if (seen[s]) sorted.push_back(s);
        return sorted;
    };
    auto live = [&](const std::vector<uint32_t>& set) { for (uint32_t s : set) if (reach[s]) return true; return false; };
    std::map<std::vector<uint32_t>, uint32_t> ids;
    std::vector<std::vector<uint32_t>> sets;
    g.states.clear();
    g.states.emplace_back();   // 0 = dead
    g.states[0].dead = true;
    g.states[0].allowed.assign(256, 0);
    g.states[0].next.assign(256, 0);
    sets.emplace_back();
    auto intern = [&](const std::vector<uint32_t>& set) -> uint32_t {
        if (set.empty() || !live(set)) return 0;
        auto it = ids.find(set);
        if (it != ids.end()) return it->second;
        uint32_t id = (uint32_t)g.states.size();
        ids[set] = id;
        g.states.emplace_back();
        sets.push_back(set);
        return id;
    };
    g.start = intern(closure({nfa.start}));
    for (uint32_t cur = 1; cur < g.states.size(); cur++) {
        if (g.states.size() > limit) { err = "regex needs too many DFA states"; return false; }
        const std::vector<uint32_t> set = sets[cur];
        MaskState ms;
        ms.allowed.assign(256, 0);
        ms.next.assign(256, 0);
        for (uint32_t s : set) ms.complete |= nfa.accept[s] != 0;
        std::vector<std::vector<uint32_t>> by_byte(256);
        for (uint32_t s : set)
            for (const Edge& e : nfa.st[s]) if (e.c >= 0) by_byte[e.c].push_back(e.to);
        for (int b = 0; b < 256; b++) {
            if (by_byte[b].empty()) continue;
            const uint32_t nx = intern(closure(by_byte[b]));
            ms.next[b] = nx;
            ms.allowed[b] = nx != 0;
        }
        g.states[cur] = ms;
    }
    return true;
}

}  // namespace

// ------------------------------------------------------------------------------------ C ABI

extern "C" int pgs_grammar_regex(const char* pattern, pgs_grammar** out, char* err, size_t err_len) {
    if (!pattern || !out) return PGS_ERR_INVALID;
    *out = nullptr;
    Nfa nfa;
    std::string pat(pattern);
    RegexParser ps(pat, nfa);
    Frag f;
    std::string msg;
    bool ok = ps.alt(&f);
    if (!ok) msg = ps.err;
    else if (ps.pos != pat.size()) {
        char buf[96];
        snprintf(buf, sizeof buf, "unexpected byte '%c' at position %zu", pat[ps.pos], ps.pos);
        msg = buf;
        ok = false;
    }
    pgs_grammar* g = nullptr;
    if (ok) {
        nfa.accept[f.e] = 1;
        nfa.start = f.s;
        g = new pgs_grammar();
        if (!regex_build(*g, nfa, 1u << 16, msg)) { delete g; g = nullptr; ok = false; }
    }
    if (!ok) {
        if (err && err_len) snprintf(err, err_len, "%s", msg.c_str());
        return PGS_ERR_INVALID;
    }
    *out = g;
    return PGS_OK;
}

extern "C" int pgs_grammar_json(pgs_grammar** out) {
    if (!out) return PGS_ERR_INVALID;
    pgs_grammar* g = new pgs_grammar();
    json_build(*g);
    g->start = C_VALUE;
    *out = g;
    return PGS_OK;
}

extern "C" void pgs_grammar_free(pgs_grammar* g) { delete g; }
extern "C" uint32_t pgs_grammar_n_states(const pgs_grammar* g) { return g ? (uint32_t)g->states.size() : 0; }

extern "C" int pgs_grammar_state_new(const pgs_grammar* g, pgs_gstate** out) {
    if (!g || !out) return PGS_ERR_INVALID;
    pgs_gstate* s = new pgs_gstate();
    s->dfa = g->start;
    if (g->is_json) s->stack.push_back(J_VALUE);
    *out = s;
    return PGS_OK;
}
extern "C" void pgs_grammar_state_free(pgs_gstate* s) { delete s; }

extern "C" int pgs_grammar_state_reset(const pgs_grammar* g, pgs_gstate* s) {
    if (!g || !s) return PGS_ERR_INVALID;
    *s = pgs_gstate();
    s->dfa = g->start;
    if (g->is_json) s->stack.push_back(J_VALUE);
    return PGS_OK;
}

extern "C" int pgs_grammar_advance(const pgs_grammar* g, pgs_gstate* s, const uint8_t* bytes, size_t n) {
    if (!g || !s || (!bytes && n)) return PGS_ERR_INVALID;
    for (size_t i = 0; i < n; i++) {
        if (g->is_json) json_advance(*s, bytes[i]);
        else s->dfa = g->states[s->dfa].next[bytes[i]];
    }
    return PGS_OK;
}

extern "C" uint32_t pgs_grammar_mask_state(const pgs_grammar* g, const pgs_gstate* s) {
    if (!g || !s) return 0;
    return g->is_json ? json_class(*s) : s->dfa;
}

extern "C" int pgs_grammar_state_info(const pgs_grammar* g, uint32_t state, uint8_t* allowed256, int* complete,
                                      int* dead) {
    if (!g || state >= g->states.size()) return PGS_ERR_INVALID;
    const MaskState& m = g->states[state];
    if (allowed256) memcpy(allowed256, m.allowed.data(), 256);
    if (complete) *complete = m.complete;
    if (dead) *dead = m.dead;
    return PGS_OK;
}

extern "C" int pgs_grammar_build_table(const pgs_grammar* g, uint32_t vocab, uint32_t first_byte_id,
                                       uint32_t* words_out, uint8_t* flags_out) {
    if (!g || !words_out || !flags_out || vocab == 0) return PGS_ERR_INVALID;
    const size_t wps = (vocab + 31) / 32;
    memset(words_out, 0, g->states.size() * wps * sizeof(uint32_t));
    for (size_t s = 0; s < g->states.size(); s++) {
        const MaskState& m = g->states[s];
        for (uint32_t b = 0; b < 256; b++) {
            const uint64_t tok = (uint64_t)first_byte_id + b;
            if (m.allowed[b] && tok < vocab) words_out[s * wps + (tok >> 5)] |= 1u << (tok & 31);
        }
        flags_out[s] = (uint8_t)((m.complete ? 1 : 0) | (m.dead ? 2 : 0));
    }
    return PGS_OK;
}
