// The reference's own unit tests for the logits -> token path, written against the C++ mirror of
// its API (include/pagoda_sampler.hpp) and run on the GPU.  Each test names the Rust test it
// transcribes (paths inside the reference project).
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>

#include "pagoda_sampler.hpp"

using namespace pagoda;

static int failures = 0;
#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) { printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); failures++; } \
    } while (0)

static void greedy_is_argmax() {   // pagoda/src/sampler.rs:157-162
    Sampler s(0);
    CHECK(s.sample({0.1f, 5.0f, 2.0f}, SamplingParams{}) == 1);
}

static void sampler_is_reproducible() {   // sampler.rs:165-176
    std::vector<float> logits(100, 1.0f);
    SamplingParams p;
    p.temperature = 1.0f;
    Sampler a(99), b(99);
    std::vector<TokenId> sa, sb;
    for (int i = 0; i < 20; i++) { sa.push_back(a.sample(logits, p)); sb.push_back(b.sample(logits, p)); }
    CHECK(sa == sb);
}

static void top_k_mass_is_some() {   // sampler.rs:179-189
    SamplingParams p;
    p.temperature = 1.0f; p.top_k = 3;
    Sampler s(1);
    TokenId t = s.sample({0.0f, 10.0f, 9.0f, 8.0f, 1.0f}, p);
    CHECK(t == 1 || t == 2 || t == 3);
}

static void top_p_keeps_only_the_nucleus() {   // sampler.rs:192-207
    SamplingParams p;
    p.temperature = 1.0f; p.top_p = 0.75f;
    Sampler s(123);
    for (int i = 0; i < 200; i++) { TokenId t = s.sample({1.0f, 0.0f, -1.0f}, p); CHECK(t == 0 || t == 1); }
}

static void penalties() {   // pagoda/src/engine.rs:1781-1809, observed through the greedy choice
    Sampler s(0);
    std::vector<float> logits(8, 0.0f);
    logits[3] = 5.0f; logits[7] = 4.5f;
    SamplingParams p;
    p.frequency_penalty = 1.0f;   // token 3 seen twice: 5 -> 3, below token 7's 4.5 - 1
    std::vector<TokenId> out = {3, 7, 3};
    auto r = s.advance_batch({&logits}, {&p}, {&out}, {""}, 8, -1);
    CHECK(r[0].token == 7 && r[0].status == RowStatus::Ok);
    SamplingParams q;
    q.presence_penalty = 1.0f;    // once per token: 5 -> 4, 4.5 -> 3.5
    std::vector<TokenId> out2 = {3, 3, 7};
    r = s.advance_batch({&logits}, {&q}, {&out2}, {""}, 8, -1);
    CHECK(r[0].token == 3);
}

static void regex_grammar() {   // pagoda/src/grammar.rs:1024-1054
    Grammar g = Grammar::regex("(ab)+c");
    CHECK(g.is_complete("abc") && g.is_complete("ababc") && !g.is_complete("ab") && !g.is_complete("abcd"));
    Grammar d = Grammar::regex("[a-z][0-9]{2}");
    CHECK(d.is_complete("x42") && !d.is_complete("x4") && !d.is_complete("X42"));
    Grammar c = Grammar::regex("[abc]+");
    auto allowed = c.allowed_bytes("cb");
    CHECK(allowed && *allowed == std::vector<uint8_t>({'a', 'b', 'c'}));
    CHECK(!c.allowed_bytes("z"));
    for (const char* bad : {"(", "[a", "a|"}) {
        bool threw = false;
        try { Grammar::regex(bad); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw);
    }
}

static void json_grammar() {   // grammar.rs:1057-1085
    Grammar j = Grammar::json();
    for (const char* t : {"null", "true", "false", "42", "-3.5e2", "\"hi\"", "{}", "[]", "{\"a\":1,\"b\":[true,null]}"})
        CHECK(j.is_complete(t));
    CHECK(!j.is_complete("") && !j.is_complete("{"));
    auto a = j.allowed_bytes("");
    CHECK(a && std::string(a->begin(), a->end()).find('{') != std::string::npos);
    CHECK(!j.allowed_bytes("{\"a\":1}  ]"));
}

static void grammar_walk_and_fault_isolation() {   // pagoda/tests/grammar_tests.rs:9-49, fault_tests.rs:63-82
    Sampler s(0);
    Grammar g = Grammar::regex("\"[a-z]{3}\"");
    SamplingParams p;
    p.grammar = g;
    std::vector<float> logits(259);
    for (int i = 0; i < 259; i++) logits[i] = std::sin(0.37f * i);
    std::vector<float> nan_row(259, NAN);
    SamplingParams plain;
    std::string text;
    std::vector<TokenId> out;
    for (int step = 0; step < 8; step++) {
        auto r = s.advance_batch({&logits, &nan_row}, {&p, &plain}, {&out, nullptr}, {text, ""}, 259, 2);
        CHECK(r[1].status == RowStatus::Fault);           // the NaN row faults alone, every step
        if (r[0].status == RowStatus::Stop || r[0].token == 2) break;
        CHECK(r[0].status == RowStatus::Ok);
        out.push_back(r[0].token);
        text.push_back((char)(r[0].token - 3));
    }
    CHECK(g.is_complete(text));
    CHECK(text.size() == 5 && text.front() == '"' && text.back() == '"');
}

// The draw-order rule of the serial loop (pagoda/src/engine.rs:511-544, sampler.rs:43-46): one next_f32() per row that
// really samples, in `pending` order; a faulted row and a grammar dead end take nothing from the stream.  The batch
// below has both in the middle.  Its tokens must equal those of the same rows advanced one by one (a single-row batch
// is trivially in order), and the line printed at the end is compared with the CPU oracle's Sampler stream by the
// Python side of this test.
static void draw_order_matches_the_serial_loop() {
    const uint32_t vocab = 64;
    std::vector<std::vector<float>> rows(6, std::vector<float>(vocab));
    for (int r = 0; r < 6; r++)
        for (uint32_t i = 0; i < vocab; i++) rows[r][i] = (float)((i * 37u + (uint32_t)r * 11u) % 17u) * 0.25f;
    rows[1][5] = NAN;                         // row 1 faults
    Grammar g = Grammar::regex("abc");
    SamplingParams p;
    p.temperature = 0.8f; p.top_k = 10; p.top_p = 0.9f;
    SamplingParams dead = p;
    dead.grammar = g;                          // row 3: the partial output "z" is a dead end
    std::vector<const std::vector<float>*> lp;
    for (auto& r : rows) lp.push_back(&r);
    std::vector<const SamplingParams*> pp = {&p, &p, &p, &dead, &p, &p};
    std::vector<const std::vector<TokenId>*> outs(6, nullptr);
    std::vector<std::string> partials = {"", "", "", "z", "", ""};
    Sampler batched(1234), serial(1234);
    auto b = batched.advance_batch(lp, pp, outs, partials, vocab, -1);
    CHECK(b[1].status == RowStatus::Fault && b[3].status == RowStatus::Stop);
    printf("DRAW_ORDER");
    for (int r = 0; r < 6; r++) {
        auto one = serial.advance_batch({lp[r]}, {pp[r]}, {nullptr}, {partials[r]}, vocab, -1);
        CHECK(one[0].token == b[r].token && one[0].status == b[r].status);
        printf(" %u:%d", b[r].token, (int)b[r].status);
    }
    // both generators stand where the reference's would: the next sample agrees too
    const TokenId nb = batched.sample(rows[0], p), ns = serial.sample(rows[0], p);
    CHECK(nb == ns);
    printf(" next %u\n", nb);
}

int main() {
    greedy_is_argmax();
    sampler_is_reproducible();
    top_k_mass_is_some();
    top_p_keeps_only_the_nucleus();
    penalties();
    regex_grammar();
    json_grammar();
    grammar_walk_and_fault_isolation();
    draw_order_matches_the_serial_loop();
    printf("%s (%d failures)\n", failures ? "FAILED" : "CPP_OK", failures);
    return failures != 0;
}
