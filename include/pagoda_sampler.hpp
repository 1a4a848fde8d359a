// C++ mirror of the reference's Rust surface for the logits -> token path, on top of the C ABI
// (pagoda_sampler.h).  Same names, argument meaning and error behaviour as the reference:
//   pagoda::Rng              pagoda/src/rng.rs:7-31 (host side, supplies the per-row uniform)
//   pagoda::SamplingParams   pagoda/src/spec.rs:65-105 (defaults included)
//   pagoda::Sampler          pagoda/src/sampler.rs:11-37 (new / seed / sample)
//   pagoda::argmax           pagoda/src/sampler.rs:59-70
//   pagoda::Grammar          pagoda/src/grammar.rs:25-66 (regex / json / allowed_bytes / is_complete)
//   pagoda::apply_penalties + Engine::advance_with_logits are folded into Sampler::advance_batch,
//   the batched form of the loop at pagoda/src/engine.rs:511-544.
// Everything numeric runs on the GPU; there is no host fallback.  Header only.
#pragma once

#include <cstdint>
#include <limits>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "pagoda_sampler.h"

namespace pagoda {

using TokenId = uint32_t;

struct Rng {   // SplitMix64, rng.rs:10-30
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed + 0x9e3779b97f4a7c15ULL) {}
    uint64_t next_u64() {
        s += 0x9e3779b97f4a7c15ULL;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
        return z ^ (z >> 31);
    }
    double next_f64() { return (double)(next_u64() >> 11) * (1.0 / (double)(1ULL << 53)); }
    float next_f32() { return (float)next_f64(); }
    void unread() { s -= 0x9e3779b97f4a7c15ULL; }   // give back a draw the chain did not consume
};

class Grammar {   // grammar.rs:25-66; tabulated once, queried per prefix
  public:
    static Grammar regex(const std::string& pattern) {   // Err(String) -> std::invalid_argument
        pgs_grammar* g = nullptr;
        char err[256] = "";
        if (pgs_grammar_regex(pattern.c_str(), &g, err, sizeof err) != PGS_OK) throw std::invalid_argument(err);
        return Grammar(g, "regex");
    }
    static Grammar json() {
        pgs_grammar* g = nullptr;
        pgs_grammar_json(&g);
        return Grammar(g, "json");
    }
    const char* name() const { return name_; }
    // Bytes that may legally follow `partial`; nullopt when the string is already dead.
    std::optional<std::vector<uint8_t>> allowed_bytes(const std::string& partial) const {
        uint8_t flags[256];
        int complete = 0, dead = 0;
        pgs_grammar_state_info(g_.get(), state_of(partial), flags, &complete, &dead);
        if (dead) return std::nullopt;
        std::vector<uint8_t> out;
        for (int b = 0; b < 256; b++) if (flags[b]) out.push_back((uint8_t)b);
        return out;
    }
    bool is_complete(const std::string& partial) const {
        int complete = 0, dead = 0;
        pgs_grammar_state_info(g_.get(), state_of(partial), nullptr, &complete, &dead);
        return complete != 0;
    }
    uint32_t state_of(const std::string& partial) const {
        pgs_gstate* s = nullptr;
        pgs_grammar_state_new(g_.get(), &s);
        pgs_grammar_advance(g_.get(), s, (const uint8_t*)partial.data(), partial.size());
        const uint32_t st = pgs_grammar_mask_state(g_.get(), s);
        pgs_grammar_state_free(s);
        return st;
    }
    const pgs_grammar* raw() const { return g_.get(); }

  private:
    Grammar(pgs_grammar* g, const char* n) : g_(g, pgs_grammar_free), name_(n) {}
    std::shared_ptr<pgs_grammar> g_;
    const char* name_;
};

struct SamplingParams {   // spec.rs:65-105
    size_t max_tokens = 128;
    float temperature = 0.0f;
    float top_p = 1.0f;
    size_t top_k = std::numeric_limits<size_t>::max();   // 0 / max disables
    float frequency_penalty = 0.0f;
    float presence_penalty = 0.0f;
    float repetition_penalty = 1.0f;                     // extension
    uint64_t seed = 42;
    std::optional<Grammar> grammar;
};

enum class RowStatus { Ok = 0, Fault = 1, Stop = 2, Empty = 3, BadParam = 4 };   // FinishReason of the row

struct Advance { TokenId token; RowStatus status; };

class Sampler {   // sampler.rs:11-37, bound to one device
  public:
    explicit Sampler(uint64_t seed, int device = 0, uint32_t max_rows = 256, uint32_t max_vocab = 262144,
                     uint32_t max_history = 4096)
        : rng_(seed) {
        if (pgs_create(device, max_rows, max_vocab, max_history, &h_) != PGS_OK)
            throw std::runtime_error(pgs_last_error(nullptr));
    }
    ~Sampler() { pgs_destroy(h_); }
    Sampler(const Sampler&) = delete;
    Sampler& operator=(const Sampler&) = delete;

    void seed(uint64_t seed) { rng_ = Rng(seed); }                       // sampler.rs:21-23
    void set_exact(bool on) { pgs_set_exact(h_, on ? 1 : 0); }

    // Sampler::sample (sampler.rs:28-37): one row, no penalties, no grammar.
    TokenId sample(const std::vector<float>& logits, const SamplingParams& p) {
        std::vector<Advance> r = advance_batch({&logits}, {&p}, {nullptr}, {""}, 259, -1);
        return r[0].token;
    }

    // The batched form of Engine::advance_with_logits (engine.rs:1286-1314) for the pending sequences of
    // one step, in `pending` order: sanity, penalties over `outputs[i]` (the generated ids), grammar mask
    // for the decoded output `partials[i]`, EOS fix, sample.  The rows see the generator's stream exactly as the
    // reference's serial loop would hand it out.
    std::vector<Advance> advance_batch(const std::vector<const std::vector<float>*>& logits,
                                       const std::vector<const SamplingParams*>& params,
                                       const std::vector<const std::vector<TokenId>*>& outputs,
                                       const std::vector<std::string>& partials, uint32_t vocab, int32_t eos) {
        const uint32_t rows = (uint32_t)logits.size();
        if (rows && logits[0]) vocab = (uint32_t)logits[0]->size();
        std::vector<float> x((size_t)rows * vocab), temp(rows), top_p(rows), freq(rows), pres(rows), rep(rows), uni(rows, 0.0f);
        std::vector<uint32_t> top_k(rows), ho(rows + 1, 0), hi, token(rows);
        std::vector<int32_t> mtab(rows, -1), mst(rows, 0), status(rows);
        std::vector<uint8_t> drew(rows);
        std::vector<int32_t> uploaded;
        for (uint32_t r = 0; r < rows; r++) {
            if (logits[r]->size() != vocab) throw std::invalid_argument("rows of one batch share one vocabulary");
            std::copy(logits[r]->begin(), logits[r]->end(), x.begin() + (size_t)r * vocab);
            const SamplingParams& p = *params[r];
            temp[r] = p.temperature; top_p[r] = p.top_p;
            top_k[r] = p.top_k >= vocab ? 0u : (uint32_t)p.top_k;
            freq[r] = p.frequency_penalty; pres[r] = p.presence_penalty; rep[r] = p.repetition_penalty;
            if (outputs[r]) hi.insert(hi.end(), outputs[r]->begin(), outputs[r]->end());
            ho[r + 1] = (uint32_t)hi.size();
            if (p.grammar) {
                const pgs_grammar* g = p.grammar->raw();
                const uint32_t ns = pgs_grammar_n_states(g), wps = (vocab + 31) / 32;
                std::vector<uint32_t> words((size_t)ns * wps);
                std::vector<uint8_t> flags(ns);
                pgs_grammar_build_table(g, vocab, 3, words.data(), flags.data());
                int32_t id = -1;
                if (pgs_mask_table_upload(h_, ns, wps, words.data(), flags.data(), &id) != PGS_OK)
                    throw std::runtime_error(pgs_last_error(h_));
                uploaded.push_back(id);
                mtab[r] = id;
                mst[r] = (int32_t)p.grammar->state_of(partials[r]);
            }
        }
        // One draw per stochastic row, in `pending` order (sampler.rs:43-46); greedy rows draw nothing.  A stochastic
        // row that ends without sampling (faulted, grammar dead end, nothing finite left) consumes no draw in the
        // reference (engine.rs:1292-1303, sampler.rs:43-46), so the rows behind it must see the stream one draw
        // earlier: the generator is put back to where it stood before that row's draw and the rows behind it are run
        // again with fresh draws.  Such rows are rare, and every pass makes at least one more row final.
        pgs_batch_desc d{};
        d.struct_size = sizeof d; d.vocab = vocab; d.logits_dtype = PGS_F32; d.row_stride = vocab;
        d.logits_mem = PGS_MEM_HOST; d.aux_mem = PGS_MEM_HOST; d.eos_token_id = eos;
        std::vector<Rng> before(rows, rng_);
        uint32_t start = 0;
        int rc = PGS_OK;
        while (start < rows) {
            for (uint32_t r = start; r < rows; r++) {
                before[r] = rng_;
                uni[r] = (temp[r] < 1e-5f) ? 0.0f : rng_.next_f32();
            }
            d.rows = rows - start;
            d.logits = x.data() + (size_t)start * vocab;
            d.temperature = temp.data() + start; d.top_k = top_k.data() + start; d.top_p = top_p.data() + start;
            d.frequency_penalty = freq.data() + start; d.presence_penalty = pres.data() + start;
            d.repetition_penalty = rep.data() + start;
            d.hist_offsets = ho.data() + start;   // offsets stay absolute
            d.hist_ids = hi.empty() ? ho.data() : hi.data();
            d.mask_table = mtab.data() + start; d.mask_state = mst.data() + start; d.uniform = uni.data() + start;
            d.token = token.data() + start; d.status = status.data() + start; d.drew = drew.data() + start;
            rc = pgs_sample_batch(h_, &d);
            if (rc != PGS_OK) break;
            uint32_t stop = rows;
            for (uint32_t r = start; r < rows; r++)
                if (!(temp[r] < 1e-5f) && !drew[r]) { stop = r; break; }
            if (stop == rows) break;
            rng_ = before[stop];   // row `stop` keeps its result; it used nothing of the stream
            start = stop + 1;
        }
        for (int32_t id : uploaded) pgs_mask_table_free(h_, id);
        if (rc != PGS_OK) throw std::runtime_error(pgs_last_error(h_));
        std::vector<Advance> out(rows);
        for (uint32_t r = 0; r < rows; r++) out[r] = {token[r], (RowStatus)status[r]};
        return out;
    }

  private:
    Rng rng_;
    pgs_handle* h_ = nullptr;
};

// sampler.rs:59-70 through the device: greedy decoding of one row
inline TokenId argmax(Sampler& s, const std::vector<float>& xs) { return s.sample(xs, SamplingParams{}); }

}  // namespace pagoda
