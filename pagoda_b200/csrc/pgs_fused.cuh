// Definitions shared by the fused cluster kernel, the finish kernel and the host launcher.
#pragma once

#include <stdint.h>

namespace pgs {

constexpr int F_MAXC = 8;          // largest cluster
constexpr int F_LCAP = 1024;       // candidates per CTA
constexpr int F_MCAP = 2048;       // candidates per row
constexpr int F_HASH_BITS = 10;
constexpr int F_HASH = 1 << F_HASH_BITS;   // id->count slots per CTA
constexpr int F_KMAX = 1024;       // largest top-k served by the fused path

// What the fused kernel leaves behind for a stochastic row; the finish kernel turns it into a token.
struct RowRec {
    uint32_t kind;        // 0 = nothing to finish (row already final, or handed to the general kernel)
    uint32_t n_cand;      // candidates stored at [row * F_MCAP ...)
    uint32_t amax;        // argmax of the processed logits
    int32_t status;
    float m;              // max over finite processed logits
    float t;              // max(temperature, 1e-9)
    uint32_t n_parts;     // warps that contributed a partial fold
    uint32_t pad;
    double part[F_MAXC * 32];  // per-warp increments of the sequential f32 sum
};

struct FusedLaunch {
    uint32_t cluster;       // CTAs per row
    uint32_t slice_len;     // floats per CTA (multiple of 32)
    uint32_t chunk;         // consecutive floats per thread in the sum pass (odd)
    uint32_t* work_rows;    // rows handed to the general kernel
    uint32_t* work_count;
    RowRec* recs;           // [rows]
    uint32_t* cand_id;      // [rows x F_MCAP]
    float* cand_x;          // [rows x F_MCAP]
    long long* prof;        // optional phase timers, [gridDim.x x 16]
};

}  // namespace pgs
