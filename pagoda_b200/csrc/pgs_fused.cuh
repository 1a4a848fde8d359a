// Hand-off from the streaming row kernel (pgs_stream.cu) to the finish kernel (pgs_finish.cu): rows whose candidate
// list is too long to be finished inside the streaming kernel.
#pragma once

#include <stdint.h>

namespace pgs {

constexpr int F_MCAP = 2048;       // candidates per row

// What the streaming kernel leaves behind for such a row; the finish kernel turns it into a token.
struct RowRec {
    uint32_t n_cand;      // candidates stored at [row * F_MCAP ...)
    uint32_t amax;        // argmax of the processed logits
    int32_t status;
    float m;              // max over finite processed logits
    float t;              // max(temperature, 1e-9)
    float S;              // the f32 left-fold sum of the softmax numerators
};

struct Handoff {
    RowRec* recs;           // [rows]
    uint32_t* cand_id;      // [rows x F_MCAP]
    float* cand_x;          // [rows x F_MCAP]
    uint32_t* long_rows;    // the rows handed over in this step
    uint32_t* long_count;   // [0] = how many, [1] = CTAs of the finish kernel that are done with the list
};

}  // namespace pgs
