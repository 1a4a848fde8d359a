// Launch block of the streaming row kernel (pgs_stream.cu), shared with the host launcher.
#pragma once

#include <stdint.h>


namespace pgs {

constexpr int S_KMAX = 1024;         // largest top-k the streaming kernel serves
constexpr int S_MAX_VOCAB = 1 << 20;  // longest row the streaming kernel serves
constexpr int S_MAX_HASH = 4096;     // id -> count slots (histories of up to 2048 ids)

struct StreamLaunch {
    uint32_t hash_slots;        // id -> count slots in use: a power of two >= 2 x the longest history, <= S_MAX_HASH
    uint32_t cohort;            // rows that may be in their first pass (the one that reads HBM) at once
    uint32_t done_base;         // value of *p1_done when this launch starts
    uint32_t gate_polls;        // bound of the gate's wait, in polls
    uint32_t* p1_done;          // rows that have finished their first pass, counted over all launches
    uint32_t* work_rows;        // rows handed to the general kernel
    uint32_t* work_count;
    long long* prof;            // optional phase timers, [gridDim.x x 16]
};

}  // namespace pgs
