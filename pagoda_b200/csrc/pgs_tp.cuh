// Arguments of the vocabulary-sharded kernels, shared by the kernels and the host side of the C ABI.
#pragma once

#include <stdint.h>

namespace pgs {

constexpr int TP_MAX_SHARDS = 8;

struct TpArgs {
    const float* logits;            // [rows x row_stride] this rank's columns
    unsigned long long row_stride;
    uint32_t rows, vocab, shard_vocab, shard_lo, n_shards, cand;
    const float* temperature;
    const float* top_p;
    const float* uniform;
    const uint32_t* top_k;          // merge: per row, 0 = off; must not exceed cand
    unsigned char* records;         // partial: out [rows x rec_bytes]; merge: in [n_shards x rows x rec_bytes]
    uint32_t rec_bytes;
    // peer-store exchange (all zero for the plain calls)
    unsigned char* peer_records[TP_MAX_SHARDS];   // partial: this shard's [rows x rec_bytes] block in every rank's gather buffer
    uint32_t* peer_flags[TP_MAX_SHARDS];          // partial: every rank's flag array [n_shards]
    uint32_t* flags;                // merge: this rank's flag array [n_shards], raised by the emitters
    uint32_t* done;                 // partial: CTAs finished in this launch
    uint32_t epoch;                 // step number the flags are raised to / waited for
    uint32_t shard_rank;
    uint32_t wait_polls;            // merge: bound of the flag wait, in polls of about half a microsecond each
    unsigned long long* timeouts;   // merge: rows that gave up waiting, counted over all launches
};


struct TpOut {
    uint32_t* token; int32_t* status; uint8_t* drew; uint32_t* argmax;
    float* gmax; float* gsum; float* total; uint32_t* n_kept;
};

}  // namespace pgs
