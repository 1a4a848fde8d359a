// Kernel argument blocks shared by the host-side C ABI and the row kernels.
#pragma once

#include <stdint.h>

namespace pgs {

// One uploaded grammar table (device memory owned by the handle).
struct TableDir {
    const uint32_t* words;            // [n_states x words_per_state]
    const uint8_t* flags;             // [n_states] bit 0 = complete, bit 1 = dead
    uint32_t words_per_state;
    uint32_t n_states;
    uint32_t live;
    uint32_t pad;
};

constexpr int MAX_TABLES = 256;

// Row status values mirror pgs_row_status of the C ABI.
enum { ROW_OK = 0, ROW_NONFINITE = 1, ROW_DEAD = 2, ROW_EMPTY = 3, ROW_BAD_PARAM = 4, ROW_LOAD_TIMEOUT = 5 };

struct RowArgs {
    // inputs (device pointers)
    const void* logits;
    uint32_t dtype;           // 0 = f32, 1 = bf16
    uint32_t rows, vocab;
    unsigned long long row_stride;
    const float* temperature;
    const uint32_t* top_k;
    const float* top_p;
    const float* freq;
    const float* pres;
    const float* rep;
    const uint32_t* hist_offsets;
    const uint32_t* hist_ids;
    const int32_t* mask_table;
    const int32_t* mask_state;
    int32_t eos;
    const float* uniform;
    // grammar tables
    const TableDir* tables;           // [MAX_TABLES]
    // outputs
    uint32_t* token;
    int32_t* status;
    uint8_t* drew;
    uint32_t* argmax;
    float* row_max;
    float* sumexp;
    float* total;
    uint32_t* n_kept;
    uint32_t dump_cap;
    uint32_t* dump_ids;
    float* dump_probs;
    // per-CTA scratch slots in global memory (slot = blockIdx.x)
    float* sx;                      // [slots x vocab_pad] processed logits, then softmax numerators
    uint32_t* sl_id;                // [slots x vocab_pad] candidate list: ids
    float* sl_p;                    // [slots x vocab_pad] candidate list: probabilities
    unsigned long long* sl_key;     // [slots x sort_pad] sort keys
    uint32_t* sh_key;               // [slots x hash_cap] history hash table: ids
    uint32_t* sh_cnt;               // [slots x hash_cap] history hash table: counts
    uint32_t vocab_pad, sort_pad, hash_cap, max_history;
    // optional work list: process rows work_rows[0 .. *work_count) instead of 0 .. rows
    const uint32_t* work_rows;
    uint32_t* work_count;           // [0] = number of listed rows, [1] = CTAs that finished the list
    unsigned long long* faulted;    // optional: rows that ended as ROW_NONFINITE, counted over all launches
    // vocabulary-sharded emit mode (tp_records != nullptr): `logits` holds the columns id_base .. id_base + vocab
    // of every row, history ids are global ids, and a row ends as a record (TpRecHead + candidates) instead of a
    // token: the outputs above are not written
    unsigned char* tp_records;      // [rows x tp_rec_bytes]
    uint32_t tp_rec_bytes, tp_cand;
    uint32_t id_base;               // global id of column 0 (0 outside of the sharded mode)
};

// One shard's share of one row.  n_status: candidates in the record (low 24 bits) and the row status the shard
// found (high 8 bits: ROW_OK, ROW_NONFINITE, ROW_DEAD or ROW_BAD_PARAM).  m is the shard's maximum (-inf when the
// shard holds no finite logit), s its f32 left-fold sum of exp((x - m) / t) (0 for greedy rows), argmax a global
// id.  The head is followed by float x[cand] and uint32 id[cand], sorted by (x descending, id ascending).
struct TpRecHead { float m; float s; uint32_t n_status; uint32_t argmax; };

__device__ __forceinline__ void tp_write_head(const RowArgs& a, uint32_t row, float m, float s, uint32_t n, int status,
                                              uint32_t argmax_local) {
    TpRecHead* h = reinterpret_cast<TpRecHead*>(a.tp_records + (size_t)row * a.tp_rec_bytes);
    h->m = m; h->s = s; h->n_status = n | ((uint32_t)status << 24); h->argmax = a.id_base + argmax_local;
}

}  // namespace pgs
