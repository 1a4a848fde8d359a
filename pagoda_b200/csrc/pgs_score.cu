// log-softmax for scoring candidate continuations: the device form of `sampler::log_softmax`
// (pagoda/src/sampler.rs:73-87) as `Engine::score` uses it (pagoda/src/engine.rs:1066-1090: one
// forward per scored token, log-softmax over the vocabulary, one gather).  Per row:
//   max over all logits, e_i = exp(x_i - max), the f32 left-fold sum of the e_i (emulated exactly,
//   see pgs_block.cuh), log_sum = max(ln(sum), f32::MIN_POSITIVE), out_i = ln(e_i) - log_sum.
// exp is the exact expf of pgs_math.cuh; ln is the double-precision logarithm rounded to f32, which
// equals libm's logf except in rare last-bit cases (the tests allow 1e-6).
#include <cuda_runtime.h>

#include "pgs_args.cuh"
#include "pgs_block.cuh"

namespace pgs {

struct ScoreSmem {
    ReduceSmem rs;
    SeqSmem seq;
    unsigned long long exp_tab[32];
};

struct ScoreArgs {
    const float* logits;
    unsigned long long row_stride;
    uint32_t rows, vocab;
    const uint32_t* ids;     // optional: one id per row to gather
    float* out_gather;       // [rows]
    float* out_full;         // optional [rows x vocab]
    int32_t* status;         // optional
};

__device__ __forceinline__ float ln_f32(float v) { return __double2float_rn(log((double)v)); }

__global__ void __launch_bounds__(NT, 1) log_softmax_kernel(const ScoreArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ScoreSmem& sm = *reinterpret_cast<ScoreSmem*>(smem_raw);
    const int tid = threadIdx.x;
    if (tid < 32) sm.exp_tab[tid] = kExp2TableDev[tid];
    __syncthreads();
    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const float* x = a.logits + (size_t)row * a.row_stride;
        float mx = -INFINITY;
        int nonfinite = 0;
        for (uint32_t i = tid; i < a.vocab; i += NT) { const float v = x[i]; nonfinite |= !finite_f(v); mx = fmaxf(mx, v); }
        nonfinite = __syncthreads_or(nonfinite);
        const unsigned long long best = block_max_u64((unsigned long long)order_key(mx) << 32, sm.rs);
        if (a.status && tid == 0) a.status[row] = nonfinite ? ROW_NONFINITE : ROW_OK;
        if (nonfinite || !best) {   // the reference does not define scores for such rows
            if (tid == 0 && a.out_gather) a.out_gather[row] = NAN;
            continue;
        }
        const float m = key_to_float((uint32_t)(best >> 32));
        const float sum = seq_scan([&](int i) { return pgs_expf_tab(fsub(x[i], m), sm.exp_tab); }, (int)a.vocab, 0.0f,
                                   SEQ_SUM, 0.0f, nullptr, sm.seq, sm.rs);
        const float log_sum = fmaxf(ln_f32(sum), 1.17549435e-38f);
        if (a.out_full)
            for (uint32_t i = tid; i < a.vocab; i += NT)
                a.out_full[(size_t)row * a.vocab + i] = fsub(ln_f32(pgs_expf_tab(fsub(x[i], m), sm.exp_tab)), log_sum);
        if (a.ids && a.out_gather && tid == 0) {
            const uint32_t id = a.ids[row];
            a.out_gather[row] = id < a.vocab ? fsub(ln_f32(pgs_expf_tab(fsub(x[id], m), sm.exp_tab)), log_sum) : NAN;
        }
    }
}

cudaError_t configure_score() {
    return cudaFuncSetAttribute(log_softmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ScoreSmem));
}

cudaError_t launch_log_softmax(const ScoreArgs& a, uint32_t grid, cudaStream_t stream) {
    log_softmax_kernel<<<grid, NT, sizeof(ScoreSmem), stream>>>(a);
    return cudaGetLastError();
}

}  // namespace pgs
