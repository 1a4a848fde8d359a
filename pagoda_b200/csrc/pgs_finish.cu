// Finish kernel: one CTA per batch row turns the record the fused kernel left behind (row max,
// the f32 sum, a short candidate list that contains the whole top-k set) into a token.  All rows
// run side by side, so the short serial folds of one row overlap with those of every other row.
#include "pgs_finish.cuh"

namespace pgs {

__global__ void __launch_bounds__(NT, 1) finish_kernel(const RowArgs a, const FusedLaunch fl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FinishSmem& sm = *reinterpret_cast<FinishSmem*>(smem_raw);
    const uint32_t row = blockIdx.x;
    if (fl.recs[row].kind != 1u) return;
    const RowRec& rec = fl.recs[row];
    double s2 = 0.0;
    for (uint32_t r = 0; r < rec.n_parts; r++) s2 += rec.part[r];
    finish_row(sm, a, row, a.vocab, fl.cand_id + (size_t)row * F_MCAP, fl.cand_x + (size_t)row * F_MCAP, rec.n_cand,
               rec.m, rec.t, (float)s2, a.top_k ? a.top_k[row] : 0u, a.top_p ? a.top_p[row] : 1.0f,
               a.uniform ? a.uniform[row] : 0.0f, rec.amax, rec.status);
}

cudaError_t configure_finish() {
    return cudaFuncSetAttribute(finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FinishSmem));
}

cudaError_t launch_finish(const RowArgs& a, const FusedLaunch& fl, cudaStream_t stream) {
    finish_kernel<<<a.rows, NT, sizeof(FinishSmem), stream>>>(a, fl);
    return cudaGetLastError();
}

}  // namespace pgs
