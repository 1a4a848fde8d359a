// Finish kernel: rows whose candidate list is too long for the streaming row kernel to finish itself (more than
// 256 candidates: top-k in the hundreds).  A small grid walks the list of such rows the row kernel left behind (row
// max, the f32 sum, the candidates, which contain the whole top-k set) and turns each into a token.
#include "pgs_finish.cuh"

namespace pgs {

// (At most 48 registers per thread keeps the usually empty pass cheap to schedule.)
__global__ void __maxnreg__(48) finish_kernel(const RowArgs a, const Handoff ho) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FinishSmem& sm = *reinterpret_cast<FinishSmem*>(smem_raw);
    cudaGridDependencySynchronize();   // launched ahead of the end of the row kernel: its list is final from here on
    const uint32_t n_long = *ho.long_count;
    if (n_long == 0u) return;   // the usual case: no long list in this step, nothing to reset
    for (uint32_t i = blockIdx.x; i < n_long; i += gridDim.x) {
        const uint32_t row = ho.long_rows[i];
        const RowRec& rec = ho.recs[row];
        finish_row(sm, a, row, a.vocab, ho.cand_id + (size_t)row * F_MCAP, ho.cand_x + (size_t)row * F_MCAP, rec.n_cand,
                   rec.m, rec.t, rec.S, a.top_k ? a.top_k[row] : 0u, a.top_p ? a.top_p[row] : 1.0f,
                   a.uniform ? a.uniform[row] : 0.0f, rec.amax, rec.status);
        __syncthreads();
    }
    // the last CTA to finish empties the list for the next step
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ho.long_count + 1, 1u) == gridDim.x - 1) { ho.long_count[0] = 0u; ho.long_count[1] = 0u; }
    }
}

cudaError_t configure_finish() {
    return cudaFuncSetAttribute(finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FinishSmem));
}

// Launched with programmatic stream serialization: the kernel may be set up while the kernel before it in the stream
// still runs, and waits for it at cudaGridDependencySynchronize().
cudaError_t launch_finish(const RowArgs& a, const Handoff& ho, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.rows < 128u ? a.rows : 128u, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = sizeof(FinishSmem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, finish_kernel, a, ho);
}

}  // namespace pgs
