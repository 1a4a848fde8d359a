"""B200 (sm_100a) backend for pagoda's per-step logits -> token chain.

The product is `libpagoda_sampler.so` (CUDA kernels behind the C ABI of
`include/pagoda_sampler.h`).  This package is the thin Python view of that ABI used by the
tests and the benchmark; it never computes anything itself and has no CPU path: creating a
`Sampler` without the built library or without a CUDA device raises.
"""
from .capi import (Grammar, GrammarState, PGS_BF16, PGS_F32, ROW_BAD_PARAM, ROW_DEAD, ROW_EMPTY, ROW_NONFINITE, ROW_OK, BatchResult,
                   Sampler, SamplerError, lib_path, load_library)

__all__ = ["Grammar", "GrammarState", "Sampler", "SamplerError", "BatchResult", "load_library", "lib_path", "PGS_F32", "PGS_BF16",
           "ROW_OK", "ROW_NONFINITE", "ROW_DEAD", "ROW_EMPTY", "ROW_BAD_PARAM"]
