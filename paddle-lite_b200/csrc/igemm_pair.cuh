// Interface of the two-SM (cta_group::2) tensor-core kernel (igemm_pair.cu).
#pragma once
#include "igemm_tc.cuh"

namespace plb {

// Whether this problem should run as 256 x BN tiles on pairs of SMs: plain int8 / fp32 / accumulator output
// (no residual, no fused shortcut), a compute-bound shape (long K, wide channel tile) and enough tiles for
// every pair; PLB_TC_PAIR=0 / 1 (read when the layer was prepared) turns it off / forces it wherever it fits.
bool igemm_pair_wanted(const plb_ctx* ctx, const IgemmProblem& p);
int igemm_pair_launch(plb_ctx* ctx, const IgemmProblem& p);

}  // namespace plb
