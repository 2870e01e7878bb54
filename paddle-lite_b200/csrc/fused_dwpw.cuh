// Depthwise 3x3 convolution + the 1x1 convolution that follows it, in ONE launch (fused_dwpw.cu).
#pragma once
#include "common.cuh"
#include "igemm_tc.cuh"

namespace plb {

struct DwpwProblem {
  // depthwise stage: x is channels-last int8 [batch, h, w, c] with pixel pitch c; 3x3 filter [9][cg_pad], dilation 1
  const int8_t* x;
  int batch, h, w, c;
  int stride;          // 1 or 2, the same in both directions
  int pad_t, pad_l;
  int ho, wo;          // output of the depthwise stage = pixels of the 1x1 stage
  const int8_t* wdw;
  int cg_pad;
  EpiParams dw_epi;    // int8 requantiser of the depthwise layer (act NONE / RELU / RELU6)
  // pointwise stage: filter [cout][c] int8, K-major
  const int8_t* wpw;
  int cout;
  EpiParams pw_epi;    // int8 requantiser of the 1x1 layer
  int8_t* y;           // channels-last [batch, ho, wo, cout], pixel pitch ldy
  int ldy;
  int tw, seg_rows;    // tuning overrides: tile columns (4 / 8 / 16) and output rows per work item; <= 0: planner
};

bool dwpw_fused_supported(const plb_ctx* ctx, const DwpwProblem& p, std::string* why);
int dwpw_fused_launch(plb_ctx* ctx, const DwpwProblem& p);

}  // namespace plb
