// First layer of a network in ONE launch: fp32 NCHW image -> calib -> row-folded operand tiles -> tcgen05 GEMM -> int8
// channels-last output (stem_tc.cu).  Replaces the staging pass + convolution pair of plb_conv_run_image_f32 where it fits.
#pragma once
#include "common.cuh"

namespace plb {

struct StemProblem {
  const float* x;       // [batch, cin, h, w] fp32
  int batch, cin, h, w;
  int kh, kw, stride_h, stride_w, pad_t, pad_l;
  int ho, wo;
  int fold_h, fold_kh;  // input rows per folded row group (= stride_h), filter row groups
  const int8_t* wfold;  // [cout][fold_kh][fold_h * 32] int8, the layer's row-folded filter
  const int8_t* wfold16;  // [cout][fold_kh * fold_h][16] int8 or null: the same filter with 16-byte rows (kw * cin <= 16)
  int cout;
  float in_scale;
  EpiParams epi;        // int8 requantiser
  int8_t* y;            // [batch, ho, wo, cout] int8, pixel pitch cout
};

bool stem_tc_supported(const plb_ctx* ctx, const StemProblem& p, std::string* why);
int stem_tc_launch(plb_ctx* ctx, const StemProblem& p);

}  // namespace plb
