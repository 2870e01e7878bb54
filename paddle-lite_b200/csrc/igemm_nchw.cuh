// Interface of the NCHW-native 1x1 tensor-core kernel (igemm_nchw.cu).
#pragma once
#include "igemm_tc.cuh"

namespace plb {

// y[n][co][p] = epilogue(sum_ci w[co][ci] * x[n][ci][p]) on NCHW tensors, p = pixel of an h*w image.
struct NchwProblem {
  const int8_t* x;   // [batch][cin][hw] int8
  const int8_t* w;   // [cout][cin_pad] int8, rows zero-padded to cin_pad (multiple of 32)
  int batch, cin, cin_pad, cout, hw;
  int x_pitch, y_pitch;  // elements between the rows (channels) of x and of y; 0 = hw (dense NCHW)
  int out_mode;      // OUT_I8 / OUT_F32 / OUT_ACC
  void* y;           // [batch][cout][hw] int8 / float / int32
  EpiParams epi;
  int bres_switch;   // gather kernel only: 0 = never the pixel-resident order, 1 = wherever it fits (tuning switch; else planner)
};

bool igemm_nchw_supported(const NchwProblem& p, std::string* why);
int igemm_nchw_launch(plb_ctx* ctx, const NchwProblem& p);
// The same on images whose rows TMA cannot address (pixel counts that are not a multiple of 16; igemm_nchw_gather.cu):
// dense tensors (no pitch), 4-byte aligned.
bool igemm_nchw_gather_supported(const plb_ctx* ctx, const NchwProblem& p, std::string* why);
int igemm_nchw_gather_launch(plb_ctx* ctx, const NchwProblem& p);

}  // namespace plb
