// Interface of the tcgen05 implicit-GEMM kernel (igemm_tc.cu).
#pragma once
#include "common.cuh"

namespace plb {

enum OutMode : int {
  OUT_F32 = 0,       // y = act(fma(acc, scale, bias)) as float
  OUT_I8 = 1,        // y = clamp(rne(act(fma(acc, scale, bias)))) as int8
  OUT_ACC = 2,       // raw int32 accumulators
  OUT_ADD_RELU = 3,  // v = fma(acc, scale, bias) + residual; relu; optional f32 and calib-int8 stores
};

// One launch computes D[m, n] = sum_k A[m, k] * B[n, k] over int8 operands with int32
// accumulation and applies the epilogue.  m indexes output pixels (or fc rows), n output
// channels.  A is either a plain row-major [m_total, cin_pad] matrix (flat) or the
// im2col view of an NHWC tensor; B is the filter repacked to [cout, taps * cin_pad].
struct IgemmProblem {
  // A operand
  const int8_t* a;   // flat: [m_total, cin_pad]; im2col: NHWC [batch, h, w, cin_pad]
  int im2col;        // 0 flat, 1 im2col
  int batch, h, w;   // im2col only
  int cin_pad;       // bytes per pixel / row, multiple of 32 (flat: multiple of 16)
  int kh, kw, stride_h, stride_w, pad_t, pad_b, pad_l, pad_r, dil_h, dil_w;
  int ho, wo;
  int m_total;       // batch*ho*wo, or fc rows
  // B operand
  const int8_t* b;   // [cout, taps*cin_pad]
  int cout;
  // epilogue
  int out_mode;
  void* y;           // OUT_F32 / OUT_I8 / OUT_ACC destination, row-major [m_total, ldy]
  int ldy;
  EpiParams epi;
  const float* residual;  // OUT_ADD_RELU
  float* y_f32;           // OUT_ADD_RELU, nullable
  int8_t* y_i8;           // OUT_ADD_RELU, nullable
  float inv_next_scale;   // OUT_ADD_RELU: 1 / scale of the next layer's input
  // Dual mode (OUT_ADD_RELU with a flat main GEMM and no residual tensor): the residual value is a
  // second 1x1 GEMM, D2[m, n] = sum_k A2[m, k] * B2[n, k], turned into fma(D2, scale2, bias2) --
  // the shortcut convolution of a residual block, computed in the same launch.
  const int8_t* a2;       // nullptr: no second GEMM.  Flat [m_total, cin_pad2], or (im2col2) NHWC [batch, h2, w2, cin_pad2]
  int im2col2;            // 1: A2 is read at pixel (oh * stride2_h, ow * stride2_w) of an h2 x w2 image
  int h2, w2, cin_pad2, stride2_h, stride2_w;
  const int8_t* b2;       // [cout, cin_pad2]
  const float* scale2;    // [cout] folded ws * in_s of the shortcut
  const float* bias2;     // [cout]
};

// Whether the tensor-core kernel can take this problem (shape and alignment rules).
bool igemm_tc_supported(const IgemmProblem& p, std::string* why);
// Enqueue on ctx->stream.  Returns PLB_OK or an error code.
int igemm_tc_launch(plb_ctx* ctx, const IgemmProblem& p);

}  // namespace plb
