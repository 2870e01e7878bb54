// CUDA-core kernels of the path: direct convolution, depthwise 3x3-style convolution,
// sparse 1x1 convolution over the decoded reference encoding, and the glue between int8
// layers (layout staging, calib, pooling).  Launchers are declared here and defined in
// kernels_simple.cu.
#pragma once
#include "common.cuh"

namespace plb {

struct ConvGeom {
  int batch, cin, h, w;       // logical input
  int cin_stride;             // bytes between pixels of the NHWC input
  int cout, kh, kw;
  int stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int groups;
  int ho, wo;
  int cg_pad;                 // filter row length per tap: [cout][kh][kw][cg_pad]
  int dw_strip;               // depthwise 3x3: output rows per strip (0 = register-tiled kernel, -1 = cost model)
};

struct OutSpec {
  int mode;                   // OutMode of igemm_tc.cuh
  void* y;                    // [m_total, ldy]
  int ldy;
  EpiParams epi;
  const float* residual;
  float* y_f32;
  int8_t* y_i8;
  float inv_next_scale;
  // tensor-core path only: shortcut GEMM of a residual block computed in the same launch (see IgemmProblem)
  const int8_t* a2;
  const int8_t* b2;
  int im2col2, h2, w2, cin_pad2, stride2_h, stride2_w;
  const float* scale2;
  const float* bias2;
};

// Generic grouped convolution, NHWC in / NHWC out, one thread per output value.
int conv_direct_launch(plb_ctx* ctx, const ConvGeom& g, const int8_t* x, const int8_t* w_rsc,
                       const OutSpec& out);
// Depthwise convolution, NHWC, channels multiple of 4 in storage; filter [kh*kw][c_stride].
int dwconv_launch(plb_ctx* ctx, const ConvGeom& g, const int8_t* x, const int8_t* w_tc,
                  const OutSpec& out);

// Sparse 1x1 convolution on NCHW tensors over CSR rows decoded from the reference encoding.
struct SparseGeom {
  int batch, cin, cout, hw;
  int is_int8;     // input/weight type
  int out_mode;    // OUT_F32 / OUT_I8
};
// col_val (fp32 only, nullable): {input channel, weight bits} pairs, one 8-byte word per non-zero, for the pixel-tile
// kernel.
int sparse_csr_launch(plb_ctx* ctx, const SparseGeom& g, const void* x, const int* row_ptr,
                      const int* col, const void* val, const void* col_val, const float* bias_raw,
                      const EpiParams& epi, void* y);

// int8 variant that stages the input slab in shared memory and walks non-zeros four at a time
// with dp4a (grp_ptr [cout+1], grp_idx = 4 x uint16 input channels, grp_w = 4 x int8 weights).
int sparse_slab_supported(const SparseGeom& g, const void* x, const void* y);
int sparse_slab_launch(plb_ctx* ctx, const SparseGeom& g, const int8_t* x, const int* grp_ptr,
                       const void* grp_idx, const void* grp_w, const EpiParams& epi, void* y);

int softmax_rows_launch(plb_ctx* ctx, const float* x, float* y, int rows, int cols);
int calib_f32_to_i8_launch(plb_ctx* ctx, const float* x, int8_t* q, size_t n, float scale);
int calib_i8_to_f32_launch(plb_ctx* ctx, const int8_t* q, float* y, size_t n, float scale);
int nchw_to_nhwc_i8_launch(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w,
                           int cpad);
// Stem staging: int8 or fp32 (quantised with `scale`) NCHW -> folded [n, ht, wo, fh*32] int8
// (fh input rows x kw taps x cin channels per staged pixel; see fold_rows_kernel).
int fold_rows_launch(plb_ctx* ctx, const void* x, int x_is_f32, int8_t* y, int n, int c, int h, int w,
                     int ht, int wo, int kw, int fh, int stride_w, int pad_t, int pad_l, int dil_w,
                     float scale);
int nhwc_to_nchw_launch(plb_ctx* ctx, const void* x, void* y, int n, int c, int h, int w,
                        int elem_bytes);
int calib_nchw_f32_to_nhwc_i8_launch(plb_ctx* ctx, const float* x, int8_t* y, int n, int c, int h,
                                     int w, int cpad, float scale);
// Rows of `len` bytes back to back -> rows of `pitch` bytes (multiple of 16), and back (1- or 4-byte elements;
// len and pitch in elements there): what TMA needs for NCHW images whose pixel count is not a multiple of 16.
int pitch_rows_i8_launch(plb_ctx* ctx, const void* src, void* dst, long rows, int len, int pitch);
int unpitch_rows_launch(plb_ctx* ctx, const void* src, void* dst, long rows, int len, int pitch, int elem_bytes);
int maxpool_nhwc_i8_launch(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w,
                           int k, int stride, int pad);
int global_avgpool_nhwc_f32_launch(plb_ctx* ctx, const float* x, float* y, int8_t* q, int n, int hw,
                                   int c, float scale);

}  // namespace plb
