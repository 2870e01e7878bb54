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

// Tuning switches of the tensor-core kernel.  They are read from the environment (PLB_TC_*) ONCE,
// when a layer is prepared, and travel with the prepared layer; -1 means "let the planner decide".
// Nothing on the run path reads the environment.
struct TcSwitches {
  int slab = -1;          // PLB_TC_SLAB: window mode off (0) / forced wherever it fits (1)
  int bn = -1;            // PLB_TC_BN: channel tile
  int kc = -1;            // PLB_TC_KC: bytes of K per pipeline stage (32 / 64 / 128), at most what the channels allow
  int stages = -1;        // PLB_TC_STAGES: operand ring depth
  int acc_bufs = -1;      // PLB_TC_ACC_BUFS: accumulator buffers in tensor memory (2, 4, 8)
  int resident = 1;       // PLB_TC_RESIDENT=0: never keep the filter in shared memory
  int staged = 1;         // PLB_TC_STAGED=0: epilogue with direct global accesses
  int res_prefetch_tiles = -1;  // PLB_TC_RES_PREFETCH_TILES: ... by default for launches of up to this many tiles per SM
  int res_prefetch = -1;  // PLB_TC_RES_PREFETCH: residual tile fetched one chunk ahead
  int acc_small = 1;      // PLB_TC_ACC_SMALL=0: int -> float through the conversion pipe always
  int sb_smem = 1;        // PLB_TC_SB_SMEM=0: scale / bias tables stay in global memory
  int fast_flat = 1, fast_im2col = 1, fast_mma = 1, fast_dual = 1, fast_window = 1;  // PLB_TC_FAST_*=0: generic role loops
  int pair = -1;          // PLB_TC_PAIR: two-SM tiles (cta_group::2) off (0) / forced wherever they fit (1)
  int nchw = -1;          // PLB_TC_NCHW: NCHW-native 1x1 kernel off (0) / forced wherever it fits (1)
  int nchw_gather = -1;   // PLB_TC_NCHW_GATHER=0: images whose pixel count is not a multiple of 16 are re-pitched / staged instead
  int nchw_bres = -1;     // PLB_TC_NCHW_BRES=0: that kernel never keeps a pixel tile resident for all channel tiles
  int dw_strip = -1;      // PLB_DW_STRIP: depthwise 3x3 rows per strip (0 = the register-tiled kernel)
  int stem = -1;          // PLB_STEM=0: first layers always run as a staging pass + convolution
  int dwpw = -1;          // PLB_DWPW=0: depthwise + 1x1 pairs never run as one launch
  int dwpw_tw = -1;       // PLB_DWPW_TW: tile columns of the fused depthwise + 1x1 kernel (4 / 8 / 16)
  int dwpw_seg = -1;      // PLB_DWPW_SEG: output rows per work item of that kernel
};
TcSwitches tc_switches_from_env();

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
  const TcSwitches* sw;   // nullptr: defaults
};

// Plans (tile shapes, tensor maps, kernel choice) of the problems a prepared layer has been run on.
// A run with the same pointers and sizes as an earlier one re-launches the stored plan without
// re-deriving it or re-encoding tensor maps.  Owned by the prepared layer; not thread-safe.
struct IgemmPlanCache;
IgemmPlanCache* igemm_plan_cache_create();
void igemm_plan_cache_destroy(IgemmPlanCache* c);
long igemm_plan_cache_hits(const IgemmPlanCache* c);

// Whether the tensor-core kernel can take this problem (shape and alignment rules).
bool igemm_tc_supported(const IgemmProblem& p, std::string* why);
// Enqueue on ctx->stream.  Returns PLB_OK or an error code.
int igemm_tc_launch(plb_ctx* ctx, const IgemmProblem& p, IgemmPlanCache* cache = nullptr);

}  // namespace plb
