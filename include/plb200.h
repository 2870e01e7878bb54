/*
 * plb200 — C ABI of the B200 (sm_100a) int8 conv / depthwise / fc / sparse_conv kernels.
 *
 * This is the boundary a `kCUDA` / `kInt8` target of Paddle-Lite binds: every prepared
 * object corresponds to what one reference kernel instance holds after PrepareForRun(),
 * every *_run() to one Run().  Plain pointers and sizes only; no C++ or torch types.
 *
 * Conventions
 *   - every function returns 0 on success or a PLB_E_* code; nothing aborts or throws.
 *     plb_last_error() gives the message of the last failure on the calling thread.
 *   - pointers are DEVICE pointers unless the name ends in _h (host).
 *   - a plb_ctx is bound to one device and one CUDA stream; all work of objects prepared
 *     on it is enqueued on that stream.  One ctx per host thread / stream; objects are
 *     not thread-safe.
 *   - tensors at this boundary use the reference layouts (NCHW activations, OIHW filters,
 *     [K,N] fc weights) unless a function says NHWC.
 *   - *_run() calls are asynchronous; plb_ctx_sync() and plb_copy_d2h() wait and report
 *     kernel-side faults (a pipeline wait that ran out) as PLB_E_DEVICE.
 *   - tuning switches (PLB_TC_*, PLB_DW_STRIP in the environment) are read when a layer is
 *     prepared, never on the run path.
 */
#ifndef PLB200_H_
#define PLB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLB_OK 0
#define PLB_E_INVALID 1     /* bad argument (null pointer, bad dims, scale-vector length) */
#define PLB_E_UNSUPPORTED 2 /* valid request this build has no kernel for */
#define PLB_E_CUDA 3        /* a CUDA runtime / driver call failed */
#define PLB_E_DEVICE 4      /* a kernel reported a fault through the ctx status word */
#define PLB_E_NOMEM 5       /* workspace could not be allocated */

/* activation codes = relu_type of the reference GEMM (lite/kernels/x86/conv_compute.cc:257-270) */
#define PLB_ACT_NONE 0
#define PLB_ACT_RELU 1
#define PLB_ACT_RELU6 2 /* bound = act_alpha (ActivationParam::Relu_clipped_coef) */
#define PLB_ACT_LEAKY 3 /* slope = act_alpha (ActivationParam::Leaky_relu_alpha) */

#define PLB_OUT_F32 0 /* alias fp32_out */
#define PLB_OUT_I8 1  /* alias int8_out */

/* kernel choice for conv; AUTO is what a caller wants, the others exist for tests */
#define PLB_IMPL_AUTO 0
#define PLB_IMPL_DIRECT 1 /* CUDA-core direct convolution */
#define PLB_IMPL_TC 2     /* tcgen05 implicit GEMM */

typedef struct plb_ctx plb_ctx;
typedef struct plb_conv plb_conv;
typedef struct plb_fc plb_fc;
typedef struct plb_sparse plb_sparse;

/* ------------------------------------------------------------------ context
 * Replaces Context<TARGET> + the stream the reference keeps per kernel
 * (lite/core/context.h:430-484, KernelBase::SetContext lite/core/kernel.h:133-136). */
int plb_ctx_create(int device, void* cuda_stream, plb_ctx** out);
void plb_ctx_destroy(plb_ctx* ctx);
/* Wait for the ctx stream; returns PLB_E_DEVICE if any kernel flagged a fault since the
 * last call (the flag is cleared). */
int plb_ctx_sync(plb_ctx* ctx);
/* Optional: hand the ctx a caller-owned scratch buffer (layout staging for the NCHW entry
 * points).  Without it the ctx grows its own with cudaMalloc on demand.  Replaces the
 * per-Run TargetMalloc of the im2col buffer (conv_compute.cc:306-310). */
int plb_ctx_set_workspace(plb_ctx* ctx, void* dptr, size_t bytes);
/* Bytes of scratch the NCHW entry points of this object need for `batch` images. */
size_t plb_conv_workspace_bytes(const plb_conv* conv, int batch);
const char* plb_last_error(void);
/* Number of kernels this library has launched on the ctx since creation. */
long plb_ctx_launch_count(const plb_ctx* ctx);
/* How many of those were tensor-core convolutions in window mode (each input pixel of a tile
 * fetched once and shared by all filter taps).  For tests and tuning; no reference counterpart. */
long plb_ctx_window_launch_count(const plb_ctx* ctx);
/* How many 1x1 convolutions ran directly on NCHW tensors (no layout staging passes).  For tests. */
long plb_ctx_nchw_launch_count(const plb_ctx* ctx);
/* ... of which on images whose pixel count is not a multiple of 16 (operand tiles filled by gather warps).  For tests. */
long plb_ctx_nchw_gather_launch_count(const plb_ctx* ctx);
/* How many GEMMs ran as two-SM tiles (256 x N output tiles on pairs of SMs).  For tests. */
long plb_ctx_pair_launch_count(const plb_ctx* ctx);
/* How many first layers ran from the fp32 image in one launch (plb_conv_run_image_f32 without a staging pass).  For tests. */
long plb_ctx_stem_launch_count(const plb_ctx* ctx);
/* How many depthwise + 1x1 pairs ran as one launch (plb_conv_run_nhwc_dwpw).  For tests. */
long plb_ctx_dwpw_launch_count(const plb_ctx* ctx);
/* Bytes of layout-staging scratch the ctx currently holds (its own or the caller's).  Test hook. */
size_t plb_ctx_workspace_size(const plb_ctx* ctx);

/* ------------------------------------------------------------------ conv2d / depthwise_conv2d
 * plb_conv_desc carries what operators::ConvParam holds for an int8 kernel
 * (lite/operators/op_params.h:403-455 + WITH_INT8_CONFIG :39-44 + ActivationParam :331-362). */
typedef struct plb_conv_desc {
  int cin, h, w;                 /* input [N,cin,h,w]; N is given per run                */
  int cout, kh, kw;              /* filter [cout, cin/groups, kh, kw]                     */
  int stride_h, stride_w;        /* ConvParam::strides                                    */
  int pad_top, pad_bottom, pad_left, pad_right; /* ConvParam::paddings (4 entries)        */
  int dil_h, dil_w;              /* ConvParam::dilations                                  */
  int groups;                    /* groups == cin == cout selects the depthwise kernel    */
  int act;                       /* PLB_ACT_*                                             */
  float act_alpha;
  float in_scale;                /* ConvParam::input_scale                                */
  float out_scale;               /* ConvParam::output_scale (int8 out only)               */
  int out_dtype;                 /* PLB_OUT_F32 | PLB_OUT_I8                              */
  int leaky_compat;              /* !=0: int8-out leaky slope is alpha/out_scale as in
                                    conv_compute.cc:394; 0: slope is alpha               */
  int impl;                      /* PLB_IMPL_*                                            */
} plb_conv_desc;

/* = Conv2dCompute<kInt8,*>::PrepareForRun (conv_compute.cc:216-289, :344-420): copies the
 * filter (OIHW, host), expands weight_scale (n_wscale must be 1 or cout, else
 * PLB_E_INVALID like the reference's LOG(FATAL) at :242-244), folds scales and bias. */
int plb_conv_prepare(plb_ctx* ctx, const plb_conv_desc* desc, const int8_t* filter_h,
                     const float* wscale_h, int n_wscale, const float* bias_h /* nullable */,
                     plb_conv** out);
/* = Conv2dCompute<kInt8,*>::Run (conv_compute.cc:292-341, :423-472).
 * x [batch,cin,h,w] int8 NCHW; y [batch,cout,ho,wo] float or int8 NCHW. */
int plb_conv_run(plb_conv* conv, const int8_t* x, void* y, int batch);
/* Same arithmetic on channels-last tensors, no layout staging: x [batch,h,w,cin] int8 with
 * cin a multiple of 32 (depthwise: 16), y [batch,ho,wo,cout]. */
int plb_conv_run_nhwc(plb_conv* conv, const int8_t* x, void* y, int batch);
/* First layer of a network: x is the fp32 NCHW image [batch,cin,h,w].  Quantises it with the
 * layer's input_scale (the `calib` op the reference inserts in front of the first int8 layer,
 * lite/core/optimizer/mir/type_precision_cast_pass.cc:75-105, arithmetic of
 * lite/backends/x86/math/calib.cc:25-151), stages it in the ctx workspace and runs the layer;
 * y is channels-last [batch,ho,wo,cout].  Layers with few input channels (cin*kw <= 32, e.g.
 * RGB stems) are staged row-folded so the tensor cores see 32-byte pixels. */
int plb_conv_run_image_f32(plb_conv* conv, const float* x, void* y, int batch);
/* plb_conv_run without any device allocation.  No counterpart in the reference: this entry
 * exists for hosts that must not have a library allocate behind their back — a serving loop
 * in which a cudaMalloc would synchronise the whole device and stall the other predictors
 * sharing the GPU, or a runtime that has given all device memory to its own planned arena
 * (what memory_optimize_pass does for the reference's buffers).  The NCHW<->channels-last
 * staging that plb_conv_run keeps in the ctx workspace lives here in a fixed array inside the
 * library image: 8 MiB, held by every GPU that loads the library until the process exits.
 *   - a call whose staging (plb_conv_workspace_bytes(conv, batch)) exceeds 8 MiB is rejected
 *     with PLB_E_INVALID and a message that names both sizes; nothing is launched.
 *   - the first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before starting any stream capture.  The lookup
 *     is guarded, so first calls may come from several host threads.
 *   - all calls of the process on one device share the array, and it keeps whatever the last
 *     call left there.  Every byte a call reads it has written first, so consecutive calls on
 *     one stream are safe; calls that can overlap on the GPU (different streams or contexts)
 *     race on it and must be serialised by the caller.
 * Same arguments and result as plb_conv_run. */
int plb_conv_run_static(plb_conv* conv, const int8_t* x, void* y, int batch);
/* Test hook: the raw int32 accumulators, NCHW [batch,cout,ho,wo] (bit-exact check). */
int plb_conv_acc_i32(plb_conv* conv, const int8_t* x, int32_t* acc, int batch);
/* conv (fp32 value, no activation of its own) + fp32 residual + ReLU, then optionally the
 * calib fp32->int8 step of the next layer, in one pass.  NHWC.  Fuses what the reference
 * graph runs as conv(fp32_out) -> elementwise_add -> relu -> calib
 * (lite/backends/x86/math/calib.cc:25-151 for the last step).
 *   residual [batch,ho,wo,cout] float (nullable = no add)
 *   y_f32    [batch,ho,wo,cout] float (nullable = not stored)
 *   y_i8     [batch,ho,wo,cout] int8  (nullable = not stored), q = calib(y, next_scale) */
int plb_conv_run_nhwc_add_relu(plb_conv* conv, const int8_t* x, const float* residual,
                               float* y_f32, int8_t* y_i8, float next_scale, int batch);
/* A whole projection block tail in one launch: y = relu(conv(x) + shortcut(x_shortcut)), where both
 * are unpadded 1x1 convolutions with the same output shape (the shortcut may have a stride) and no
 * activation of their own, i.e. the reference sequence  conv2d(fp32_out) [main], conv2d(fp32_out)
 * [shortcut], elementwise_add + relu, calib  with the shortcut's fp32 tensor never written.  The
 * shortcut value is fma(acc2, ws2*in_s2, bias2) exactly as its own fp32_out kernel computes it, so
 * the outputs are bit-identical to the unfused sequence.  Both layers prepared with
 * out_dtype = PLB_OUT_F32 on the same ctx; x and x_shortcut channels-last.  A graph-level fusion of
 * the kind the reference's MIR fusion passes perform; it has no single-kernel counterpart there. */
int plb_conv_run_nhwc_block_add_relu(plb_conv* conv, const int8_t* x, plb_conv* shortcut, const int8_t* x_shortcut,
                                     float* y_f32, int8_t* y_i8, float next_scale, int batch);
/* A depthwise 3x3 layer and the 1x1 layer that consumes it in one launch (a MobileNet block): the int8
 * tensor between them is produced in shared memory as the tensor-core operand and never written, so the
 * pair reads x and writes y and nothing else.  Arithmetic of the two-kernel sequence  depthwise_conv2d
 * (int8_out) -> conv2d (int8_out)  bit for bit (lite/kernels/x86/conv_compute.cc:216-341 run twice).
 * `dw` prepared with groups == cin == cout, 3x3, stride 1 or 2, int8 out, activation none / relu / relu6,
 * 32 / 64 / 128 / 256 channels; `pw` an unpadded 1x1 layer on the depthwise output, int8 out, 32 .. 512
 * output channels (a power of two), its filter small enough to stay in shared memory; both on the same
 * ctx; x [batch,h,w,c], y [batch,ho,wo,cout] channels-last.  plb_conv_dwpw_fusable() tells whether a pair
 * qualifies (1) or the two layers have to be run one after the other (0); the run call returns
 * PLB_E_UNSUPPORTED for a pair that does not.  A graph-level fusion beyond the reference's fusion passes
 * (lite/core/optimizer/mir/fusion/): it has no counterpart there. */
int plb_conv_dwpw_fusable(const plb_conv* dw, const plb_conv* pw);
int plb_conv_run_nhwc_dwpw(plb_conv* dw, plb_conv* pw, const int8_t* x, int8_t* y, int batch);
int plb_conv_out_dims(const plb_conv* conv, int* ho, int* wo);
/* A prepared layer keeps the tile plan and the TMA descriptors of the (batch, pointers) it has been
 * run on, so that a repeated Run() costs one kernel launch on the host (the reference re-derives
 * nothing per Run either: its GEMM objects are built in PrepareForRun, conv_compute.cc:271-288).
 * Returns how many runs of this layer re-used a stored plan.  Test hook. */
long plb_conv_plan_cache_hits(const plb_conv* conv);
void plb_conv_destroy(plb_conv* conv);

/* ------------------------------------------------------------------ fc
 * = FcCompute<kInt8,*> (lite/kernels/x86/fc_compute.cc:176-269) with scale and bias
 * indexed by output feature as lite/kernels/arm/fc_compute.cc:207-260 defines it.
 * w_h is FcParam::w, [K,N] row-major int8 on the host; n_wscale is 1 or N. */
int plb_fc_prepare(plb_ctx* ctx, int k, int n, int act, float act_alpha, float in_scale,
                   float out_scale, int out_dtype, const int8_t* w_h, const float* wscale_h,
                   int n_wscale, const float* bias_h /* nullable */, plb_fc** out);
/* x [m,k] int8, y [m,n] float or int8. */
int plb_fc_run(plb_fc* fc, const int8_t* x, void* y, int m);
int plb_fc_acc_i32(plb_fc* fc, const int8_t* x, int32_t* acc, int m);
void plb_fc_destroy(plb_fc* fc);

/* ------------------------------------------------------------------ sparse_conv2d (1x1)
 * = SparseConvCompute<*> (lite/kernels/arm/sparse_conv_compute.cc:33-267) over the encoding
 * built by sparse_conv_detect_pass (lite/core/optimizer/mir/sparse_conv_detect_pass.cc:35-301):
 *   nonzero_weights_h  SparseConvParam::nonzero_weights (int8 or float), n_weights entries
 *   oc_nonzeros_h      SparseConvParam::oc_nonzeros, [cout] cumulative counts
 *   diffs_h            SparseConvParam::diffs, byte offsets scaled by hw = ho*wo
 *   first_ic, flag_semi  the attributes of the same names
 * is_int8 == 0 is the fp32 kernel (alias def: fp32 in, fp32 out; weights padded to
 * multiples of 4 per channel unless flag_semi); is_int8 != 0 takes int8 input and
 * out_dtype picks int8_fp32_out / int8_int8_out.  The batch dimension is honoured. */
typedef struct plb_sparse_desc {
  int cin, cout, h, w;
  int is_int8;
  int out_dtype;
  int flag_semi, first_ic;
  int act;
  float act_alpha;
  float in_scale, out_scale;
  int leaky_compat;
  int impl; /* PLB_IMPL_AUTO (int8 with >= 32 channels: densified, else walk) | PLB_IMPL_DIRECT (walk the encoding) | PLB_IMPL_TC (densified) */
} plb_sparse_desc;
int plb_sparse_prepare(plb_ctx* ctx, const plb_sparse_desc* desc, const void* nonzero_weights_h,
                       int n_weights, const uint32_t* oc_nonzeros_h, const int32_t* diffs_h,
                       int n_diffs, const float* wscale_h, int n_wscale,
                       const float* bias_h /* nullable */, plb_sparse** out);
/* x [batch,cin,h,w] (int8 or float), y [batch,cout,h,w] (float or int8), NCHW. */
int plb_sparse_run(plb_sparse* sp, const void* x, void* y, int batch);
void plb_sparse_destroy(plb_sparse* sp);

/* ------------------------------------------------------------------ glue between int8 layers
 * calib fp32 -> int8 (lite/backends/x86/math/calib.cc:25-151): q = sat(rne(max(x/scale,-127))). */
int plb_calib_f32_to_i8(plb_ctx* ctx, const float* x, int8_t* q, size_t n, float scale);
/* calib int8 -> fp32 (calib.cc:153-239). */
int plb_calib_i8_to_f32(plb_ctx* ctx, const int8_t* q, float* y, size_t n, float scale);
/* Host <-> device copies on the ctx stream: what the io_copy kernels of a target do with
 * TargetWrapper<T>::MemcpySync (lite/kernels/xpu/io_copy_compute.cc:54-116, CopySync in
 * lite/core/memory.h:65-93).  h2d is enqueued (the host buffer must stay valid until the stream
 * reaches it; pinned memory makes it asynchronous), d2h returns when the bytes are on the host, or
 * PLB_E_DEVICE when a kernel in front of the copy recorded a fault (the bytes are then garbage). */
int plb_copy_h2d(plb_ctx* ctx, void* dst_device, const void* src_host, size_t bytes);
int plb_copy_d2h(plb_ctx* ctx, void* dst_host, const void* src_device, size_t bytes);
/* layout staging: [n,c,h,w] <-> [n,h,w,cpad] (extra channels are zero / dropped). */
int plb_nchw_to_nhwc_i8(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w,
                        int cpad);
int plb_nhwc_to_nchw(plb_ctx* ctx, const void* x, void* y, int n, int c, int h, int w,
                     int elem_bytes);
/* fp32 NCHW image -> int8 NHWC with cpad channels: calib and layout staging in one pass. */
int plb_calib_nchw_f32_to_nhwc_i8(plb_ctx* ctx, const float* x, int8_t* y, int n, int c, int h,
                                  int w, int cpad, float scale);
/* max pooling on int8 NHWC, square window, symmetric padding (pool2d, max). */
int plb_maxpool_nhwc_i8(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w,
                        int k, int stride, int pad);
/* global average pool of fp32 NHWC [n,h*w,c] -> [n,c], then calib to int8 when q != NULL. */
int plb_global_avgpool_nhwc_f32(plb_ctx* ctx, const float* x, float* y, int8_t* q, int n, int hw,
                                int c, float scale);
/* softmax over the last axis of a [rows, cols] fp32 matrix (the classifier head after fc):
 * y = exp(max(x - rowmax, -64)) / sum, the shift-and-clip form of
 * lite/backends/x86/math/softmax_impl.h:36-41, :110-131 (axis = last, num_remain = 1). */
int plb_softmax_f32(plb_ctx* ctx, const float* x, float* y, int rows, int cols);

#ifdef __cplusplus
}
#endif
#endif /* PLB200_H_ */
