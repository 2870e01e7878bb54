// Paddle-Lite kernels of the new target: `kCUDA` / `kInt8` / `kNCHW` conv2d,
// depthwise_conv2d, fc and sparse_conv2d implemented on the plb200 C ABI.
//
// This file is compiled AGAINST THE REFERENCE HEADERS (it is the code a maintainer adds to
// the reference tree as lite/kernels/cuda/int8_kernels.cc); it registers through the
// reference's own REGISTER_LITE_KERNEL macro (lite/core/op_registry.h:268-291), takes its
// parameters from operators::ConvParam / FcParam / SparseConvParam
// (lite/operators/op_params.h:403-455, :100-118, :373-400) and follows the life cycle of
// KernelBase::Launch (lite/core/kernel.h:84-124): PrepareForRun() once, then Run().
// Registration names, aliases and tensor bindings mirror the x86 int8 kernels
// (lite/kernels/x86/conv_compute.cc:509-553, lite/kernels/x86/fc_compute.cc:296-308) and the
// ARM sparse kernels (lite/kernels/arm/sparse_conv_compute.cc:393-430).
//
// Tensors handed to these kernels hold DEVICE memory (TargetType::kCUDA buffers, e.g. wrapped
// with lite::Buffer(void*, TargetType, size_t), lite/core/memory.h:98-99); filters, scales
// and biases are read on the host at PrepareForRun, exactly like the x86 kernels do.
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <utility>
#include <vector>

#include "include/plb200.h"
#include "lite/core/kernel.h"
#include "lite/core/op_registry.h"
#include "lite/operators/op_params.h"

namespace paddle {
namespace lite {
namespace kernels {
namespace cuda {

// Which device and stream a kernel runs on.  The reference keeps both in Context<TARGET>, created per
// predictor by ContextScheduler (lite/core/context.h:430-484) and handed to the kernel through
// KernelBase::SetContext (lite/core/kernel.h:133-136).  In a tree that has Context<TargetType::kCUDA> (the patch
// kcuda_target.patch next to this file, built with -DLITE_WITH_CUDA) the binding is read from there; otherwise from a per-thread
// binding that the host sets with SetPlbBinding() before it prepares a predictor on that thread (what
// PaddlePredictor::SetStream(TargetType, void*), lite/api/paddle_api.h:141, forwards to).  A kernel instance
// looks its plb_ctx up once, in PrepareForRun, and keeps it: two predictors on different devices, streams or
// threads never share a context, a workspace or a status word.
struct PlbBinding {
  int device = 0;
  void* stream = nullptr;
};
inline PlbBinding& ThreadBinding() {
  static thread_local PlbBinding b;
  return b;
}
inline void SetPlbBinding(int device, void* stream) {
  ThreadBinding().device = device;
  ThreadBinding().stream = stream;
}
#define PLB_CHECK(call) CHECK_EQ((call), PLB_OK) << plb_last_error()

inline plb_ctx* CtxFor(int device, void* stream) {
  static std::mutex mu;
  static std::map<std::pair<int, void*>, plb_ctx*> table;  // contexts live as long as the process
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_pair(device, stream);
  auto it = table.find(key);
  if (it != table.end()) return it->second;
  plb_ctx* ctx = nullptr;
  PLB_CHECK(plb_ctx_create(device, stream, &ctx));
  table[key] = ctx;
  return ctx;
}

template <typename Kernel>
inline plb_ctx* CtxOf(Kernel* kernel) {
#ifdef LITE_WITH_CUDA
  auto& c = kernel->mutable_context()->template As<CUDAContext>();
  return CtxFor(c.device_id(), c.exec_stream());
#else
  (void)kernel;
  return CtxFor(ThreadBinding().device, ThreadBinding().stream);
#endif
}

// relu_type of the int8 kernels.  `strict` (sparse_conv2d): the ARM reference applies every activation the fuse
// pass may hand it, hard_swish included (lite/kernels/arm/sparse_conv_compute.cc:91-100); this target implements
// relu / relu6 / leaky_relu, so anything else must stop the program rather than run without activation.  conv2d /
// depthwise_conv2d mirror the x86 int8 kernel, which leaves relu_type 0 for other types
// (lite/kernels/x86/conv_compute.cc:257-270).
inline int ActCode(const operators::ActivationParam& act, float* alpha, bool strict = false) {
  *alpha = 0.f;
  if (!act.has_active) return PLB_ACT_NONE;
  switch (act.active_type) {
    case lite_api::ActivationType::kRelu:
      return PLB_ACT_RELU;
    case lite_api::ActivationType::kRelu6:
      *alpha = act.Relu_clipped_coef;
      return PLB_ACT_RELU6;
    case lite_api::ActivationType::kLeakyRelu:
      *alpha = act.Leaky_relu_alpha;
      return PLB_ACT_LEAKY;
    default:
      if (strict) {
        // builds without LITE_WITH_LOG abort silently on LOG(FATAL): say why first
        std::fprintf(stderr, "sparse_conv2d on kCUDA: activation type %d (e.g. hard_swish) is not implemented; "
                             "supported: relu, relu6, leaky_relu\n", static_cast<int>(act.active_type));
        LOG(FATAL) << "sparse_conv2d on kCUDA: unsupported activation type " << static_cast<int>(act.active_type);
      }
      return PLB_ACT_NONE;
  }
}

template <PrecisionType OutType>
class ConvInt8Compute : public KernelLite<TARGET(kCUDA), PRECISION(kInt8)> {
 public:
  using param_t = operators::ConvParam;

  void PrepareForRun() override {
    auto& param = this->Param<param_t>();
    auto x_dims = param.x->dims();
    auto w_dims = param.filter->dims();
    auto paddings = *param.paddings;
    auto dilations = *param.dilations;
    plb_conv_desc d{};
    d.cin = x_dims[1];
    d.h = x_dims[2];
    d.w = x_dims[3];
    d.cout = w_dims[0];
    d.kh = w_dims[2];
    d.kw = w_dims[3];
    d.stride_h = param.strides[0];
    d.stride_w = param.strides[1];
    d.pad_top = paddings[0];
    d.pad_bottom = paddings[1];
    d.pad_left = paddings[2];
    d.pad_right = paddings[3];
    d.dil_h = dilations[0];
    d.dil_w = dilations[1];
    d.groups = param.groups;
    d.act = ActCode(param.activation_param, &d.act_alpha);
    d.in_scale = param.input_scale;
    d.out_scale = param.output_scale;
    d.out_dtype = OutType == PRECISION(kInt8) ? PLB_OUT_I8 : PLB_OUT_F32;
    d.leaky_compat = 1;  // the drop-in reproduces conv_compute.cc:394
    d.impl = PLB_IMPL_AUTO;
    const float* bias = param.bias ? param.bias->template data<float>() : nullptr;
    plb_conv* conv = nullptr;
    PLB_CHECK(plb_conv_prepare(CtxOf(this), &d, param.filter->template data<int8_t>(),
                               param.weight_scale.data(), static_cast<int>(param.weight_scale.size()),
                               bias, &conv));
    conv_.reset(conv);
    in_c_ = d.cin;
    in_h_ = d.h;
    in_w_ = d.w;
  }

  void ReInitWhenNeeded() override {
    // A prepared layer is bound to its input channels / height / width (the batch is given per run); re-plan
    // when they change.  (The x86 kernel freezes them at the first PrepareForRun, conv_compute.cc:225-228.)
    auto x_dims = this->Param<param_t>().x->dims();
    if (conv_ && (x_dims[1] != in_c_ || x_dims[2] != in_h_ || x_dims[3] != in_w_)) PrepareForRun();
  }

  void Run() override {
    auto& param = this->Param<param_t>();
    const int batch = param.x->dims()[0];
    void* out = OutType == PRECISION(kInt8)
                    ? static_cast<void*>(param.output->template mutable_data<int8_t>(TARGET(kCUDA)))
                    : static_cast<void*>(param.output->template mutable_data<float>(TARGET(kCUDA)));
    PLB_CHECK(plb_conv_run(conv_.get(), param.x->template data<int8_t>(), out, batch));
  }

 private:
  struct Deleter {
    void operator()(plb_conv* p) const { plb_conv_destroy(p); }
  };
  std::unique_ptr<plb_conv, Deleter> conv_;
  int64_t in_c_{0}, in_h_{0}, in_w_{0};
};

// The same layer on channels-last tensors (DATALAYOUT(kNHWC)).  Registered next to the NCHW
// kernels so that the reference's own type_layout_cast_pass
// (lite/core/optimizer/mir/type_layout_cast_pass.cc) inserts `layout` ops at the edges of a run
// of these kernels only, and consecutive int8 layers exchange NHWC tensors without any staging.
template <PrecisionType OutType>
class ConvInt8NhwcCompute : public KernelLite<TARGET(kCUDA), PRECISION(kInt8), DATALAYOUT(kNHWC)> {
 public:
  using param_t = operators::ConvParam;

  void PrepareForRun() override {
    auto& param = this->Param<param_t>();
    auto x_dims = param.x->dims();  // the op keeps logical NCHW dims; only the memory is channels-last
    auto w_dims = param.filter->dims();
    auto paddings = *param.paddings;
    auto dilations = *param.dilations;
    plb_conv_desc d{};
    d.cin = x_dims[1];
    d.h = x_dims[2];
    d.w = x_dims[3];
    d.cout = w_dims[0];
    d.kh = w_dims[2];
    d.kw = w_dims[3];
    d.stride_h = param.strides[0];
    d.stride_w = param.strides[1];
    d.pad_top = paddings[0];
    d.pad_bottom = paddings[1];
    d.pad_left = paddings[2];
    d.pad_right = paddings[3];
    d.dil_h = dilations[0];
    d.dil_w = dilations[1];
    d.groups = param.groups;
    d.act = ActCode(param.activation_param, &d.act_alpha);
    d.in_scale = param.input_scale;
    d.out_scale = param.output_scale;
    d.out_dtype = OutType == PRECISION(kInt8) ? PLB_OUT_I8 : PLB_OUT_F32;
    d.leaky_compat = 1;
    d.impl = PLB_IMPL_AUTO;
    const float* bias = param.bias ? param.bias->template data<float>() : nullptr;
    plb_conv* conv = nullptr;
    PLB_CHECK(plb_conv_prepare(CtxOf(this), &d, param.filter->template data<int8_t>(),
                               param.weight_scale.data(), static_cast<int>(param.weight_scale.size()),
                               bias, &conv));
    conv_.reset(conv);
    in_c_ = d.cin;
    in_h_ = d.h;
    in_w_ = d.w;
  }

  void ReInitWhenNeeded() override {
    auto x_dims = this->Param<param_t>().x->dims();
    if (conv_ && (x_dims[1] != in_c_ || x_dims[2] != in_h_ || x_dims[3] != in_w_)) PrepareForRun();
  }

  void Run() override {
    auto& param = this->Param<param_t>();
    const int batch = param.x->dims()[0];
    void* out = OutType == PRECISION(kInt8)
                    ? static_cast<void*>(param.output->template mutable_data<int8_t>(TARGET(kCUDA)))
                    : static_cast<void*>(param.output->template mutable_data<float>(TARGET(kCUDA)));
    PLB_CHECK(plb_conv_run_nhwc(conv_.get(), param.x->template data<int8_t>(), out, batch));
  }

 private:
  struct Deleter {
    void operator()(plb_conv* p) const { plb_conv_destroy(p); }
  };
  std::unique_ptr<plb_conv, Deleter> conv_;
  int64_t in_c_{0}, in_h_{0}, in_w_{0};
};

template <PrecisionType OutType>
class FcInt8Compute : public KernelLite<TARGET(kCUDA), PRECISION(kInt8)> {
 public:
  using param_t = operators::FcParam;

  void PrepareForRun() override {
    auto& param = this->Param<param_t>();
    auto w_dims = param.w->dims();
    const int k = w_dims[0], n = w_dims[1];
    int act = PLB_ACT_NONE;
    float alpha = 0.f;
    if (param.activation_type == "relu") act = PLB_ACT_RELU;
    if (param.activation_type == "relu6") {
      act = PLB_ACT_RELU6;
      alpha = param.alpha;
    }
    const float* bias = param.bias ? param.bias->template data<float>() : nullptr;
    plb_fc* fc = nullptr;
    PLB_CHECK(plb_fc_prepare(CtxOf(this), k, n, act, alpha, param.input_scale, param.output_scale,
                             OutType == PRECISION(kInt8) ? PLB_OUT_I8 : PLB_OUT_F32,
                             param.w->template data<int8_t>(), param.weight_scale.data(),
                             static_cast<int>(param.weight_scale.size()), bias, &fc));
    fc_.reset(fc);
  }

  void Run() override {
    auto& param = this->Param<param_t>();
    const int m = param.input->dims().count(0, param.in_num_col_dims);
    void* out = OutType == PRECISION(kInt8)
                    ? static_cast<void*>(param.output->template mutable_data<int8_t>(TARGET(kCUDA)))
                    : static_cast<void*>(param.output->template mutable_data<float>(TARGET(kCUDA)));
    PLB_CHECK(plb_fc_run(fc_.get(), param.input->template data<int8_t>(), out, m));
  }

 private:
  struct Deleter {
    void operator()(plb_fc* p) const { plb_fc_destroy(p); }
  };
  std::unique_ptr<plb_fc, Deleter> fc_;
};

template <PrecisionType InType, PrecisionType OutType>
class SparseConvCompute : public KernelLite<TARGET(kCUDA), InType> {
 public:
  using param_t = operators::SparseConvParam;

  void PrepareForRun() override {
    auto& param = this->template Param<param_t>();
    auto x_dims = param.x->dims();
    plb_sparse_desc d{};
    d.cin = x_dims[1];
    d.h = x_dims[2];
    d.w = x_dims[3];
    d.cout = param.oc_nonzeros->dims()[0];
    d.is_int8 = InType == PRECISION(kInt8);
    d.out_dtype = OutType == PRECISION(kInt8) ? PLB_OUT_I8 : PLB_OUT_F32;
    d.flag_semi = param.flag_semi;
    d.first_ic = param.first_ic;
    d.act = ActCode(param.activation_param, &d.act_alpha, /*strict=*/true);
    d.in_scale = param.input_scale;
    d.out_scale = param.output_scale;
    d.leaky_compat = 1;  // sparse_conv_compute.cc:86-90 divides the slope as well
    d.impl = PLB_IMPL_AUTO;
    const void* nz = d.is_int8 ? static_cast<const void*>(param.nonzero_weights->template data<int8_t>())
                               : static_cast<const void*>(param.nonzero_weights->template data<float>());
    const float* bias = param.bias ? param.bias->template data<float>() : nullptr;
    plb_sparse* sp = nullptr;
    PLB_CHECK(plb_sparse_prepare(CtxOf(this), &d, nz, static_cast<int>(param.nonzero_weights->numel()),
                                 param.oc_nonzeros->template data<uint32_t>(),
                                 param.diffs->template data<int32_t>(),
                                 static_cast<int>(param.diffs->numel()), param.weight_scale.data(),
                                 static_cast<int>(param.weight_scale.size()), bias, &sp));
    sp_.reset(sp);
    in_c_ = d.cin;
    in_h_ = d.h;
    in_w_ = d.w;
  }

  void ReInitWhenNeeded() override {
    // diffs are byte offsets scaled by H*W, so the encoding itself belongs to one image size; a graph that
    // changes it re-runs the detect pass and hands this kernel new tensors
    auto x_dims = this->template Param<param_t>().x->dims();
    if (sp_ && (x_dims[1] != in_c_ || x_dims[2] != in_h_ || x_dims[3] != in_w_)) PrepareForRun();
  }

  void Run() override {
    auto& param = this->template Param<param_t>();
    const int batch = param.x->dims()[0];
    const void* x = InType == PRECISION(kInt8) ? static_cast<const void*>(param.x->template data<int8_t>())
                                               : static_cast<const void*>(param.x->template data<float>());
    void* out = OutType == PRECISION(kInt8)
                    ? static_cast<void*>(param.output->template mutable_data<int8_t>(TARGET(kCUDA)))
                    : static_cast<void*>(param.output->template mutable_data<float>(TARGET(kCUDA)));
    PLB_CHECK(plb_sparse_run(sp_.get(), x, out, batch));
  }

 private:
  struct Deleter {
    void operator()(plb_sparse* p) const { plb_sparse_destroy(p); }
  };
  std::unique_ptr<plb_sparse, Deleter> sp_;
  int64_t in_c_{0}, in_h_{0}, in_w_{0};
};

// calib fp32 <-> int8 between layers (mirrors lite/kernels/x86/calib_compute.cc:28-36, :156-168;
// operators::CalibParam, lite/operators/op_params.h:74-78).
class CalibFp32ToInt8Compute : public KernelLite<TARGET(kCUDA), PRECISION(kInt8)> {
 public:
  void PrepareForRun() override { plb_ = CtxOf(this); }
  void Run() override {
    auto& param = this->Param<operators::CalibParam>();
    PLB_CHECK(plb_calib_f32_to_i8(plb_, param.input->template data<float>(),
                                  param.output->template mutable_data<int8_t>(TARGET(kCUDA)),
                                  static_cast<size_t>(param.input->numel()), param.scale));
  }

 private:
  plb_ctx* plb_{nullptr};
};
class CalibInt8ToFp32Compute : public KernelLite<TARGET(kCUDA), PRECISION(kInt8)> {
 public:
  void PrepareForRun() override { plb_ = CtxOf(this); }
  void Run() override {
    auto& param = this->Param<operators::CalibParam>();
    PLB_CHECK(plb_calib_i8_to_f32(plb_, param.input->template data<int8_t>(),
                                  param.output->template mutable_data<float>(TARGET(kCUDA)),
                                  static_cast<size_t>(param.input->numel()), param.scale));
  }

 private:
  plb_ctx* plb_{nullptr};
};

// softmax over the last axis of an fp32 tensor (classifier head; operators::SoftmaxParam,
// lite/operators/op_params.h:292-297; x86 kernel lite/kernels/x86/softmax_compute.h).
class SoftmaxCompute : public KernelLite<TARGET(kCUDA), PRECISION(kFloat)> {
 public:
  void PrepareForRun() override { plb_ = CtxOf(this); }
  void Run() override {
    auto& param = this->Param<operators::SoftmaxParam>();
    auto dims = param.x->dims();
    const int rank = static_cast<int>(dims.size());
    const int axis = param.axis < 0 ? param.axis + rank : param.axis;
    CHECK_EQ(axis, rank - 1) << "the kCUDA softmax kernel handles the last axis";
    const int cols = static_cast<int>(dims[rank - 1]);
    const int rows = static_cast<int>(dims.production() / cols);
    PLB_CHECK(plb_softmax_f32(plb_, param.x->template data<float>(),
                              param.output->template mutable_data<float>(TARGET(kCUDA)), rows, cols));
  }

 private:
  plb_ctx* plb_{nullptr};
};

// io_copy host <-> device (mirrors lite/kernels/xpu/io_copy_compute.cc:54-116; operators::IoCopyParam,
// lite/operators/op_params.h:60-66).  The destination keeps the source's dims, precision and LoD.
class IoCopyHostToCudaCompute : public KernelLite<TARGET(kCUDA), PRECISION(kAny), DATALAYOUT(kAny)> {
 public:
  void PrepareForRun() override { plb_ = CtxOf(this); }
  void Run() override {
    auto& param = this->Param<operators::IoCopyParam>();
    CHECK(param.x != nullptr && param.y != nullptr) << "io_copy handles single tensors";
    const size_t bytes = param.x->memory_size();
    param.y->Resize(param.x->dims());
    param.y->set_precision(param.x->precision());
    param.y->set_lod(param.x->lod());
    void* dst = param.y->mutable_data(TARGET(kCUDA), bytes);
    PLB_CHECK(plb_copy_h2d(plb_, dst, param.x->raw_data(), bytes));
  }

 private:
  plb_ctx* plb_{nullptr};
};
class IoCopyCudaToHostCompute : public KernelLite<TARGET(kCUDA), PRECISION(kAny), DATALAYOUT(kAny)> {
 public:
  void PrepareForRun() override { plb_ = CtxOf(this); }
  void Run() override {
    auto& param = this->Param<operators::IoCopyParam>();
    CHECK(param.x != nullptr && param.y != nullptr) << "io_copy handles single tensors";
    const size_t bytes = param.x->memory_size();
    param.y->Resize(param.x->dims());
    param.y->set_precision(param.x->precision());
    param.y->set_lod(param.x->lod());
    void* dst = param.y->mutable_data(TARGET(kHost), bytes);
    PLB_CHECK(plb_copy_d2h(plb_, dst, param.x->raw_data(), bytes));
  }

 private:
  plb_ctx* plb_{nullptr};
};

}  // namespace cuda
}  // namespace kernels
}  // namespace lite
}  // namespace paddle

namespace plbk = paddle::lite::kernels::cuda;
typedef plbk::ConvInt8Compute<PRECISION(kInt8)> CudaConvInt8_Int8;
typedef plbk::ConvInt8Compute<PRECISION(kFloat)> CudaConvInt8_Fp32;
typedef plbk::FcInt8Compute<PRECISION(kInt8)> CudaFcInt8_Int8;
typedef plbk::FcInt8Compute<PRECISION(kFloat)> CudaFcInt8_Fp32;
typedef plbk::SparseConvCompute<PRECISION(kFloat), PRECISION(kFloat)> CudaSparseConvFp32;
typedef plbk::SparseConvCompute<PRECISION(kInt8), PRECISION(kFloat)> CudaSparseConvInt8Fp32;
typedef plbk::SparseConvCompute<PRECISION(kInt8), PRECISION(kInt8)> CudaSparseConvInt8Int8;

#define PLB_T(prec) LiteType::GetTensorTy(TARGET(kCUDA), PRECISION(prec))

REGISTER_LITE_KERNEL(conv2d, kCUDA, kInt8, kNCHW, CudaConvInt8_Int8, int8_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("SecondInput", {PLB_T(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_T(kInt8)})
    .BindPaddleOpVersion("conv2d", 1)
    .Finalize();

REGISTER_LITE_KERNEL(conv2d, kCUDA, kInt8, kNCHW, CudaConvInt8_Fp32, fp32_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("SecondInput", {PLB_T(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_T(kFloat)})
    .BindPaddleOpVersion("conv2d", 1)
    .Finalize();

typedef plbk::ConvInt8NhwcCompute<PRECISION(kInt8)> CudaConvInt8Nhwc_Int8;
typedef plbk::ConvInt8NhwcCompute<PRECISION(kFloat)> CudaConvInt8Nhwc_Fp32;
#define PLB_TN(prec) LiteType::GetTensorTy(TARGET(kCUDA), PRECISION(prec), DATALAYOUT(kNHWC))

REGISTER_LITE_KERNEL(conv2d, kCUDA, kInt8, kNHWC, CudaConvInt8Nhwc_Int8, int8_out_nhwc)
    .BindInput("Input", {PLB_TN(kInt8)})
    .BindInput("SecondInput", {PLB_TN(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_TN(kInt8)})
    .BindPaddleOpVersion("conv2d", 1)
    .Finalize();

REGISTER_LITE_KERNEL(conv2d, kCUDA, kInt8, kNHWC, CudaConvInt8Nhwc_Fp32, fp32_out_nhwc)
    .BindInput("Input", {PLB_TN(kInt8)})
    .BindInput("SecondInput", {PLB_TN(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_TN(kFloat)})
    .BindPaddleOpVersion("conv2d", 1)
    .Finalize();

REGISTER_LITE_KERNEL(depthwise_conv2d, kCUDA, kInt8, kNHWC, CudaConvInt8Nhwc_Int8, int8_out_nhwc)
    .BindInput("Input", {PLB_TN(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_TN(kInt8)})
    .BindPaddleOpVersion("depthwise_conv2d", 1)
    .Finalize();

REGISTER_LITE_KERNEL(depthwise_conv2d, kCUDA, kInt8, kNCHW, CudaConvInt8_Int8, int8_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_T(kInt8)})
    .BindPaddleOpVersion("depthwise_conv2d", 1)
    .Finalize();

REGISTER_LITE_KERNEL(depthwise_conv2d, kCUDA, kInt8, kNCHW, CudaConvInt8_Fp32, fp32_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("Filter", {PLB_T(kInt8)})
    .BindOutput("Output", {PLB_T(kFloat)})
    .BindPaddleOpVersion("depthwise_conv2d", 1)
    .Finalize();

REGISTER_LITE_KERNEL(fc, kCUDA, kInt8, kNCHW, CudaFcInt8_Int8, int8_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("W", {PLB_T(kInt8)})
    .BindOutput("Out", {PLB_T(kInt8)})
    .Finalize();

REGISTER_LITE_KERNEL(fc, kCUDA, kInt8, kNCHW, CudaFcInt8_Fp32, fp32_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindInput("W", {PLB_T(kInt8)})
    .BindOutput("Out", {PLB_T(kFloat)})
    .Finalize();

REGISTER_LITE_KERNEL(sparse_conv2d, kCUDA, kFloat, kNCHW, CudaSparseConvFp32, def)
    .BindInput("Input", {PLB_T(kFloat)})
    .BindInput("NonZeroWeights", {PLB_T(kFloat)})
    .BindInput("OcNonZeros", {PLB_T(kInt32)})
    .BindInput("Diffs", {PLB_T(kInt32)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindOutput("Output", {PLB_T(kFloat)})
    .Finalize();

REGISTER_LITE_KERNEL(sparse_conv2d, kCUDA, kInt8, kNCHW, CudaSparseConvInt8Fp32, int8_fp32_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("NonZeroWeights", {PLB_T(kInt8)})
    .BindInput("OcNonZeros", {PLB_T(kInt32)})
    .BindInput("Diffs", {PLB_T(kInt32)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindOutput("Output", {PLB_T(kFloat)})
    .Finalize();

REGISTER_LITE_KERNEL(sparse_conv2d, kCUDA, kInt8, kNCHW, CudaSparseConvInt8Int8, int8_int8_out)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindInput("NonZeroWeights", {PLB_T(kInt8)})
    .BindInput("OcNonZeros", {PLB_T(kInt32)})
    .BindInput("Diffs", {PLB_T(kInt32)})
    .BindInput("Bias", {PLB_T(kFloat)})
    .BindOutput("Output", {PLB_T(kInt8)})
    .Finalize();

// calib between fp32 and int8 layers (x86 registrations: lite/kernels/x86/calib_compute.cc:153-168)
REGISTER_LITE_KERNEL(calib, kCUDA, kInt8, kNCHW, plbk::CalibFp32ToInt8Compute, fp32_to_int8)
    .BindInput("Input", {PLB_T(kFloat)})
    .BindOutput("Out", {PLB_T(kInt8)})
    .Finalize();
REGISTER_LITE_KERNEL(calib, kCUDA, kInt8, kNCHW, plbk::CalibInt8ToFp32Compute, int8_to_fp32)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindOutput("Out", {PLB_T(kFloat)})
    .Finalize();
REGISTER_LITE_KERNEL(calib_once, kCUDA, kInt8, kNCHW, plbk::CalibFp32ToInt8Compute, fp32_to_int8)
    .BindInput("Input", {PLB_T(kFloat)})
    .BindOutput("Out", {PLB_T(kInt8)})
    .Finalize();
REGISTER_LITE_KERNEL(calib_once, kCUDA, kInt8, kNCHW, plbk::CalibInt8ToFp32Compute, int8_to_fp32)
    .BindInput("Input", {PLB_T(kInt8)})
    .BindOutput("Out", {PLB_T(kFloat)})
    .Finalize();

// host <-> device copies (XPU registrations: lite/kernels/xpu/io_copy_compute.cc:175-269)
#define PLB_ANY(target) LiteType::GetTensorTy(TARGET(target), PRECISION(kAny), DATALAYOUT(kAny))
REGISTER_LITE_KERNEL(io_copy, kCUDA, kAny, kAny, plbk::IoCopyHostToCudaCompute, host_to_device)
    .BindInput("Input", {PLB_ANY(kHost)})
    .BindOutput("Out", {PLB_ANY(kCUDA)})
    .Finalize();
REGISTER_LITE_KERNEL(io_copy, kCUDA, kAny, kAny, plbk::IoCopyCudaToHostCompute, device_to_host)
    .BindInput("Input", {PLB_ANY(kCUDA)})
    .BindOutput("Out", {PLB_ANY(kHost)})
    .Finalize();
REGISTER_LITE_KERNEL(io_copy_once, kCUDA, kAny, kAny, plbk::IoCopyHostToCudaCompute, host_to_device)
    .BindInput("Input", {PLB_ANY(kHost)})
    .BindOutput("Out", {PLB_ANY(kCUDA)})
    .Finalize();
REGISTER_LITE_KERNEL(io_copy_once, kCUDA, kAny, kAny, plbk::IoCopyCudaToHostCompute, device_to_host)
    .BindInput("Input", {PLB_ANY(kCUDA)})
    .BindOutput("Out", {PLB_ANY(kHost)})
    .Finalize();

REGISTER_LITE_KERNEL(softmax, kCUDA, kFloat, kNCHW, plbk::SoftmaxCompute, def)
    .BindInput("X", {PLB_T(kFloat)})
    .BindOutput("Out", {PLB_T(kFloat)})
    .Finalize();
