// Drop-in probe (test driver): drives every kernel the new kCUDA target registers the way the reference
// drives its own (lite/tests/math/x86_conv_int8_compute_test.cc:156-198): the kernel object comes out of the
// reference's KernelRegistry, receives an operators::*Param whose activation tensors wrap device memory, and
// runs through KernelBase::Launch().  Results are compared on the host with plain exact loops (and, for
// sparse_conv2d, with tensors produced by the restated weight encoder of the test oracle).  Built against the
// reference headers and linked with a handful of the reference's core objects; runs on an sm_100 GPU.
//
//   lite_target_probe                 all checks; prints "PROBE OK"
//   lite_target_probe --hard-swish    a sparse_conv2d with hard_swish: must die with LOG(FATAL), not compute
//   lite_target_probe --time          also times a three-layer chain through Launch(), NHWC and NCHW kernels
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "lite/core/kernel.h"
#include "lite/core/op_registry.h"
#include "lite/core/tensor.h"
#include "lite/operators/op_params.h"

extern "C" {
// restated weight encoders of the test oracle (oracle/plb_oracle.c)
int orc_sparse_encode_i8(const int8_t* w, int m, int k, int hw, int8_t* nonzero_out, uint32_t* oc_nonzeros, int32_t* diffs);
int orc_sparse_encode_pad4_f32(const float* w, int m, int k, int hw, float* nonzero_out, uint32_t* oc_nonzeros,
                               int32_t* diffs, int* n_stored);
}

using paddle::lite::Buffer;
using paddle::lite::DDim;
using paddle::lite::KernelBase;
using paddle::lite::KernelRegistry;
using paddle::lite::Tensor;
namespace op = paddle::lite::operators;
typedef paddle::lite_api::PrecisionType Prec;
typedef paddle::lite_api::DataLayoutType Layout;

static uint32_t g_seed = 12345;
static int rnd(int lo, int hi) {
  g_seed = g_seed * 1664525u + 1013904223u;
  return lo + static_cast<int>((g_seed >> 8) % static_cast<uint32_t>(hi - lo + 1));
}
static int g_failures = 0;

#define CUDA_OK(x)                                                      \
  do {                                                                  \
    cudaError_t e_ = (x);                                               \
    if (e_ != cudaSuccess) {                                            \
      std::printf("CUDA error %s at %s\n", cudaGetErrorString(e_), #x); \
      std::exit(1);                                                     \
    }                                                                   \
  } while (0)

// device memory the probe owns, with host mirror helpers
struct Dev {
  void* p = nullptr;
  size_t bytes = 0;
  explicit Dev(size_t n) : bytes(n) { CUDA_OK(cudaMalloc(&p, n ? n : 16)); }
  ~Dev() { cudaFree(p); }
  template <typename T>
  void up(const std::vector<T>& h) { CUDA_OK(cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice)); }
  template <typename T>
  std::vector<T> down() const {
    std::vector<T> h(bytes / sizeof(T));
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(h.data(), p, bytes, cudaMemcpyDeviceToHost));
    return h;
  }
};

static void wrap_device(Tensor* t, const Dev& d, const std::vector<int64_t>& dims, Prec prec) {
  t->Resize(DDim(dims));
  t->set_precision(prec);
  t->ResetBuffer(std::make_shared<Buffer>(d.p, TARGET(kCUDA), d.bytes), d.bytes);
}
template <typename T>
static void host_tensor(Tensor* t, const std::vector<T>& v, const std::vector<int64_t>& dims, Prec prec) {
  t->Resize(DDim(dims));
  t->set_precision(prec);
  std::copy(v.begin(), v.end(), t->mutable_data<T>());
}

static std::unique_ptr<KernelBase> pick(const char* op_type, Prec prec, Layout layout, const char* alias) {
  auto list = KernelRegistry::Global().Create(op_type, TARGET(kCUDA), prec, layout);
  for (auto& k : list)
    if (k->alias() == alias) {
      k->SetContext(std::unique_ptr<paddle::lite::KernelContext>(new paddle::lite::KernelContext));
      return std::move(k);
    }
  std::printf("FAIL: %s/%s is not in the KernelRegistry\n", op_type, alias);
  std::exit(1);
}

template <typename T>
static void check(const char* what, const std::vector<T>& got, const std::vector<T>& want) {
  size_t bad = 0;
  for (size_t i = 0; i < want.size(); ++i) bad += got[i] != want[i];
  std::printf("%s: %zu of %zu outputs differ\n", what, bad, want.size());
  g_failures += bad != 0;
}

static float act_relu(float v) { return v > 0.f ? v : 0.f; }
static int8_t requant(float g) {
  float r = std::nearbyintf(g);
  r = r > 127.f ? 127.f : (r < -127.f ? -127.f : r);
  return static_cast<int8_t>(r);
}

// A conv layer on the host: exact accumulators, then the canonical epilogue (ReLU).  NCHW.
struct HostConv {
  int N, C, H, W, O, K, S, P, G;
  std::vector<int8_t> w;  // [O][C/G][K][K]
  std::vector<float> ws, bias;
  float in_s, out_s;
  int Ho() const { return (H + 2 * P - K) / S + 1; }
  int Wo() const { return (W + 2 * P - K) / S + 1; }
  void init() {
    w.resize(static_cast<size_t>(O) * (C / G) * K * K);
    ws.resize(O);
    bias.resize(O);
    for (auto& v : w) v = static_cast<int8_t>(rnd(-127, 127));
    for (int o = 0; o < O; ++o) {
      ws[o] = 0.001f + 0.0001f * rnd(0, 50);
      bias[o] = 0.01f * rnd(-100, 100);
    }
  }
  void run(const std::vector<int8_t>& x, std::vector<float>* yf, std::vector<int8_t>* yq) const {
    const int ho = Ho(), wo = Wo(), cg = C / G, og = O / G;
    if (yf) yf->assign(static_cast<size_t>(N) * O * ho * wo, 0.f);
    if (yq) yq->assign(static_cast<size_t>(N) * O * ho * wo, 0);
    for (int n = 0; n < N; ++n)
      for (int o = 0; o < O; ++o)
        for (int oh = 0; oh < ho; ++oh)
          for (int ow = 0; ow < wo; ++ow) {
            int acc = 0;
            const int g = o / og;
            for (int c = 0; c < cg; ++c)
              for (int r = 0; r < K; ++r)
                for (int s = 0; s < K; ++s) {
                  const int ih = oh * S - P + r, iw = ow * S - P + s;
                  if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                  acc += static_cast<int>(x[((static_cast<size_t>(n) * C + g * cg + c) * H + ih) * W + iw]) *
                         static_cast<int>(w[((static_cast<size_t>(o) * cg + c) * K + r) * K + s]);
                }
            const size_t idx = ((static_cast<size_t>(n) * O + o) * ho + oh) * wo + ow;
            if (yf) (*yf)[idx] = act_relu(std::fmaf(static_cast<float>(acc), ws[o] * in_s, bias[o]));
            if (yq) (*yq)[idx] = requant(act_relu(std::fmaf(static_cast<float>(acc), ws[o] * in_s / out_s, bias[o] / out_s)));
          }
  }
};

template <typename T>
static std::vector<T> to_nhwc(const std::vector<T>& x, int n, int c, int h, int w) {
  std::vector<T> y(x.size());
  for (int a = 0; a < n; ++a)
    for (int b = 0; b < c; ++b)
      for (int i = 0; i < h * w; ++i) y[(static_cast<size_t>(a) * h * w + i) * c + b] = x[(static_cast<size_t>(a) * c + b) * h * w + i];
  return y;
}

static void fill_conv_param(op::ConvParam* p, const HostConv& L, Tensor* x, Tensor* w, Tensor* b, Tensor* out) {
  p->x = x;
  p->filter = w;
  p->bias = b;
  p->output = out;
  p->strides = {L.S, L.S};
  p->paddings = std::make_shared<std::vector<int>>(std::vector<int>{L.P, L.P, L.P, L.P});
  p->dilations = std::make_shared<std::vector<int>>(std::vector<int>{1, 1});
  p->groups = L.G;
  p->activation_param.has_active = true;
  p->activation_param.active_type = paddle::lite_api::ActivationType::kRelu;
  p->enable_int8 = true;
  p->input_scale = L.in_s;
  p->output_scale = L.out_s;
  p->weight_scale = L.ws;
}

// conv2d / depthwise_conv2d through the registry: both aliases, a second Launch, and a Launch after the
// input shape changed (ReInitWhenNeeded)
static void conv_checks(const char* op_type, HostConv L) {
  L.init();
  for (int pass = 0; pass < 2; ++pass) {
    const bool i8 = pass == 0;
    auto kernel = pick(op_type, PRECISION(kInt8), DATALAYOUT(kNCHW), i8 ? "int8_out" : "fp32_out");
    if (pass == 0)
      std::printf("created %s alias %s serialised as %s\n", kernel->name().c_str(), kernel->alias().c_str(),
                  kernel->SerializedKernelType().c_str());
    Tensor tw, tb;
    host_tensor(&tw, L.w, {L.O, L.C / L.G, L.K, L.K}, PRECISION(kInt8));
    host_tensor(&tb, L.bias, {L.O}, PRECISION(kFloat));
    for (int shape = 0; shape < 2; ++shape) {
      HostConv M = L;
      if (shape == 1) {  // same kernel object, smaller image
        M.H = L.H - 3;
        M.W = L.W - 2;
      }
      std::vector<int8_t> x(static_cast<size_t>(M.N) * M.C * M.H * M.W);
      for (auto& v : x) v = static_cast<int8_t>(rnd(-127, 127));
      std::vector<float> want_f;
      std::vector<int8_t> want_q;
      M.run(x, i8 ? nullptr : &want_f, i8 ? &want_q : nullptr);
      const size_t outs = static_cast<size_t>(M.N) * M.O * M.Ho() * M.Wo();
      Dev dx(x.size()), dy(outs * (i8 ? 1 : 4));
      dx.up(x);
      Tensor tx, ty;
      wrap_device(&tx, dx, {M.N, M.C, M.H, M.W}, PRECISION(kInt8));
      wrap_device(&ty, dy, {M.N, M.O, M.Ho(), M.Wo()}, i8 ? PRECISION(kInt8) : PRECISION(kFloat));
      op::ConvParam param{};
      fill_conv_param(&param, M, &tx, &tw, &tb, &ty);
      kernel->SetParam(param);
      kernel->Launch();  // PrepareForRun on the first call (or a re-plan after the shape change), then Run
      kernel->Launch();  // and a second Run through the same prepared object
      const std::string what = std::string(op_type) + (i8 ? " int8_out" : " fp32_out") + (shape ? " after a shape change" : "");
      if (i8) check(what.c_str(), dy.down<int8_t>(), want_q);
      else check(what.c_str(), dy.down<float>(), want_f);
    }
  }
}

static void fc_checks() {
  const int M = 5, KK = 64, NN = 40;
  const float in_s = 0.02f, out_s = 0.06f;
  std::vector<int8_t> fx(M * KK), fw(KK * NN);
  std::vector<float> fws(NN), fb(NN), want(M * NN);
  std::vector<int8_t> want_q(M * NN);
  for (auto& v : fx) v = static_cast<int8_t>(rnd(-127, 127));
  for (auto& v : fw) v = static_cast<int8_t>(rnd(-127, 127));
  for (int j = 0; j < NN; ++j) {
    fws[j] = 0.002f + 0.0001f * rnd(0, 20);
    fb[j] = 0.01f * rnd(-50, 50);
  }
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < NN; ++j) {
      int acc = 0;
      for (int k = 0; k < KK; ++k) acc += static_cast<int>(fx[i * KK + k]) * static_cast<int>(fw[k * NN + j]);
      want[i * NN + j] = act_relu(std::fmaf(static_cast<float>(acc), fws[j] * in_s, fb[j]));
      want_q[i * NN + j] = requant(act_relu(std::fmaf(static_cast<float>(acc), fws[j] * in_s / out_s, fb[j] / out_s)));
    }
  Dev dx(fx.size());
  dx.up(fx);
  Tensor tx, tw, tb;
  wrap_device(&tx, dx, {M, KK}, PRECISION(kInt8));
  host_tensor(&tw, fw, {KK, NN}, PRECISION(kInt8));
  host_tensor(&tb, fb, {NN}, PRECISION(kFloat));
  for (int pass = 0; pass < 2; ++pass) {
    const bool i8 = pass == 1;
    Dev dy(static_cast<size_t>(M) * NN * (i8 ? 1 : 4));
    Tensor ty;
    wrap_device(&ty, dy, {M, NN}, i8 ? PRECISION(kInt8) : PRECISION(kFloat));
    op::FcParam param{};
    param.input = &tx;
    param.w = &tw;
    param.bias = &tb;
    param.output = &ty;
    param.in_num_col_dims = 1;
    param.activation_type = "relu";
    param.enable_int8 = true;
    param.input_scale = in_s;
    param.output_scale = i8 ? out_s : 1.f;
    param.weight_scale = fws;
    auto kernel = pick("fc", PRECISION(kInt8), DATALAYOUT(kNCHW), i8 ? "int8_out" : "fp32_out");
    kernel->SetParam(param);
    kernel->Launch();
    if (i8) check("fc int8_out", dy.down<int8_t>(), want_q);
    else check("fc fp32_out", dy.down<float>(), want);
  }
}

// sparse_conv2d: dense weights masked to ~20 %, encoded by the restated detect-pass encoders, result = dense conv
static void sparse_checks() {
  const int N = 2, C = 48, H = 8, W = 8, O = 40, HW = H * W;
  const float in_s = 0.02f, out_s = 0.05f;
  std::vector<int8_t> wd(O * C, 0);
  for (auto& v : wd) v = rnd(0, 4) == 0 ? static_cast<int8_t>(rnd(-127, 127)) : 0;
  std::vector<float> ws(O), bias(O);
  for (int o = 0; o < O; ++o) {
    ws[o] = 0.001f + 0.0001f * rnd(0, 50);
    bias[o] = 0.01f * rnd(-100, 100);
  }
  std::vector<int8_t> x(N * C * HW);
  for (auto& v : x) v = static_cast<int8_t>(rnd(-127, 127));
  std::vector<float> want_f(N * O * HW);
  std::vector<int8_t> want_q(N * O * HW);
  for (int n = 0; n < N; ++n)
    for (int o = 0; o < O; ++o)
      for (int p = 0; p < HW; ++p) {
        int acc = 0;
        for (int c = 0; c < C; ++c) acc += static_cast<int>(wd[o * C + c]) * static_cast<int>(x[(n * C + c) * HW + p]);
        want_f[(n * O + o) * HW + p] = act_relu(std::fmaf(static_cast<float>(acc), ws[o] * in_s, bias[o]));
        want_q[(n * O + o) * HW + p] = requant(act_relu(std::fmaf(static_cast<float>(acc), ws[o] * in_s / out_s, bias[o] / out_s)));
      }
  size_t nnz = 0;
  for (auto v : wd) nnz += v != 0;
  std::vector<int8_t> nz(nnz ? nnz : 1);
  std::vector<uint32_t> cum(O);
  std::vector<int32_t> diffs(nnz ? nnz : 1);
  const int first_ic = orc_sparse_encode_i8(wd.data(), O, C, HW, nz.data(), cum.data(), diffs.data());
  Dev dx(x.size());
  dx.up(x);
  Tensor tx, tnz, tcum, tdiff, tb;
  wrap_device(&tx, dx, {N, C, H, W}, PRECISION(kInt8));
  host_tensor(&tnz, nz, {static_cast<int64_t>(nnz)}, PRECISION(kInt8));
  host_tensor(&tcum, cum, {O}, PRECISION(kInt32));
  host_tensor(&tdiff, diffs, {static_cast<int64_t>(nnz)}, PRECISION(kInt32));
  host_tensor(&tb, bias, {O}, PRECISION(kFloat));
  auto fill = [&](op::SparseConvParam* p, Tensor* xin, Tensor* w, Tensor* out, int fic) {
    p->x = xin;
    p->nonzero_weights = w;
    p->oc_nonzeros = &tcum;
    p->diffs = &tdiff;
    p->bias = &tb;
    p->output = out;
    p->first_ic = fic;
    p->flag_semi = 0;
    p->activation_param.has_active = true;
    p->activation_param.active_type = paddle::lite_api::ActivationType::kRelu;
    p->enable_int8 = true;
    p->input_scale = in_s;
    p->output_scale = out_s;
    p->weight_scale = ws;
  };
  for (int pass = 0; pass < 2; ++pass) {
    const bool i8 = pass == 0;
    Dev dy(static_cast<size_t>(N) * O * HW * (i8 ? 1 : 4));
    Tensor ty;
    wrap_device(&ty, dy, {N, O, H, W}, i8 ? PRECISION(kInt8) : PRECISION(kFloat));
    op::SparseConvParam param{};
    fill(&param, &tx, &tnz, &ty, first_ic);
    auto kernel = pick("sparse_conv2d", PRECISION(kInt8), DATALAYOUT(kNCHW), i8 ? "int8_int8_out" : "int8_fp32_out");
    kernel->SetParam(param);
    kernel->Launch();
    kernel->Launch();
    if (i8) check("sparse_conv2d int8_int8_out", dy.down<int8_t>(), want_q);
    else check("sparse_conv2d int8_fp32_out", dy.down<float>(), want_f);
  }
  {
    // fp32 kernel (alias def): weights padded to multiples of four per channel; accumulate in ascending-ic order
    // starting from the bias, fused multiply-adds, as the ARM kernel does
    std::vector<float> wf(O * C), xf(N * C * HW), want(N * O * HW);
    for (size_t i = 0; i < wf.size(); ++i) wf[i] = wd[i] * 0.01f;
    for (auto& v : xf) v = 0.05f * rnd(-40, 40);
    for (int n = 0; n < N; ++n)
      for (int o = 0; o < O; ++o)
        for (int p = 0; p < HW; ++p) {
          float acc = bias[o];
          for (int c = 0; c < C; ++c)
            if (wf[o * C + c] != 0.f) acc = std::fmaf(wf[o * C + c], xf[(n * C + c) * HW + p], acc);
          want[(n * O + o) * HW + p] = act_relu(acc);
        }
    std::vector<float> nzf(nnz + 4 * O);
    std::vector<int32_t> df(nnz + 4 * O);
    std::vector<uint32_t> cf(O);
    int stored = 0;
    const int fic = orc_sparse_encode_pad4_f32(wf.data(), O, C, HW, nzf.data(), cf.data(), df.data(), &stored);
    nzf.resize(stored);
    df.resize(stored);
    Dev dxf(xf.size() * 4), dy(want.size() * 4);
    dxf.up(xf);
    Tensor txf, tnzf, tcf, tdf, ty;
    wrap_device(&txf, dxf, {N, C, H, W}, PRECISION(kFloat));
    wrap_device(&ty, dy, {N, O, H, W}, PRECISION(kFloat));
    host_tensor(&tnzf, nzf, {stored}, PRECISION(kFloat));
    host_tensor(&tcf, cf, {O}, PRECISION(kInt32));
    host_tensor(&tdf, df, {stored}, PRECISION(kInt32));
    op::SparseConvParam param{};
    fill(&param, &txf, &tnzf, &ty, fic);
    param.oc_nonzeros = &tcf;
    param.diffs = &tdf;
    param.enable_int8 = false;
    auto kernel = pick("sparse_conv2d", PRECISION(kFloat), DATALAYOUT(kNCHW), "def");
    kernel->SetParam(param);
    kernel->Launch();
    check("sparse_conv2d fp32 def", dy.down<float>(), want);
  }
}

// a sparse_conv2d whose fused activation this target does not implement must stop the program
static int hard_swish_must_be_fatal() {
  std::vector<int8_t> nz = {5};
  std::vector<uint32_t> cum = {1, 1, 1, 1};
  std::vector<int32_t> diffs = {0};
  std::vector<float> ws = {0.01f, 0.01f, 0.01f, 0.01f};
  Dev dx(4 * 16), dy(4 * 16);
  Tensor tx, tnz, tcum, tdiff, ty;
  wrap_device(&tx, dx, {1, 4, 4, 4}, PRECISION(kInt8));
  wrap_device(&ty, dy, {1, 4, 4, 4}, PRECISION(kInt8));
  host_tensor(&tnz, nz, {1}, PRECISION(kInt8));
  host_tensor(&tcum, cum, {4}, PRECISION(kInt32));
  host_tensor(&tdiff, diffs, {1}, PRECISION(kInt32));
  op::SparseConvParam p{};
  p.x = &tx;
  p.nonzero_weights = &tnz;
  p.oc_nonzeros = &tcum;
  p.diffs = &tdiff;
  p.output = &ty;
  p.activation_param.has_active = true;
  p.activation_param.active_type = paddle::lite_api::ActivationType::kHardSwish;
  p.enable_int8 = true;
  p.input_scale = 0.02f;
  p.output_scale = 0.05f;
  p.weight_scale = ws;
  auto kernel = pick("sparse_conv2d", PRECISION(kInt8), DATALAYOUT(kNCHW), "int8_int8_out");
  kernel->SetParam(p);
  kernel->Launch();  // LOG(FATAL) inside PrepareForRun
  std::printf("FAIL: sparse_conv2d ran with hard_swish\n");
  return 0;
}

static void glue_checks() {
  // io_copy(_once) -> calib(_once) -> calib -> io_copy, as type_precision_cast_pass and the io_copy pass chain
  // them around an int8 sub-graph; then softmax on the device
  for (int once = 0; once < 2; ++once) {
    const int n = 5000;
    const float scale = 0.037f;
    std::vector<float> src(n), want(n);
    for (auto& v : src) v = 0.01f * rnd(-600, 600);
    for (int i = 0; i < n; ++i) {
      float v = src[i] * (1.f / scale);
      v = v > -127.f ? v : -127.f;
      float r = std::nearbyintf(v);
      r = r > 127.f ? 127.f : r;
      want[i] = r * scale;
    }
    Dev d_f(n * 4), d_q(n), d_g(n * 4);
    Tensor h_in, t_f, t_q, t_g, h_out;
    host_tensor(&h_in, src, {n}, PRECISION(kFloat));
    wrap_device(&t_f, d_f, {n}, PRECISION(kFloat));
    wrap_device(&t_q, d_q, {n}, PRECISION(kInt8));
    wrap_device(&t_g, d_g, {n}, PRECISION(kFloat));
    auto k_in = pick(once ? "io_copy_once" : "io_copy", PRECISION(kAny), DATALAYOUT(kAny), "host_to_device");
    auto k_q = pick(once ? "calib_once" : "calib", PRECISION(kInt8), DATALAYOUT(kNCHW), "fp32_to_int8");
    auto k_f = pick(once ? "calib_once" : "calib", PRECISION(kInt8), DATALAYOUT(kNCHW), "int8_to_fp32");
    auto k_out = pick(once ? "io_copy_once" : "io_copy", PRECISION(kAny), DATALAYOUT(kAny), "device_to_host");
    op::IoCopyParam p_in{};
    p_in.x = &h_in;
    p_in.y = &t_f;
    k_in->SetParam(p_in);
    k_in->Launch();
    op::CalibParam p_q{};
    p_q.input = &t_f;
    p_q.output = &t_q;
    p_q.scale = scale;
    k_q->SetParam(p_q);
    k_q->Launch();
    op::CalibParam p_f{};
    p_f.input = &t_q;
    p_f.output = &t_g;
    p_f.scale = scale;
    k_f->SetParam(p_f);
    k_f->Launch();
    op::IoCopyParam p_out{};
    p_out.x = &t_g;
    p_out.y = &h_out;
    k_out->SetParam(p_out);
    k_out->Launch();
    std::vector<float> got(h_out.data<float>(), h_out.data<float>() + n);
    check(once ? "io_copy_once -> calib_once -> calib_once -> io_copy_once" : "io_copy -> calib -> calib -> io_copy", got, want);
  }
  {
    const int rows = 7, cols = 1000;
    std::vector<float> x(rows * cols), want(rows * cols);
    for (auto& v : x) v = 0.01f * rnd(-900, 900);
    Dev dx(x.size() * 4), dy(x.size() * 4);
    dx.up(x);
    Tensor tx, ty;
    wrap_device(&tx, dx, {rows, cols}, PRECISION(kFloat));
    wrap_device(&ty, dy, {rows, cols}, PRECISION(kFloat));
    op::SoftmaxParam p{};
    p.x = &tx;
    p.output = &ty;
    p.axis = -1;
    auto k = pick("softmax", PRECISION(kFloat), DATALAYOUT(kNCHW), "def");
    k->SetParam(p);
    k->Launch();
    auto got = dy.down<float>();
    double worst = 0;
    for (int r = 0; r < rows; ++r) {
      float m = x[r * cols];
      for (int c = 1; c < cols; ++c) m = std::max(m, x[r * cols + c]);
      double sum = 0;
      for (int c = 0; c < cols; ++c) sum += std::exp(static_cast<double>(std::max(x[r * cols + c] - m, -64.f)));
      for (int c = 0; c < cols; ++c) {
        const double w = std::exp(static_cast<double>(std::max(x[r * cols + c] - m, -64.f))) / sum;
        worst = std::max(worst, std::fabs(got[r * cols + c] - w) / std::max(w, 1e-12));
      }
    }
    std::printf("softmax: max relative error %.3g\n", worst);
    g_failures += worst > 1e-5;
  }
}

// pointwise -> depthwise 3x3 -> pointwise through the kNHWC registrations (consecutive int8 layers exchange
// channels-last tensors, no layout staging in between), checked against the host chain; optionally timed
// against the same chain through the kNCHW registrations
static void chain_checks(bool timed) {
  const int N = timed ? 128 : 2, HW = timed ? 56 : 10;
  HostConv A{N, 32, HW, HW, 64, 1, 1, 0, 1}, B{N, 64, HW, HW, 64, 3, 1, 1, 64}, Cc{N, 64, HW, HW, 64, 1, 1, 0, 1};
  A.in_s = 0.02f; A.out_s = 0.9f;
  B.in_s = 0.9f; B.out_s = 40.f;
  Cc.in_s = 40.f; Cc.out_s = 1.f;
  A.init(); B.init(); Cc.init();
  std::vector<int8_t> x(static_cast<size_t>(N) * 32 * HW * HW);
  for (auto& v : x) v = static_cast<int8_t>(rnd(-127, 127));
  std::vector<int8_t> a, b;
  std::vector<float> want;
  if (!timed) {
    A.run(x, nullptr, &a);
    B.run(a, nullptr, &b);
    Cc.run(b, &want, nullptr);
  }
  const size_t px = static_cast<size_t>(N) * HW * HW;
  for (int nhwc = 1; nhwc >= 0; --nhwc) {
    const Layout lay = nhwc ? DATALAYOUT(kNHWC) : DATALAYOUT(kNCHW);
    Dev dx(x.size()), da(px * 64), db(px * 64), dc(px * 64 * 4);
    dx.up(nhwc ? to_nhwc(x, N, 32, HW, HW) : x);
    Tensor tx, ta, tb_, tc;
    wrap_device(&tx, dx, {N, 32, HW, HW}, PRECISION(kInt8));   // logical NCHW dims; the memory is channels-last
    wrap_device(&ta, da, {N, 64, HW, HW}, PRECISION(kInt8));
    wrap_device(&tb_, db, {N, 64, HW, HW}, PRECISION(kInt8));
    wrap_device(&tc, dc, {N, 64, HW, HW}, PRECISION(kFloat));
    Tensor wA, bA, wB, bB, wC, bC;
    host_tensor(&wA, A.w, {64, 32, 1, 1}, PRECISION(kInt8));
    host_tensor(&bA, A.bias, {64}, PRECISION(kFloat));
    host_tensor(&wB, B.w, {64, 1, 3, 3}, PRECISION(kInt8));
    host_tensor(&bB, B.bias, {64}, PRECISION(kFloat));
    host_tensor(&wC, Cc.w, {64, 64, 1, 1}, PRECISION(kInt8));
    host_tensor(&bC, Cc.bias, {64}, PRECISION(kFloat));
    auto k1 = pick("conv2d", PRECISION(kInt8), lay, nhwc ? "int8_out_nhwc" : "int8_out");
    auto k2 = pick("depthwise_conv2d", PRECISION(kInt8), lay, nhwc ? "int8_out_nhwc" : "int8_out");
    auto k3 = pick("conv2d", PRECISION(kInt8), lay, nhwc ? "fp32_out_nhwc" : "fp32_out");
    op::ConvParam p1{}, p2{}, p3{};
    fill_conv_param(&p1, A, &tx, &wA, &bA, &ta);
    fill_conv_param(&p2, B, &ta, &wB, &bB, &tb_);
    fill_conv_param(&p3, Cc, &tb_, &wC, &bC, &tc);
    k1->SetParam(p1);
    k2->SetParam(p2);
    k3->SetParam(p3);
    auto run_chain = [&] {
      k1->Launch();
      k2->Launch();
      k3->Launch();
    };
    run_chain();
    if (!timed) {
      auto got = dc.down<float>();
      check(nhwc ? "conv2d -> depthwise_conv2d -> conv2d through the kNHWC kernels"
                 : "conv2d -> depthwise_conv2d -> conv2d through the kNCHW kernels",
            got, nhwc ? to_nhwc(want, N, 64, HW, HW) : want);
    } else {
      for (int i = 0; i < 5; ++i) run_chain();
      cudaEvent_t e0, e1;
      CUDA_OK(cudaEventCreate(&e0));
      CUDA_OK(cudaEventCreate(&e1));
      CUDA_OK(cudaDeviceSynchronize());
      CUDA_OK(cudaEventRecord(e0, 0));
      const int iters = 50;
      for (int i = 0; i < iters; ++i) run_chain();
      CUDA_OK(cudaEventRecord(e1, 0));
      CUDA_OK(cudaEventSynchronize(e1));
      float ms = 0.f;
      CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
      std::printf("CHAIN_US %s %.2f\n", nhwc ? "nhwc" : "nchw", 1e3 * ms / iters);
    }
  }
}

int main(int argc, char** argv) {
  if (argc > 1 && std::strcmp(argv[1], "--hard-swish") == 0) return hard_swish_must_be_fatal();
  conv_checks("conv2d", HostConv{2, 32, 12, 10, 48, 3, 1, 1, 1, {}, {}, {}, 0.02f, 0.05f});
  conv_checks("conv2d", HostConv{3, 64, 16, 16, 96, 1, 1, 0, 1, {}, {}, {}, 0.02f, 0.05f});  // 1x1: NCHW-native kernel
  conv_checks("depthwise_conv2d", HostConv{2, 32, 12, 10, 32, 3, 1, 1, 32, {}, {}, {}, 0.02f, 0.3f});
  fc_checks();
  sparse_checks();
  glue_checks();
  chain_checks(false);
  if (argc > 1 && std::strcmp(argv[1], "--time") == 0) chain_checks(true);
  std::printf(g_failures ? "PROBE FAILED\n" : "PROBE OK\n");
  return g_failures ? 1 : 0;
}
