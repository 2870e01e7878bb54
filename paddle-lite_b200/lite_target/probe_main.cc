// Drop-in probe: drives the new kCUDA/kInt8 kernels the way the reference drives its own
// (lite/tests/math/x86_conv_int8_compute_test.cc:156-198): the kernel object comes out of the
// reference's KernelRegistry, receives an operators::ConvParam / FcParam whose activation
// tensors wrap device memory, and runs through KernelBase::Launch().  Results are compared
// on the host with a plain exact loop.  Built against the reference headers and linked with a
// handful of the reference's core objects; run on a machine with an sm_100 GPU.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <vector>

#include "lite/core/kernel.h"
#include "lite/core/op_registry.h"
#include "lite/core/tensor.h"
#include "lite/operators/op_params.h"

using paddle::lite::Buffer;
using paddle::lite::DDim;
using paddle::lite::KernelBase;
using paddle::lite::KernelRegistry;
using paddle::lite::Tensor;

static uint32_t g_seed = 12345;
static int rnd(int lo, int hi) {
  g_seed = g_seed * 1664525u + 1013904223u;
  return lo + static_cast<int>((g_seed >> 8) % static_cast<uint32_t>(hi - lo + 1));
}

#define CUDA_OK(x)                                                      \
  do {                                                                  \
    cudaError_t e = (x);                                                \
    if (e != cudaSuccess) {                                             \
      std::printf("CUDA error %s at %s\n", cudaGetErrorString(e), #x); \
      return 1;                                                         \
    }                                                                   \
  } while (0)

// a lite::Tensor over device memory that the probe owns
static void wrap_device(Tensor* t, void* dptr, size_t bytes, const std::vector<int64_t>& dims,
                        paddle::lite_api::PrecisionType prec) {
  t->Resize(DDim(dims));
  t->set_precision(prec);
  t->ResetBuffer(std::make_shared<Buffer>(dptr, TARGET(kCUDA), bytes), bytes);
}

static std::unique_ptr<KernelBase> create(const char* op, const char* alias) {
  auto list = KernelRegistry::Global().Create(op, TARGET(kCUDA), PRECISION(kInt8), DATALAYOUT(kNCHW));
  for (auto& k : list) {
    if (k->alias() == alias) return std::move(k);
  }
  return nullptr;
}

int main() {
  int failures = 0;
  // ---------------------------------------------------------------- conv2d, int8_out and fp32_out
  const int N = 2, C = 32, H = 12, W = 10, O = 48, K = 3, P = 1;
  std::vector<int8_t> x(N * C * H * W), w(O * C * K * K);
  std::vector<float> ws(O), bias(O);
  for (auto& v : x) v = static_cast<int8_t>(rnd(-127, 127));
  for (auto& v : w) v = static_cast<int8_t>(rnd(-127, 127));
  for (int o = 0; o < O; ++o) {
    ws[o] = 0.001f + 0.0001f * rnd(0, 50);
    bias[o] = 0.01f * rnd(-100, 100);
  }
  const float in_s = 0.02f, out_s = 0.05f;
  std::vector<float> want_f(N * O * H * W);
  std::vector<int8_t> want_q(N * O * H * W);
  for (int n = 0; n < N; ++n)
    for (int o = 0; o < O; ++o)
      for (int oh = 0; oh < H; ++oh)
        for (int ow = 0; ow < W; ++ow) {
          int acc = 0;
          for (int c = 0; c < C; ++c)
            for (int r = 0; r < K; ++r)
              for (int s = 0; s < K; ++s) {
                const int ih = oh - P + r, iw = ow - P + s;
                if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                acc += static_cast<int>(x[((n * C + c) * H + ih) * W + iw]) *
                       static_cast<int>(w[((o * C + c) * K + r) * K + s]);
              }
          const size_t idx = ((static_cast<size_t>(n) * O + o) * H + oh) * W + ow;
          float f = std::fmaf(static_cast<float>(acc), ws[o] * in_s, bias[o]);
          want_f[idx] = f > 0.f ? f : 0.f;
          float g = std::fmaf(static_cast<float>(acc), ws[o] * in_s / out_s, bias[o] / out_s);
          g = g > 0.f ? g : 0.f;
          float r8 = std::nearbyintf(g);
          r8 = r8 > 127.f ? 127.f : (r8 < -127.f ? -127.f : r8);
          want_q[idx] = static_cast<int8_t>(r8);
        }

  void *dx = nullptr, *dq = nullptr, *df = nullptr;
  CUDA_OK(cudaMalloc(&dx, x.size()));
  CUDA_OK(cudaMalloc(&dq, want_q.size()));
  CUDA_OK(cudaMalloc(&df, want_f.size() * 4));
  CUDA_OK(cudaMemcpy(dx, x.data(), x.size(), cudaMemcpyHostToDevice));

  Tensor tx, tw, tb, tq, tf;
  wrap_device(&tx, dx, x.size(), {N, C, H, W}, PRECISION(kInt8));
  wrap_device(&tq, dq, want_q.size(), {N, O, H, W}, PRECISION(kInt8));
  wrap_device(&tf, df, want_f.size() * 4, {N, O, H, W}, PRECISION(kFloat));
  tw.Resize(DDim(std::vector<int64_t>{O, C, K, K}));
  tw.set_precision(PRECISION(kInt8));
  std::copy(w.begin(), w.end(), tw.mutable_data<int8_t>());
  tb.Resize(DDim(std::vector<int64_t>{O}));
  tb.set_precision(PRECISION(kFloat));
  std::copy(bias.begin(), bias.end(), tb.mutable_data<float>());

  for (int pass = 0; pass < 2; ++pass) {
    const bool i8 = pass == 0;
    paddle::lite::operators::ConvParam param{};
    param.x = &tx;
    param.filter = &tw;
    param.bias = &tb;
    param.output = i8 ? &tq : &tf;
    param.strides = {1, 1};
    param.paddings = std::make_shared<std::vector<int>>(std::vector<int>{P, P, P, P});
    param.dilations = std::make_shared<std::vector<int>>(std::vector<int>{1, 1});
    param.groups = 1;
    param.activation_param.has_active = true;
    param.activation_param.active_type = paddle::lite_api::ActivationType::kRelu;
    param.enable_int8 = true;
    param.input_scale = in_s;
    param.output_scale = out_s;
    param.weight_scale = ws;
    auto kernel = create("conv2d", i8 ? "int8_out" : "fp32_out");
    if (!kernel) {
      std::printf("FAIL: conv2d/%s is not in the KernelRegistry\n", i8 ? "int8_out" : "fp32_out");
      return 1;
    }
    std::printf("created %s alias %s serialised as %s\n", kernel->name().c_str(), kernel->alias().c_str(),
                kernel->SerializedKernelType().c_str());
    kernel->SetParam(param);
    kernel->SetContext(std::unique_ptr<paddle::lite::KernelContext>(new paddle::lite::KernelContext));
    kernel->Launch();  // PrepareForRun on the first call, then Run
    kernel->Launch();  // and a second Run through the same prepared object
    CUDA_OK(cudaDeviceSynchronize());
    size_t bad = 0;
    if (i8) {
      std::vector<int8_t> got(want_q.size());
      CUDA_OK(cudaMemcpy(got.data(), dq, got.size(), cudaMemcpyDeviceToHost));
      for (size_t i = 0; i < got.size(); ++i) bad += got[i] != want_q[i];
    } else {
      std::vector<float> got(want_f.size());
      CUDA_OK(cudaMemcpy(got.data(), df, got.size() * 4, cudaMemcpyDeviceToHost));
      for (size_t i = 0; i < got.size(); ++i) bad += got[i] != want_f[i];
    }
    std::printf("conv2d %s: %zu of %zu outputs differ\n", i8 ? "int8_out" : "fp32_out", bad, want_q.size());
    failures += bad != 0;
  }

  // ---------------------------------------------------------------- fc, fp32_out
  {
    const int M = 5, KK = 64, NN = 40;
    std::vector<int8_t> fx(M * KK), fw(KK * NN);
    std::vector<float> fws(NN), fb(NN), want(M * NN);
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
        const float f = std::fmaf(static_cast<float>(acc), fws[j] * in_s, fb[j]);
        want[i * NN + j] = f > 0.f ? f : 0.f;
      }
    void *dfx = nullptr, *dfy = nullptr;
    CUDA_OK(cudaMalloc(&dfx, fx.size()));
    CUDA_OK(cudaMalloc(&dfy, want.size() * 4));
    CUDA_OK(cudaMemcpy(dfx, fx.data(), fx.size(), cudaMemcpyHostToDevice));
    Tensor tfx, tfw, tfb, tfy;
    wrap_device(&tfx, dfx, fx.size(), {M, KK}, PRECISION(kInt8));
    wrap_device(&tfy, dfy, want.size() * 4, {M, NN}, PRECISION(kFloat));
    tfw.Resize(DDim(std::vector<int64_t>{KK, NN}));
    tfw.set_precision(PRECISION(kInt8));
    std::copy(fw.begin(), fw.end(), tfw.mutable_data<int8_t>());
    tfb.Resize(DDim(std::vector<int64_t>{NN}));
    tfb.set_precision(PRECISION(kFloat));
    std::copy(fb.begin(), fb.end(), tfb.mutable_data<float>());
    paddle::lite::operators::FcParam param{};
    param.input = &tfx;
    param.w = &tfw;
    param.bias = &tfb;
    param.output = &tfy;
    param.in_num_col_dims = 1;
    param.activation_type = "relu";
    param.enable_int8 = true;
    param.input_scale = in_s;
    param.output_scale = 1.f;
    param.weight_scale = fws;
    auto kernel = create("fc", "fp32_out");
    if (!kernel) {
      std::printf("FAIL: fc/fp32_out is not in the KernelRegistry\n");
      return 1;
    }
    kernel->SetParam(param);
    kernel->SetContext(std::unique_ptr<paddle::lite::KernelContext>(new paddle::lite::KernelContext));
    kernel->Launch();
    CUDA_OK(cudaDeviceSynchronize());
    std::vector<float> got(want.size());
    CUDA_OK(cudaMemcpy(got.data(), dfy, got.size() * 4, cudaMemcpyDeviceToHost));
    size_t bad = 0;
    for (size_t i = 0; i < got.size(); ++i) bad += got[i] != want[i];
    std::printf("fc fp32_out: %zu of %zu outputs differ\n", bad, want.size());
    failures += bad != 0;
  }
  // ---------------------------------------------------------------- io_copy -> calib -> calib -> io_copy
  // host fp32 -> device (io_copy/host_to_device) -> int8 (calib/fp32_to_int8) -> fp32
  // (calib/int8_to_fp32) -> host (io_copy/device_to_host), as type_precision_cast_pass and the
  // io_copy pass chain them around an int8 sub-graph
  {
    const int n = 5000;
    const float scale = 0.037f;
    std::vector<float> src(n);
    for (auto& v : src) v = 0.01f * rnd(-600, 600);
    std::vector<float> want(n);
    for (int i = 0; i < n; ++i) {
      float v = src[i] * (1.f / scale);
      v = v > -127.f ? v : -127.f;
      float r = std::nearbyintf(v);
      r = r > 127.f ? 127.f : r;
      want[i] = r * scale;
    }
    void *d_f = nullptr, *d_q = nullptr, *d_g = nullptr;
    CUDA_OK(cudaMalloc(&d_f, n * 4));
    CUDA_OK(cudaMalloc(&d_q, n));
    CUDA_OK(cudaMalloc(&d_g, n * 4));
    Tensor h_in, t_f, t_q, t_g, h_out;
    h_in.Resize(DDim(std::vector<int64_t>{n}));
    h_in.set_precision(PRECISION(kFloat));
    std::copy(src.begin(), src.end(), h_in.mutable_data<float>());
    wrap_device(&t_f, d_f, n * 4, {n}, PRECISION(kFloat));
    wrap_device(&t_q, d_q, n, {n}, PRECISION(kInt8));
    wrap_device(&t_g, d_g, n * 4, {n}, PRECISION(kFloat));
    auto pick = [](const char* op, paddle::lite_api::PrecisionType prec, paddle::lite_api::DataLayoutType layout,
                   const char* alias) -> std::unique_ptr<KernelBase> {
      auto list = KernelRegistry::Global().Create(op, TARGET(kCUDA), prec, layout);
      for (auto& k : list)
        if (k->alias() == alias) return std::move(k);
      return nullptr;
    };
    auto run = [](std::unique_ptr<KernelBase>& k) {
      k->SetContext(std::unique_ptr<paddle::lite::KernelContext>(new paddle::lite::KernelContext));
      k->Launch();
    };
    auto k_in = pick("io_copy", PRECISION(kAny), DATALAYOUT(kAny), "host_to_device");
    auto k_q = pick("calib", PRECISION(kInt8), DATALAYOUT(kNCHW), "fp32_to_int8");
    auto k_f = pick("calib", PRECISION(kInt8), DATALAYOUT(kNCHW), "int8_to_fp32");
    auto k_out = pick("io_copy", PRECISION(kAny), DATALAYOUT(kAny), "device_to_host");
    if (!k_in || !k_q || !k_f || !k_out) {
      std::printf("FAIL: io_copy / calib kernels are not in the KernelRegistry\n");
      return 1;
    }
    paddle::lite::operators::IoCopyParam p_in{};
    p_in.x = &h_in;
    p_in.y = &t_f;
    k_in->SetParam(p_in);
    run(k_in);
    paddle::lite::operators::CalibParam p_q{};
    p_q.input = &t_f;
    p_q.output = &t_q;
    p_q.scale = scale;
    k_q->SetParam(p_q);
    run(k_q);
    paddle::lite::operators::CalibParam p_f{};
    p_f.input = &t_q;
    p_f.output = &t_g;
    p_f.scale = scale;
    k_f->SetParam(p_f);
    run(k_f);
    paddle::lite::operators::IoCopyParam p_out{};
    p_out.x = &t_g;
    p_out.y = &h_out;
    k_out->SetParam(p_out);
    run(k_out);
    const float* got = h_out.data<float>();
    size_t bad = 0;
    for (int i = 0; i < n; ++i) bad += got[i] != want[i];
    std::printf("io_copy -> calib -> calib -> io_copy: %zu of %d values differ\n", bad, n);
    failures += bad != 0;
  }
  std::printf(failures ? "PROBE FAILED\n" : "PROBE OK\n");
  return failures ? 1 : 0;
}
