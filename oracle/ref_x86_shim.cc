// Driver around the reference's OWN x86 int8 arithmetic, compiled from the reference
// source tree where it lies (nothing is copied): generate_gemm_s8u8_x86_kern<T>
// (lite/backends/x86/math/gemm_s8u8_compute.h:44-106) and im2col<int8_t>
// (lite/backends/x86/math/avx/conv_utils.cc:1349-1398).
//
// TEST INFRASTRUCTURE ONLY: used to check the exact-integer oracle against the real
// reference and as the timed CPU baseline.  The shipped library never links it.
//
// The loops below drive the reference objects the way Conv2dCompute<kInt8,*>::
// PrepareForRun / Run do (lite/kernels/x86/conv_compute.cc:216-341 and :344-472): one
// GEMM object per group prepared once, then for every image and group an im2col (skipped
// for 1x1 / stride 1 / pad 0) followed by compute().  fc runs the same GEMM in the conv
// orientation (A = W^T [N,K], B = X^T [K,M]) so that scale and bias index the output
// feature, which is what lite/kernels/arm/fc_compute.cc:207-260 computes; the x86
// FcCompute indexes them by batch row (lite/kernels/x86/fc_compute.cc:25-52,176-269).
//
// Batches are sharded over `threads` host threads, one set of GEMM objects per thread
// (their pack buffers are per object, gemm_s8u8_compute.h:128-129).  threads == 1 is the
// reference's actual behaviour: the path has no parallel loop.
#include <cstdint>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#include "lite/backends/x86/math/avx/conv_utils.h"
#include "lite/backends/x86/math/gemm_s8u8_compute.h"

namespace {

namespace xm = paddle::lite::x86::math;

template <typename T>
struct GroupGemms {
  std::vector<std::unique_ptr<xm::generate_gemm_s8u8_x86_kern<T>>> g;
};

template <typename T>
void prepare(GroupGemms<T>* out, const int8_t* w, const float* wscale, const float* bias,
             int groups, int m, int n, int k, float in_scale, float out_scale, int relu_type,
             float relu_alpha) {
  for (int g = 0; g < groups; ++g) {
    const float* b = bias ? bias + g * m : nullptr;  // reference passes bias_ptr + g*m
    out->g.emplace_back(new xm::generate_gemm_s8u8_x86_kern<T>(
        false, false, m, n, k, w + static_cast<long>(g) * m * k, n, wscale + g * m, in_scale,
        out_scale, b, relu_type, relu_alpha));
  }
}

// A prepared layer = what Conv2dCompute<kInt8,*>::PrepareForRun leaves behind (conv_compute.cc:216-289,
// :344-420): the GEMM objects with packed weights, folded scales and bias, once per kernel instance.  The
// reference runs one kernel instance per predictor and thread (Clone()d predictors own their kernels), and a
// GEMM object carries its own packed-B scratch (gemm_s8u8_compute.h:128-129), so a layer that is to run on
// `threads` host threads holds that many instances, all built here, outside any timed region.
struct PreparedConv {
  bool out_i8;
  int cin, h, wd, cout, kh, kw, sh, sw, pt, pb, pl, pr, dh, dw, groups;
  int ho, wo, m, n, k;
  bool flag_1x1;
  int threads;
  std::vector<int8_t> w;  // the GEMM's compute() takes the filter pointer again
  std::vector<GroupGemms<float>> f32;
  std::vector<GroupGemms<int8_t>> i8;
  std::vector<std::vector<int8_t>> col;  // im2col scratch per instance
};

template <typename T>
void run_instance(PreparedConv* p, GroupGemms<T>& gemms, int tid, int threads, const int8_t* x, T* out, int num) {
  for (int b = tid; b < num; b += threads) {
    for (int g = 0; g < p->groups; ++g) {
      T* dout = out + (static_cast<long>(b) * p->cout + static_cast<long>(g) * p->m) * p->n;
      const int8_t* din = x + (static_cast<long>(b) * p->cin + static_cast<long>(g) * (p->cin / p->groups)) * p->h * p->wd;
      const int8_t* wg = p->w.data() + static_cast<long>(g) * p->m * p->k;
      if (!p->flag_1x1) {
        xm::im2col<int8_t>(din, p->cin / p->groups, p->h, p->wd, p->kh, p->kw, p->pt, p->pb, p->pl, p->pr, p->sh,
                           p->sw, p->dh, p->dw, p->col[tid].data());
        gemms.g[g]->compute(wg, p->col[tid].data(), dout);
      } else {
        gemms.g[g]->compute(wg, din, dout);
      }
    }
  }
}

template <typename T>
int run_prepared(PreparedConv* p, std::vector<GroupGemms<T>>& inst, const int8_t* x, T* out, int num) {
  int threads = p->threads < num ? p->threads : num;
  if (threads <= 1) {
    run_instance<T>(p, inst[0], 0, 1, x, out, num);
    return 0;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([=, &inst] { run_instance<T>(p, inst[t], t, threads, x, out, num); });
  for (auto& t : pool) t.join();
  return 0;
}

}  // namespace

extern "C" {

// relu_type: 0 none, 1 relu, 2 relu6, 3 leaky; relu_alpha is passed to the GEMM object
// unchanged, so an int8-out caller divides by out_scale first if it wants to mirror
// conv_compute.cc:386-396.
void* ref_x86_conv_prepare(const int8_t* w, const float* bias, int out_is_int8, int cin, int h, int wd, int cout,
                           int kh, int kw, int sh, int sw, int pt, int pb, int pl, int pr, int dh, int dw, int groups,
                           const float* wscale, float in_scale, float out_scale, int relu_type, float relu_alpha,
                           int threads) {
  const int ho = (h + pt + pb - (dh * (kh - 1) + 1)) / sh + 1;
  const int wo = (wd + pl + pr - (dw * (kw - 1) + 1)) / sw + 1;
  if (ho <= 0 || wo <= 0 || cin % groups || cout % groups) return nullptr;
  PreparedConv* p = new PreparedConv;
  p->out_i8 = out_is_int8 != 0;
  p->cin = cin; p->h = h; p->wd = wd; p->cout = cout; p->kh = kh; p->kw = kw; p->sh = sh; p->sw = sw;
  p->pt = pt; p->pb = pb; p->pl = pl; p->pr = pr; p->dh = dh; p->dw = dw; p->groups = groups;
  p->ho = ho; p->wo = wo;
  p->m = cout / groups; p->n = ho * wo; p->k = cin / groups * kh * kw;
  p->flag_1x1 = kh == 1 && kw == 1 && sh == 1 && sw == 1 && pt == 0 && pb == 0 && pl == 0 && pr == 0;
  p->threads = threads < 1 ? 1 : threads;
  p->w.assign(w, w + static_cast<size_t>(cout) * p->k);
  p->col.resize(p->threads);
  if (p->out_i8) p->i8.resize(p->threads); else p->f32.resize(p->threads);
  for (int t = 0; t < p->threads; ++t) {
    if (!p->flag_1x1) p->col[t].resize(static_cast<size_t>(p->k) * p->n);
    if (p->out_i8)
      prepare<int8_t>(&p->i8[t], p->w.data(), wscale, bias, groups, p->m, p->n, p->k, in_scale, out_scale, relu_type, relu_alpha);
    else
      prepare<float>(&p->f32[t], p->w.data(), wscale, bias, groups, p->m, p->n, p->k, in_scale, out_scale, relu_type, relu_alpha);
  }
  return p;
}

// = Conv2dCompute<kInt8,*>::Run (conv_compute.cc:292-341, :423-472) on `num` images, sharded over the instances.
int ref_x86_conv_run(void* handle, const int8_t* x, void* out, int num) {
  PreparedConv* p = static_cast<PreparedConv*>(handle);
  if (!p) return -1;
  if (p->out_i8) return run_prepared<int8_t>(p, p->i8, x, static_cast<int8_t*>(out), num);
  return run_prepared<float>(p, p->f32, x, static_cast<float*>(out), num);
}

void ref_x86_conv_destroy(void* handle) { delete static_cast<PreparedConv*>(handle); }

// Prepare + run + destroy in one call (tests and fixture generation).
int ref_x86_conv_int8(const int8_t* x, const int8_t* w, const float* bias, void* out,
                      int out_is_int8, int num, int cin, int h, int wd, int cout, int kh, int kw,
                      int sh, int sw, int pt, int pb, int pl, int pr, int dh, int dw, int groups,
                      const float* wscale, float in_scale, float out_scale, int relu_type,
                      float relu_alpha, int threads) {
  if (threads > num) threads = num;
  void* h_ = ref_x86_conv_prepare(w, bias, out_is_int8, cin, h, wd, cout, kh, kw, sh, sw, pt, pb, pl, pr, dh, dw, groups,
                                  wscale, in_scale, out_scale, relu_type, relu_alpha, threads);
  if (!h_) return -1;
  const int rc = ref_x86_conv_run(h_, x, out, num);
  ref_x86_conv_destroy(h_);
  return rc;
}

// fc in the conv orientation: wt [N,K] (the FcParam weight [K,N] transposed by the caller),
// xt [K,M] (activations transposed), out [N,M].  One GEMM, single thread per call.
int ref_x86_fc_int8_t(const int8_t* xt, const int8_t* wt, const float* bias, void* out,
                      int out_is_int8, int m, int k, int n, const float* wscale, float in_scale,
                      float out_scale, int relu_type, float relu_alpha) {
  if (out_is_int8) {
    xm::generate_gemm_s8u8_x86_kern<int8_t> gemm(false, false, n, m, k, wt, m, wscale, in_scale,
                                                 out_scale, bias, relu_type, relu_alpha);
    gemm.compute(wt, xt, static_cast<int8_t*>(out));
  } else {
    xm::generate_gemm_s8u8_x86_kern<float> gemm(false, false, n, m, k, wt, m, wscale, in_scale,
                                                out_scale, bias, relu_type, relu_alpha);
    gemm.compute(wt, xt, static_cast<float*>(out));
  }
  return 0;
}

// The reference's im2col alone (used to check the oracle's index arithmetic).
void ref_x86_im2col_int8(const int8_t* x, int c, int h, int w, int kh, int kw, int pt, int pb,
                         int pl, int pr, int sh, int sw, int dh, int dw, int8_t* col) {
  xm::im2col<int8_t>(x, c, h, w, kh, kw, pt, pb, pl, pr, sh, sw, dh, dw, col);
}

}  // extern "C"
