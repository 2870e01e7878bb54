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

template <typename T>
int conv_impl(const int8_t* x, const int8_t* w, const float* bias, T* out, int num, int cin,
              int h, int wd, int cout, int kh, int kw, int sh, int sw, int pt, int pb, int pl,
              int pr, int dh, int dw, int groups, const float* wscale, float in_scale,
              float out_scale, int relu_type, float relu_alpha, int threads) {
  const int ho = (h + pt + pb - (dh * (kh - 1) + 1)) / sh + 1;
  const int wo = (wd + pl + pr - (dw * (kw - 1) + 1)) / sw + 1;
  if (ho <= 0 || wo <= 0 || cin % groups || cout % groups) return -1;
  const int m = cout / groups, n = ho * wo, k = cin / groups * kh * kw;
  const bool flag_1x1 = kh == 1 && kw == 1 && sh == 1 && sw == 1 && pt == 0 && pb == 0 &&
                        pl == 0 && pr == 0;
  if (threads < 1) threads = 1;
  if (threads > num) threads = num;
  auto worker = [&](int tid) {
    GroupGemms<T> gemms;
    prepare<T>(&gemms, w, wscale, bias, groups, m, n, k, in_scale, out_scale, relu_type,
               relu_alpha);
    std::vector<int8_t> col;
    if (!flag_1x1) col.resize(static_cast<size_t>(k) * n);
    for (int b = tid; b < num; b += threads) {
      for (int g = 0; g < groups; ++g) {
        T* dout = out + (static_cast<long>(b) * cout + static_cast<long>(g) * m) * n;
        const int8_t* din =
            x + (static_cast<long>(b) * cin + static_cast<long>(g) * (cin / groups)) * h * wd;
        const int8_t* wg = w + static_cast<long>(g) * m * k;
        if (!flag_1x1) {
          xm::im2col<int8_t>(din, cin / groups, h, wd, kh, kw, pt, pb, pl, pr, sh, sw, dh, dw,
                             col.data());
          gemms.g[g]->compute(wg, col.data(), dout);
        } else {
          gemms.g[g]->compute(wg, din, dout);
        }
      }
    }
  };
  if (threads == 1) {
    worker(0);
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) pool.emplace_back(worker, t);
    for (auto& t : pool) t.join();
  }
  return 0;
}

}  // namespace

extern "C" {

// relu_type: 0 none, 1 relu, 2 relu6, 3 leaky; relu_alpha is passed to the GEMM object
// unchanged, so an int8-out caller divides by out_scale first if it wants to mirror
// conv_compute.cc:386-396.
int ref_x86_conv_int8(const int8_t* x, const int8_t* w, const float* bias, void* out,
                      int out_is_int8, int num, int cin, int h, int wd, int cout, int kh, int kw,
                      int sh, int sw, int pt, int pb, int pl, int pr, int dh, int dw, int groups,
                      const float* wscale, float in_scale, float out_scale, int relu_type,
                      float relu_alpha, int threads) {
  if (out_is_int8)
    return conv_impl<int8_t>(x, w, bias, static_cast<int8_t*>(out), num, cin, h, wd, cout, kh,
                             kw, sh, sw, pt, pb, pl, pr, dh, dw, groups, wscale, in_scale,
                             out_scale, relu_type, relu_alpha, threads);
  return conv_impl<float>(x, w, bias, static_cast<float*>(out), num, cin, h, wd, cout, kh, kw,
                          sh, sw, pt, pb, pl, pr, dh, dw, groups, wscale, in_scale, out_scale,
                          relu_type, relu_alpha, threads);
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
