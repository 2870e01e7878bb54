// C ABI of the library (include/plb200.h): contexts, prepared layers, dispatch.
// Host-side planning only; the arithmetic lives in igemm_tc.cu and kernels_simple.cu.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <memory>
#include <mutex>

#include "fused_dwpw.cuh"
#include "igemm_nchw.cuh"
#include "igemm_tc.cuh"
#include "kernels_simple.cuh"
#include "stem_tc.cuh"

namespace plb {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("PLB_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct DeviceBuf {
  void* p = nullptr;
  ~DeviceBuf() {
    if (p) cudaFree(p);
  }
  int upload(const void* host, size_t bytes) {
    if (bytes == 0) bytes = 16;
    PLB_CUDA(cudaMalloc(&p, align_up(bytes, 256)));
    if (host) PLB_CUDA(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice));
    return PLB_OK;
  }
  template <typename T>
  T* as() const {
    return static_cast<T*>(p);
  }
};

// scale / bias / alpha folding of the reference GEMM object
// (gemm_s8u8_compute.cc:26-98, conv_compute.cc:386-396), same float operation order as the
// exact-integer oracle.
struct Folded {
  std::vector<float> scale_f32, bias_f32, scale_i8, bias_i8;
  float alpha_f32 = 0.f, alpha_i8 = 0.f;
};

Folded fold(int c, const float* wscale, int n_wscale, const float* bias, float in_scale,
            float out_scale, int act, float alpha, int leaky_compat) {
  Folded f;
  f.scale_f32.resize(c);
  f.bias_f32.resize(c);
  f.scale_i8.resize(c);
  f.bias_i8.resize(c);
  for (int i = 0; i < c; ++i) {
    const float ws = wscale[n_wscale == 1 ? 0 : i];
    const float s = ws * in_scale;
    const float b = bias ? bias[i] : 0.f;
    f.scale_f32[i] = s;
    f.bias_f32[i] = b;
    f.scale_i8[i] = s / out_scale;
    f.bias_i8[i] = b / out_scale;
  }
  f.alpha_f32 = alpha;
  f.alpha_i8 = alpha;
  if (act == PLB_ACT_RELU6) f.alpha_i8 = alpha / out_scale;
  if (act == PLB_ACT_LEAKY && leaky_compat) f.alpha_i8 = alpha / out_scale;
  return f;
}

}  // namespace
}  // namespace plb

using namespace plb;

int plb_ctx::reserve(size_t bytes) {
  if (bytes <= ws_bytes) return PLB_OK;
  if (!ws_owned && ws != nullptr)
    return fail(PLB_E_NOMEM, "caller-provided workspace of %zu bytes is too small (%zu needed)",
                ws_bytes, bytes);
  // growing: wait for work that may still use the old buffer
  PLB_CUDA(cudaStreamSynchronize(stream));
  if (ws) PLB_CUDA(cudaFree(ws));
  ws = nullptr;
  ws_bytes = 0;
  cudaError_t e = cudaMalloc(&ws, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(PLB_E_NOMEM, "cudaMalloc of %zu workspace bytes failed: %s", bytes,
                cudaGetErrorString(e));
  }
  ws_bytes = bytes;
  ws_owned = true;
  return PLB_OK;
}

struct plb_conv {
  plb_ctx* ctx = nullptr;
  plb_conv_desc d;
  int ho = 0, wo = 0;
  int kind = 0;        // 0 tensor core, 1 direct, 2 depthwise
  bool fold = false;   // stem layer: kw taps x fold_h rows of the filter are folded into the channels
  int fold_h = 1;      // input rows per staged pixel (= stride_h)
  int fold_kh = 0;     // filter rows of the folded convolution, ceil(kh / fold_h)
  int fold_ht = 0;     // rows of the staged tensor, ho + fold_kh - 1
  int cin_pad = 0;     // channel stride of the NHWC staging input
  int cg_pad = 0;      // filter row length per tap
  DeviceBuf w;         // repacked filter
  DeviceBuf w16;       // first layers with filter rows of at most 16 bytes: the folded filter with 16-byte rows
  DeviceBuf scale_f32, bias_f32, scale_i8, bias_i8;
  std::vector<float> h_scale_i8, h_bias_i8;  // host copies of the int8-out tables (row-folded first layers only)
  float alpha_f32 = 0.f, alpha_i8 = 0.f;
  bool acc_small = false;  // 128 * max over channels of sum |w| < 2^22: accumulators convert to float exactly by the mantissa trick
  TcSwitches sw;           // tuning switches, read from the environment when the layer was prepared
  IgemmPlanCache* plans = nullptr;  // tile plans and tensor maps of the (batch, pointers) this layer has run on
  ~plb_conv() { igemm_plan_cache_destroy(plans); }
};

struct plb_fc {
  plb_ctx* ctx = nullptr;
  int k = 0, n = 0, k_pad = 0;
  int act = 0, out_dtype = 0;
  bool tc = false;
  DeviceBuf wt;  // [n, k_pad]
  DeviceBuf scale_f32, bias_f32, scale_i8, bias_i8;
  float alpha_f32 = 0.f, alpha_i8 = 0.f;
  bool acc_small = false;
  TcSwitches sw;
  IgemmPlanCache* plans = nullptr;
  ~plb_fc() { igemm_plan_cache_destroy(plans); }
};

struct plb_sparse {
  plb_ctx* ctx = nullptr;
  plb_sparse_desc d;
  int nnz = 0;
  DeviceBuf row_ptr, col, val, bias_raw;
  DeviceBuf col_val;  // fp32: {input channel, weight bits} per non-zero
  DeviceBuf grp_ptr, grp_idx, grp_w;  // int8: non-zeros in groups of four for the slab kernel
  DeviceBuf scale, bias;
  float alpha = 0.f;
  plb_conv* dense = nullptr;  // densified tensor-core variant
};

// ------------------------------------------------------------------ scratch that is never allocated
// Staging memory of plb_conv_run_static(): part of the library image, so every GPU that loads
// the library holds these bytes until the process exits.  In host code this name is only a
// handle; the device address is looked up once per device with cudaGetSymbolAddress().
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static void* g_static_scratch_addr[64] = {nullptr};  // per device ordinal
static std::mutex g_static_scratch_mutex;            // first-use lookups from several host threads

extern "C" {

const char* plb_last_error(void) { return g_last_error.c_str(); }

int plb_ctx_create(int device, void* cuda_stream, plb_ctx** out) {
  PLB_REQUIRE(out != nullptr, "out must not be null");
  *out = nullptr;
  int count = 0;
  PLB_CUDA(cudaGetDeviceCount(&count));
  PLB_REQUIRE(device >= 0 && device < count, "device %d out of range (%d visible)", device, count);
  PLB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  PLB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(PLB_E_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                device, prop.major, prop.minor);
  std::unique_ptr<plb_ctx> c(new plb_ctx);
  c->device = device;
  c->stream = static_cast<cudaStream_t>(cuda_stream);
  c->sm_count = prop.multiProcessorCount;
  PLB_CUDA(cudaMalloc(&c->d_status, 2 * sizeof(int)));
  PLB_CUDA(cudaMemset(c->d_status, 0, 2 * sizeof(int)));
  PLB_CUDA(cudaMallocHost(&c->h_status, 2 * sizeof(int)));
  c->h_status[0] = c->h_status[1] = 0;
  *out = c.release();
  return PLB_OK;
}

void plb_ctx_destroy(plb_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->ws && ctx->ws_owned) cudaFree(ctx->ws);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  delete ctx;
}

// Waits for the ctx stream and reports (and clears) a fault recorded by a kernel.  The status word
// rides back on the same stream in front of the wait, so a host-side wait costs one synchronisation.
static int wait_and_check_status(plb_ctx* ctx) {
  PLB_CUDA(cudaMemcpyAsync(ctx->h_status, ctx->d_status, 2 * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  PLB_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->h_status[0] != 0) {
    const int code = ctx->h_status[0], block = ctx->h_status[1];
    ctx->h_status[0] = ctx->h_status[1] = 0;
    cudaMemsetAsync(ctx->d_status, 0, 2 * sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return fail(PLB_E_DEVICE, "kernel fault %d (pipeline wait ran out) in block %d", code, block);
  }
  return PLB_OK;
}

int plb_ctx_sync(plb_ctx* ctx) {
  PLB_REQUIRE(ctx != nullptr, "ctx must not be null");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return wait_and_check_status(ctx);
}

int plb_ctx_set_workspace(plb_ctx* ctx, void* dptr, size_t bytes) {
  PLB_REQUIRE(ctx != nullptr, "ctx must not be null");
  PLB_REQUIRE((reinterpret_cast<uintptr_t>(dptr) & 255) == 0, "workspace must be 256-byte aligned");
  PLB_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->ws && ctx->ws_owned) PLB_CUDA(cudaFree(ctx->ws));
  ctx->ws = dptr;
  ctx->ws_bytes = dptr ? bytes : 0;
  ctx->ws_owned = false;
  return PLB_OK;
}

long plb_ctx_launch_count(const plb_ctx* ctx) { return ctx ? ctx->launches : 0; }
long plb_ctx_window_launch_count(const plb_ctx* ctx) { return ctx ? ctx->window_launches : 0; }
long plb_ctx_nchw_launch_count(const plb_ctx* ctx) { return ctx ? ctx->nchw_launches : 0; }
long plb_ctx_nchw_gather_launch_count(const plb_ctx* ctx) { return ctx ? ctx->nchw_gather_launches : 0; }
long plb_ctx_stem_launch_count(const plb_ctx* ctx) { return ctx ? ctx->stem_launches : 0; }
long plb_ctx_dwpw_launch_count(const plb_ctx* ctx) { return ctx ? ctx->dwpw_launches : 0; }
long plb_ctx_pair_launch_count(const plb_ctx* ctx) { return ctx ? ctx->pair_launches : 0; }
size_t plb_ctx_workspace_size(const plb_ctx* ctx) { return ctx ? ctx->ws_bytes : 0; }

// ------------------------------------------------------------------ conv

int plb_conv_prepare(plb_ctx* ctx, const plb_conv_desc* desc, const int8_t* filter_h,
                     const float* wscale_h, int n_wscale, const float* bias_h, plb_conv** out) {
  PLB_REQUIRE(out != nullptr, "out must not be null");
  *out = nullptr;
  PLB_REQUIRE(ctx && desc && filter_h && wscale_h, "ctx, desc, filter and weight scale are required");
  const plb_conv_desc& d = *desc;
  PLB_REQUIRE(d.cin > 0 && d.h > 0 && d.w > 0 && d.cout > 0 && d.kh > 0 && d.kw > 0, "bad dims");
  PLB_REQUIRE(d.stride_h > 0 && d.stride_w > 0 && d.dil_h > 0 && d.dil_w > 0, "bad stride/dilation");
  PLB_REQUIRE(d.pad_top >= 0 && d.pad_bottom >= 0 && d.pad_left >= 0 && d.pad_right >= 0, "bad padding");
  PLB_REQUIRE(d.groups > 0 && d.cin % d.groups == 0 && d.cout % d.groups == 0,
              "groups must divide cin and cout");
  // conv_compute.cc:242-244: "weights scale size must equal to filter size"
  PLB_REQUIRE(n_wscale == 1 || n_wscale == d.cout, "weight scale size must be 1 or cout (got %d)", n_wscale);
  PLB_REQUIRE(d.act >= PLB_ACT_NONE && d.act <= PLB_ACT_LEAKY, "relu_type must be 0..3 (got %d)", d.act);
  PLB_REQUIRE(d.out_dtype == PLB_OUT_F32 || d.out_dtype == PLB_OUT_I8, "bad out_dtype");
  PLB_REQUIRE(d.in_scale > 0.f, "input_scale must be positive");
  PLB_REQUIRE(d.out_dtype == PLB_OUT_F32 || d.out_scale > 0.f, "output_scale must be positive for int8 out");
  const int ho = (d.h + d.pad_top + d.pad_bottom - (d.dil_h * (d.kh - 1) + 1)) / d.stride_h + 1;
  const int wo = (d.w + d.pad_left + d.pad_right - (d.dil_w * (d.kw - 1) + 1)) / d.stride_w + 1;
  PLB_REQUIRE(ho > 0 && wo > 0, "empty output (%d x %d)", ho, wo);
  PLB_CUDA(cudaSetDevice(ctx->device));

  std::unique_ptr<plb_conv> c(new plb_conv);
  c->ctx = ctx;
  c->d = d;
  c->ho = ho;
  c->wo = wo;
  c->sw = tc_switches_from_env();
  c->plans = igemm_plan_cache_create();
  const int cig = d.cin / d.groups;
  const bool depthwise = d.groups == d.cin && d.cin == d.cout;
  const int taps = d.kh * d.kw;
  {
    long worst = 0;
    const size_t per_channel = static_cast<size_t>(cig) * taps;
    for (int co = 0; co < d.cout; ++co) {
      long sum = 0;
      for (size_t i = 0; i < per_channel; ++i) sum += std::abs(static_cast<int>(filter_h[co * per_channel + i]));
      worst = std::max(worst, sum);
    }
    c->acc_small = worst * 128 < (1L << 22);
  }
  std::vector<int8_t> packed, packed16;
  if (depthwise && d.impl != PLB_IMPL_TC) {
    c->kind = 2;
    c->cin_pad = static_cast<int>(align_up(d.cin, 16));
    c->cg_pad = c->cin_pad;
    packed.assign(static_cast<size_t>(taps) * c->cg_pad, 0);  // [tap][channel]
    for (int ch = 0; ch < d.cout; ++ch)
      for (int t = 0; t < taps; ++t) packed[static_cast<size_t>(t) * c->cg_pad + ch] = filter_h[ch * taps + t];
  } else if (d.groups == 1 && d.impl != PLB_IMPL_DIRECT && d.kw > 1 && d.cin * d.kw <= 32 &&
             d.stride_w <= 8 && d.dil_h == 1 && (d.stride_h == 1 || d.stride_h == 2 || d.stride_h == 4)) {
    // stem layer (e.g. RGB input): fold the kw taps of each filter row into the channel
    // dimension, [cout][kh][s*cin + c], and run a kh x 1 convolution over staged rows
    c->kind = 0;
    c->fold = true;
    c->fold_h = d.stride_h;
    c->fold_kh = (d.kh + c->fold_h - 1) / c->fold_h;
    c->fold_ht = ho + c->fold_kh - 1;
    c->cin_pad = 32 * c->fold_h;
    c->cg_pad = c->cin_pad;
    // [cout][j][e*32 + s*cin + ci] = filter[co][ci][r = j*fold_h + e][s], zero for r >= kh
    packed.assign(static_cast<size_t>(d.cout) * c->fold_kh * c->cin_pad, 0);
    for (int co = 0; co < d.cout; ++co)
      for (int ci = 0; ci < d.cin; ++ci)
        for (int r = 0; r < d.kh; ++r)
          for (int sx = 0; sx < d.kw; ++sx)
            packed[(static_cast<size_t>(co) * c->fold_kh + r / c->fold_h) * c->cin_pad + (r % c->fold_h) * 32 +
                   sx * d.cin + ci] = filter_h[((static_cast<size_t>(co) * d.cin + ci) * d.kh + r) * d.kw + sx];
    if (d.cin * d.kw <= 16 && c->fold_kh * c->fold_h == 4) {
      // the same filter with 16-byte rows, [cout][r][s*cin + ci], for the one-launch first layer (stem_tc.cu)
      packed16.assign(static_cast<size_t>(d.cout) * 4 * 16, 0);
      for (int co = 0; co < d.cout; ++co)
        for (int ci = 0; ci < d.cin; ++ci)
          for (int r = 0; r < d.kh; ++r)
            for (int sx = 0; sx < d.kw; ++sx)
              packed16[(static_cast<size_t>(co) * 4 + r) * 16 + sx * d.cin + ci] =
                  filter_h[((static_cast<size_t>(co) * d.cin + ci) * d.kh + r) * d.kw + sx];
    }
  } else if (d.groups == 1) {
    c->cin_pad = static_cast<int>(align_up(d.cin, 32));
    c->cg_pad = c->cin_pad;
    c->kind = d.impl == PLB_IMPL_DIRECT ? 1 : 0;
    packed.assign(static_cast<size_t>(d.cout) * taps * c->cg_pad, 0);  // [cout][tap][channel]
    for (int co = 0; co < d.cout; ++co)
      for (int ci = 0; ci < d.cin; ++ci)
        for (int t = 0; t < taps; ++t)
          packed[(static_cast<size_t>(co) * taps + t) * c->cg_pad + ci] =
              filter_h[(static_cast<size_t>(co) * d.cin + ci) * taps + t];
  } else {
    if (d.impl == PLB_IMPL_TC)
      return fail(PLB_E_UNSUPPORTED, "the tensor-core kernel takes groups == 1 only");
    c->kind = 1;
    c->cin_pad = static_cast<int>(align_up(d.cin, 16));
    c->cg_pad = cig;
    packed.assign(static_cast<size_t>(d.cout) * taps * cig, 0);
    for (int co = 0; co < d.cout; ++co)
      for (int ci = 0; ci < cig; ++ci)
        for (int t = 0; t < taps; ++t)
          packed[(static_cast<size_t>(co) * taps + t) * cig + ci] =
              filter_h[(static_cast<size_t>(co) * cig + ci) * taps + t];
  }
  if (c->kind == 0 && !c->fold) {
    // shape rules of the tensor-core kernel that do not depend on pointers
    IgemmProblem probe;
    memset(&probe, 0, sizeof(probe));
    probe.cin_pad = c->cin_pad; probe.m_total = 1; probe.cout = d.cout;
    probe.im2col = 1;
    probe.kh = d.kh; probe.kw = d.kw; probe.stride_h = d.stride_h; probe.stride_w = d.stride_w;
    probe.pad_t = d.pad_top; probe.pad_b = d.pad_bottom; probe.pad_l = d.pad_left; probe.pad_r = d.pad_right;
    probe.dil_h = d.dil_h; probe.dil_w = d.dil_w;
    std::string why;
    if (!igemm_tc_supported(probe, &why)) {
      if (d.impl == PLB_IMPL_TC) return fail(PLB_E_UNSUPPORTED, "tensor-core path: %s", why.c_str());
      c->kind = 1;
    }
  }
  int rc = c->w.upload(packed.data(), packed.size());
  if (rc) return rc;
  if (!packed16.empty() && (rc = c->w16.upload(packed16.data(), packed16.size()))) return rc;
  Folded f = fold(d.cout, wscale_h, n_wscale, bias_h, d.in_scale,
                  d.out_dtype == PLB_OUT_I8 ? d.out_scale : 1.f, d.act, d.act_alpha, d.leaky_compat);
  const size_t cb = sizeof(float) * d.cout;
  if ((rc = c->scale_f32.upload(f.scale_f32.data(), cb))) return rc;
  if ((rc = c->bias_f32.upload(f.bias_f32.data(), cb))) return rc;
  if ((rc = c->scale_i8.upload(f.scale_i8.data(), cb))) return rc;
  if ((rc = c->bias_i8.upload(f.bias_i8.data(), cb))) return rc;
  if (c->fold) {  // the one-launch first layer takes its requantiser tables as kernel arguments
    c->h_scale_i8 = f.scale_i8;
    c->h_bias_i8 = f.bias_i8;
  }
  c->alpha_f32 = f.alpha_f32;
  c->alpha_i8 = f.alpha_i8;
  *out = c.release();
  return PLB_OK;
}

int plb_conv_out_dims(const plb_conv* conv, int* ho, int* wo) {
  PLB_REQUIRE(conv && ho && wo, "null argument");
  *ho = conv->ho;
  *wo = conv->wo;
  return PLB_OK;
}

long plb_conv_plan_cache_hits(const plb_conv* conv) { return conv ? igemm_plan_cache_hits(conv->plans) : 0; }

void plb_conv_destroy(plb_conv* conv) {
  if (!conv) return;
  cudaSetDevice(conv->ctx->device);
  cudaStreamSynchronize(conv->ctx->stream);
  delete conv;
}

// bytes of the staged (channels-last or row-folded) input of `batch` images
static size_t staged_input_bytes(const plb_conv* conv, int batch) {
  const size_t pixels = conv->fold ? static_cast<size_t>(conv->fold_ht) * conv->wo
                                   : static_cast<size_t>(conv->d.h) * conv->d.w;
  return align_up(static_cast<size_t>(batch) * pixels * conv->cin_pad, 256);
}

size_t plb_conv_workspace_bytes(const plb_conv* conv, int batch) {
  if (!conv || batch <= 0) return 0;
  const size_t x_bytes = staged_input_bytes(conv, batch);
  const size_t y_bytes = align_up(static_cast<size_t>(batch) * conv->ho * conv->wo * conv->d.cout * 4, 256);
  // 1x1 layers on images whose pixel count is not a multiple of 16 stage rows of a padded pitch instead
  const size_t hwp = align_up(static_cast<size_t>(conv->d.h) * conv->d.w, 16);
  const size_t pitched = align_up(static_cast<size_t>(batch) * conv->d.cin * hwp, 256) +
                         align_up(static_cast<size_t>(batch) * conv->d.cout * hwp * 4, 256);
  return std::max(x_bytes + y_bytes, pitched);
}

int plb_softmax_f32(plb_ctx* ctx, const float* x, float* y, int rows, int cols) {
  PLB_REQUIRE(ctx && (rows == 0 || (x && y)), "null argument");
  PLB_REQUIRE(rows >= 0 && cols > 0, "bad dims");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return softmax_rows_launch(ctx, x, y, rows, cols);
}

}  // extern "C"

namespace {

// x is NHWC with channel stride conv->cin_pad.
int conv_core(plb_conv* c, const int8_t* x, int batch, const OutSpec& out) {
  const plb_conv_desc& d = c->d;
  plb_ctx* ctx = c->ctx;
  if (c->kind == 0) {
    IgemmProblem p;
    memset(&p, 0, sizeof(p));
    const bool flat = d.kh == 1 && d.kw == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_top == 0 &&
                      d.pad_bottom == 0 && d.pad_left == 0 && d.pad_right == 0;
    p.a = x;
    p.im2col = flat ? 0 : 1;
    p.batch = batch; p.h = d.h; p.w = d.w; p.cin_pad = c->cin_pad;
    p.kh = d.kh; p.kw = d.kw; p.stride_h = d.stride_h; p.stride_w = d.stride_w;
    p.pad_t = d.pad_top; p.pad_b = d.pad_bottom; p.pad_l = d.pad_left; p.pad_r = d.pad_right;
    p.dil_h = d.dil_h; p.dil_w = d.dil_w;
    if (c->fold) {  // x is the folded staging tensor [batch, fold_ht, wo, 32*fold_h]: plain kh' x 1 convolution
      p.h = c->fold_ht; p.w = c->wo;
      p.kh = c->fold_kh; p.kw = 1;
      p.stride_h = 1; p.stride_w = 1;
      p.pad_t = p.pad_b = p.pad_l = p.pad_r = 0;
      p.dil_h = 1; p.dil_w = 1;
    }
    p.ho = c->ho; p.wo = c->wo;
    p.m_total = batch * c->ho * c->wo;
    p.b = c->w.as<int8_t>();
    p.cout = d.cout;
    p.out_mode = out.mode; p.y = out.y; p.ldy = out.ldy; p.epi = out.epi;
    p.residual = out.residual; p.y_f32 = out.y_f32; p.y_i8 = out.y_i8;
    p.inv_next_scale = out.inv_next_scale;
    p.a2 = out.a2; p.b2 = out.b2; p.im2col2 = out.im2col2; p.h2 = out.h2; p.w2 = out.w2; p.cin_pad2 = out.cin_pad2;
    p.stride2_h = out.stride2_h; p.stride2_w = out.stride2_w; p.scale2 = out.scale2; p.bias2 = out.bias2;
    p.sw = &c->sw;
    return igemm_tc_launch(ctx, p, c->plans);
  }
  ConvGeom g;
  g.batch = batch; g.cin = d.cin; g.h = d.h; g.w = d.w; g.cin_stride = c->cin_pad;
  g.cout = d.cout; g.kh = d.kh; g.kw = d.kw;
  g.stride_h = d.stride_h; g.stride_w = d.stride_w; g.pad_t = d.pad_top; g.pad_l = d.pad_left;
  g.dil_h = d.dil_h; g.dil_w = d.dil_w; g.groups = d.groups; g.ho = c->ho; g.wo = c->wo;
  g.cg_pad = c->cg_pad;
  g.dw_strip = c->sw.dw_strip;
  if (c->kind == 2) return dwconv_launch(ctx, g, x, c->w.as<int8_t>(), out);
  return conv_direct_launch(ctx, g, x, c->w.as<int8_t>(), out);
}

OutSpec out_spec(const plb_conv* c, int mode, void* y) {
  OutSpec o;
  memset(&o, 0, sizeof(o));
  o.mode = mode;
  o.y = y;
  o.ldy = c->d.cout;
  if (mode == OUT_I8) {
    o.epi.scale = c->scale_i8.as<float>(); o.epi.bias = c->bias_i8.as<float>();
    o.epi.alpha = c->alpha_i8;
    if (!c->h_scale_i8.empty()) {
      o.epi.h_scale = c->h_scale_i8.data();
      o.epi.h_bias = c->h_bias_i8.data();
    }
  } else {
    o.epi.scale = c->scale_f32.as<float>(); o.epi.bias = c->bias_f32.as<float>();
    o.epi.alpha = c->alpha_f32;
  }
  o.epi.act = c->d.act;
  o.epi.acc_small = c->acc_small ? 1 : 0;
  return o;
}

// Unpadded stride-1 1x1 layers can run on the NCHW tensors as they are (igemm_nchw.cu): no staging passes.
bool nchw_native(const plb_conv* c, const int8_t* x, void* y, int batch, int mode, NchwProblem* p) {
  const plb_conv_desc& d = c->d;
  if (c->kind != 0 || c->fold || c->sw.nchw == 0) return false;
  if (!(d.kh == 1 && d.kw == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_top == 0 && d.pad_bottom == 0 &&
        d.pad_left == 0 && d.pad_right == 0))
    return false;
  memset(p, 0, sizeof(*p));
  p->x = x; p->w = c->w.as<int8_t>();
  p->batch = batch; p->cin = d.cin; p->cin_pad = c->cin_pad; p->cout = d.cout; p->hw = d.h * d.w;
  p->out_mode = mode; p->y = y;
  p->bres_switch = c->sw.nchw_bres;
  if (p->hw % 16 != 0) {
    // rows TMA cannot address: gather warps fill the operand tiles (igemm_nchw_gather.cu), several small images per tile
    if (c->sw.nchw_gather != 0 && igemm_nchw_gather_supported(c->ctx, *p, nullptr)) {
      p->x_pitch = -1;  // marks the gather kernel for the caller
      return true;
    }
    // Images of fewer than 100 pixels would fill under half of a 128-pixel tile: the channels-last path, whose
    // tiles run across images, serves them better.
    if (p->hw < 100 && c->sw.nchw != 1) return false;
    // rows TMA cannot address: the caller stages x and y with rows a multiple of 16 bytes apart
    p->x_pitch = static_cast<int>(align_up(p->hw, 16));
    p->y_pitch = mode == OUT_I8 ? p->x_pitch : static_cast<int>(align_up(p->hw, 4));
    const bool aligned = (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    p->x = nullptr; p->y = nullptr;  // filled in by the caller
    return p->cin_pad % 32 == 0 && aligned;
  }
  return igemm_nchw_supported(*p, nullptr);
}

int conv_run_nchw(plb_conv* c, const int8_t* x, void* y, int batch, int mode) {
  plb_ctx* ctx = c->ctx;
  const plb_conv_desc& d = c->d;
  PLB_CUDA(cudaSetDevice(ctx->device));
  {
    NchwProblem np;
    if (nchw_native(c, x, y, batch, mode, &np)) {
      np.epi = out_spec(c, mode, y).epi;
      if (np.x_pitch < 0) {
        np.x_pitch = 0;
        return igemm_nchw_gather_launch(ctx, np);
      }
      if (np.x_pitch == 0) return igemm_nchw_launch(ctx, np);
      // pixel counts that are not a multiple of 16: re-pitch the rows into the workspace, run, copy back
      const int eb = mode == OUT_I8 ? 1 : 4;
      const size_t xs_bytes = align_up(static_cast<size_t>(batch) * d.cin * np.x_pitch, 256);
      int rc = ctx->reserve(plb_conv_workspace_bytes(c, batch));
      if (rc) return rc;
      uint8_t* base = static_cast<uint8_t*>(ctx->ws);
      np.x = reinterpret_cast<const int8_t*>(base);
      np.y = base + xs_bytes;
      if ((rc = pitch_rows_i8_launch(ctx, x, base, static_cast<long>(batch) * d.cin, np.hw, np.x_pitch))) return rc;
      if ((rc = igemm_nchw_launch(ctx, np))) return rc;
      return unpitch_rows_launch(ctx, np.y, y, static_cast<long>(batch) * d.cout, np.hw, np.y_pitch, eb);
    }
  }
  const size_t x_bytes = staged_input_bytes(c, batch);
  int rc = ctx->reserve(plb_conv_workspace_bytes(c, batch));
  if (rc) return rc;
  int8_t* xs = static_cast<int8_t*>(ctx->ws);
  void* ys = static_cast<uint8_t*>(ctx->ws) + x_bytes;
  if (c->fold)
    rc = fold_rows_launch(ctx, x, 0, xs, batch, d.cin, d.h, d.w, c->fold_ht, c->wo, d.kw, c->fold_h,
                          d.stride_w, d.pad_top, d.pad_left, d.dil_w, 1.f);
  else
    rc = nchw_to_nhwc_i8_launch(ctx, x, xs, batch, d.cin, d.h, d.w, c->cin_pad);
  if (rc) return rc;
  OutSpec o = out_spec(c, mode, ys);
  if ((rc = conv_core(c, xs, batch, o))) return rc;
  return nhwc_to_nchw_launch(ctx, ys, y, batch, d.cout, c->ho, c->wo, mode == OUT_I8 ? 1 : 4);
}

}  // namespace

extern "C" {

int plb_conv_run(plb_conv* conv, const int8_t* x, void* y, int batch) {
  PLB_REQUIRE(conv != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;  // an empty batch touches no memory
  PLB_REQUIRE(x && y, "null argument");
  return conv_run_nchw(conv, x, y, batch, conv->d.out_dtype == PLB_OUT_I8 ? OUT_I8 : OUT_F32);
}

int plb_conv_acc_i32(plb_conv* conv, const int8_t* x, int32_t* acc, int batch) {
  PLB_REQUIRE(conv != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;
  PLB_REQUIRE(x && acc, "null argument");
  return conv_run_nchw(conv, x, acc, batch, OUT_ACC);
}

int plb_conv_run_nhwc(plb_conv* conv, const int8_t* x, void* y, int batch) {
  PLB_REQUIRE(conv != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;
  PLB_REQUIRE(x && y, "null argument");
  PLB_REQUIRE(conv->cin_pad == conv->d.cin,
              "channels-last entry needs cin to be a multiple of %d (got %d)",
              conv->kind == 0 || conv->d.groups == 1 ? 32 : 16, conv->d.cin);
  if (batch == 0) return PLB_OK;
  PLB_CUDA(cudaSetDevice(conv->ctx->device));
  OutSpec o = out_spec(conv, conv->d.out_dtype == PLB_OUT_I8 ? OUT_I8 : OUT_F32, y);
  return conv_core(conv, x, batch, o);
}

namespace {
// The problem of a depthwise 3x3 layer followed by a 1x1 layer as one launch; false when the pair does not qualify.
bool dwpw_problem(const plb_conv* dw, const plb_conv* pw, int batch, const int8_t* x, int8_t* y, DwpwProblem* p,
                  std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (!dw || !pw || dw->ctx != pw->ctx) return no("both layers must belong to the same context");
  const plb_conv_desc& a = dw->d;
  const plb_conv_desc& b = pw->d;
  if (dw->kind != 2 || a.kh != 3 || a.kw != 3 || a.dil_h != 1 || a.dil_w != 1 || a.stride_h != a.stride_w)
    return no("first layer must be a depthwise 3x3 convolution");
  if (a.out_dtype != PLB_OUT_I8 || dw->cin_pad != a.cin) return no("depthwise layer must write int8 and have unpadded channels");
  if (pw->kind != 0 || pw->fold || b.kh != 1 || b.kw != 1 || b.stride_h != 1 || b.stride_w != 1 || b.pad_top || b.pad_bottom ||
      b.pad_left || b.pad_right || b.groups != 1)
    return no("second layer must be a plain 1x1 convolution");
  if (b.cin != a.cout || pw->cin_pad != b.cin || b.h != dw->ho || b.w != dw->wo) return no("the 1x1 layer does not take the depthwise output");
  if (b.out_dtype != PLB_OUT_I8) return no("the 1x1 layer must write int8");
  if (dw->sw.dwpw == 0) return no("switched off");
  memset(p, 0, sizeof(*p));
  p->x = x; p->batch = batch; p->h = a.h; p->w = a.w; p->c = a.cin;
  p->stride = a.stride_h; p->pad_t = a.pad_top; p->pad_l = a.pad_left; p->ho = dw->ho; p->wo = dw->wo;
  p->wdw = dw->w.as<int8_t>(); p->cg_pad = dw->cg_pad;
  p->dw_epi = out_spec(dw, OUT_I8, nullptr).epi;
  p->wpw = pw->w.as<int8_t>(); p->cout = b.cout;
  p->pw_epi = out_spec(pw, OUT_I8, nullptr).epi;
  p->y = y; p->ldy = b.cout;
  p->tw = dw->sw.dwpw_tw; p->seg_rows = dw->sw.dwpw_seg;
  return dwpw_fused_supported(dw->ctx, *p, why);
}
}  // namespace

int plb_conv_dwpw_fusable(const plb_conv* dw, const plb_conv* pw) {
  DwpwProblem p;
  // pointer alignment is checked at run time; any 16-byte aligned address stands in for it here
  return dwpw_problem(dw, pw, 1, reinterpret_cast<const int8_t*>(uintptr_t(256)), reinterpret_cast<int8_t*>(uintptr_t(256)), &p,
                      nullptr)
             ? 1
             : 0;
}

int plb_conv_run_nhwc_dwpw(plb_conv* dw, plb_conv* pw, const int8_t* x, int8_t* y, int batch) {
  PLB_REQUIRE(dw != nullptr && pw != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;
  PLB_REQUIRE(x && y, "null argument");
  DwpwProblem p;
  std::string why;
  if (!dwpw_problem(dw, pw, batch, x, y, &p, &why))
    return fail(PLB_E_UNSUPPORTED, "depthwise + 1x1 in one launch: %s", why.c_str());
  PLB_CUDA(cudaSetDevice(dw->ctx->device));
  return dwpw_fused_launch(dw->ctx, p);
}

int plb_conv_run_image_f32(plb_conv* conv, const float* x, void* y, int batch) {
  PLB_REQUIRE(conv != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;
  PLB_REQUIRE(x && y, "null argument");
  plb_ctx* ctx = conv->ctx;
  const plb_conv_desc& d = conv->d;
  PLB_CUDA(cudaSetDevice(ctx->device));
  if (conv->fold && d.out_dtype == PLB_OUT_I8 && conv->sw.stem != 0 && d.dil_w == 1) {
    // calib, row folding and the convolution in one launch where the shape allows it (stem_tc.cu)
    StemProblem sp;
    memset(&sp, 0, sizeof(sp));
    sp.x = x; sp.batch = batch; sp.cin = d.cin; sp.h = d.h; sp.w = d.w;
    sp.kh = d.kh; sp.kw = d.kw; sp.stride_h = d.stride_h; sp.stride_w = d.stride_w; sp.pad_t = d.pad_top; sp.pad_l = d.pad_left;
    sp.ho = conv->ho; sp.wo = conv->wo; sp.fold_h = conv->fold_h; sp.fold_kh = conv->fold_kh;
    sp.wfold = conv->w.as<int8_t>(); sp.wfold16 = conv->w16.as<int8_t>(); sp.cout = d.cout; sp.in_scale = d.in_scale;
    sp.epi = out_spec(conv, OUT_I8, y).epi;
    sp.y = static_cast<int8_t*>(y);
    if (stem_tc_supported(ctx, sp, nullptr)) return stem_tc_launch(ctx, sp);
  }
  const size_t x_bytes = staged_input_bytes(conv, batch);
  int rc = ctx->reserve(x_bytes);
  if (rc) return rc;
  int8_t* xs = static_cast<int8_t*>(ctx->ws);
  if (conv->fold)
    rc = fold_rows_launch(ctx, x, 1, xs, batch, d.cin, d.h, d.w, conv->fold_ht, conv->wo, d.kw, conv->fold_h,
                          d.stride_w, d.pad_top, d.pad_left, d.dil_w, d.in_scale);
  else
    rc = calib_nchw_f32_to_nhwc_i8_launch(ctx, x, xs, batch, d.cin, d.h, d.w, conv->cin_pad, d.in_scale);
  if (rc) return rc;
  OutSpec o = out_spec(conv, d.out_dtype == PLB_OUT_I8 ? OUT_I8 : OUT_F32, y);
  return conv_core(conv, xs, batch, o);
}

int plb_conv_run_static(plb_conv* conv, const int8_t* x, void* y, int batch) {
  PLB_REQUIRE(conv != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;
  PLB_REQUIRE(x && y, "null argument");
  plb_ctx* ctx = conv->ctx;
  const plb_conv_desc& d = conv->d;
  const size_t need = plb_conv_workspace_bytes(conv, batch);
  if (need > kStaticScratchBytes)
    return fail(PLB_E_INVALID,
                "plb_conv_run_static: %d image(s) of this layer need %zu bytes of staging, the built-in "
                "scratch holds %zu; use plb_conv_run or a smaller batch",
                batch, need, kStaticScratchBytes);
  PLB_REQUIRE(ctx->device >= 0 && ctx->device < 64, "device ordinal %d not supported here", ctx->device);
  PLB_CUDA(cudaSetDevice(ctx->device));
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[ctx->device] == nullptr) {
      // first call on this device: resolve the device address of the array (the host-side name
      // is not a device pointer)
      void* addr = nullptr;
      PLB_CUDA(cudaGetSymbolAddress(&addr, g_static_scratch));
      g_static_scratch_addr[ctx->device] = addr;
    }
    base = static_cast<unsigned char*>(g_static_scratch_addr[ctx->device]);
  }
  const size_t x_bytes = staged_input_bytes(conv, batch);
  int8_t* xs = reinterpret_cast<int8_t*>(base);
  void* ys = base + x_bytes;
  // Both staging regions are written in full before they are read (the staging kernels also
  // write the zero padding channels), so nothing of a previous call's contents is observed.
  int rc;
  if (conv->fold)
    rc = fold_rows_launch(ctx, x, 0, xs, batch, d.cin, d.h, d.w, conv->fold_ht, conv->wo, d.kw, conv->fold_h,
                          d.stride_w, d.pad_top, d.pad_left, d.dil_w, 1.f);
  else
    rc = nchw_to_nhwc_i8_launch(ctx, x, xs, batch, d.cin, d.h, d.w, conv->cin_pad);
  if (rc) return rc;
  const int mode = d.out_dtype == PLB_OUT_I8 ? OUT_I8 : OUT_F32;
  OutSpec o = out_spec(conv, mode, ys);
  if ((rc = conv_core(conv, xs, batch, o))) return rc;
  return nhwc_to_nchw_launch(ctx, ys, y, batch, d.cout, conv->ho, conv->wo, mode == OUT_I8 ? 1 : 4);
}

int plb_conv_run_nhwc_add_relu(plb_conv* conv, const int8_t* x, const float* residual, float* y_f32,
                               int8_t* y_i8, float next_scale, int batch) {
  PLB_REQUIRE(conv && x, "null argument");
  PLB_REQUIRE(y_f32 || y_i8, "at least one output is required");
  PLB_REQUIRE(!y_i8 || next_scale > 0.f, "next_scale must be positive");
  PLB_REQUIRE(batch >= 0, "negative batch");
  PLB_REQUIRE(conv->cin_pad == conv->d.cin, "channels-last entry needs cin to be a multiple of 32");
  if (batch == 0) return PLB_OK;
  PLB_CUDA(cudaSetDevice(conv->ctx->device));
  OutSpec o = out_spec(conv, OUT_ADD_RELU, nullptr);
  o.residual = residual;
  o.y_f32 = y_f32;
  o.y_i8 = y_i8;
  o.inv_next_scale = y_i8 ? 1.f / next_scale : 0.f;
  return conv_core(conv, x, batch, o);
}

int plb_conv_run_nhwc_block_add_relu(plb_conv* conv, const int8_t* x, plb_conv* shortcut, const int8_t* x_shortcut,
                                     float* y_f32, int8_t* y_i8, float next_scale, int batch) {
  PLB_REQUIRE(conv && x && shortcut && x_shortcut, "null argument");
  PLB_REQUIRE(y_f32 || y_i8, "at least one output is required");
  PLB_REQUIRE(!y_i8 || next_scale > 0.f, "next_scale must be positive");
  PLB_REQUIRE(batch >= 0, "negative batch");
  PLB_REQUIRE(conv->ctx == shortcut->ctx, "both layers must belong to the same ctx");
  const plb_conv_desc& m = conv->d;
  const plb_conv_desc& s = shortcut->d;
  PLB_REQUIRE(conv->kind == 0 && shortcut->kind == 0 && !conv->fold && !shortcut->fold, "both layers must be dense tensor-core layers");
  PLB_REQUIRE(m.kh == 1 && m.kw == 1 && m.stride_h == 1 && m.stride_w == 1 && m.pad_top == 0 && m.pad_bottom == 0 &&
                  m.pad_left == 0 && m.pad_right == 0,
              "the main layer must be a 1x1, stride-1, unpadded convolution");
  PLB_REQUIRE(s.kh == 1 && s.kw == 1 && s.pad_top == 0 && s.pad_bottom == 0 && s.pad_left == 0 && s.pad_right == 0,
              "the shortcut layer must be an unpadded 1x1 convolution");
  PLB_REQUIRE(m.cout == s.cout && conv->ho == shortcut->ho && conv->wo == shortcut->wo, "the two layers must produce the same shape");
  PLB_REQUIRE(m.act == PLB_ACT_NONE && s.act == PLB_ACT_NONE, "neither layer may have an activation of its own");
  PLB_REQUIRE(conv->cin_pad == m.cin && shortcut->cin_pad == s.cin, "channels-last entry needs cin to be a multiple of 32");
  if (batch == 0) return PLB_OK;
  PLB_CUDA(cudaSetDevice(conv->ctx->device));
  OutSpec o = out_spec(conv, OUT_ADD_RELU, nullptr);
  o.y_f32 = y_f32;
  o.y_i8 = y_i8;
  o.inv_next_scale = y_i8 ? 1.f / next_scale : 0.f;
  o.a2 = x_shortcut;
  o.b2 = shortcut->w.as<int8_t>();
  o.im2col2 = (s.stride_h != 1 || s.stride_w != 1) ? 1 : 0;
  o.h2 = s.h; o.w2 = s.w; o.cin_pad2 = shortcut->cin_pad;
  o.stride2_h = s.stride_h; o.stride2_w = s.stride_w;
  o.scale2 = shortcut->scale_f32.as<float>();
  o.bias2 = shortcut->bias_f32.as<float>();
  return conv_core(conv, x, batch, o);
}

// ------------------------------------------------------------------ fc

int plb_fc_prepare(plb_ctx* ctx, int k, int n, int act, float act_alpha, float in_scale,
                   float out_scale, int out_dtype, const int8_t* w_h, const float* wscale_h,
                   int n_wscale, const float* bias_h, plb_fc** out) {
  PLB_REQUIRE(out != nullptr, "out must not be null");
  *out = nullptr;
  PLB_REQUIRE(ctx && w_h && wscale_h, "ctx, w and weight scale are required");
  PLB_REQUIRE(k > 0 && n > 0, "bad dims");
  PLB_REQUIRE(n_wscale == 1 || n_wscale == n, "weight scale size must be 1 or n (got %d)", n_wscale);
  PLB_REQUIRE(act >= PLB_ACT_NONE && act <= PLB_ACT_LEAKY, "relu_type must be 0..3");
  PLB_REQUIRE(out_dtype == PLB_OUT_F32 || out_dtype == PLB_OUT_I8, "bad out_dtype");
  PLB_REQUIRE(in_scale > 0.f && (out_dtype == PLB_OUT_F32 || out_scale > 0.f), "scales must be positive");
  PLB_CUDA(cudaSetDevice(ctx->device));
  std::unique_ptr<plb_fc> f(new plb_fc);
  f->ctx = ctx;
  f->k = k;
  f->n = n;
  f->act = act;
  f->out_dtype = out_dtype;
  f->sw = tc_switches_from_env();
  f->plans = igemm_plan_cache_create();
  f->tc = (k % 32) == 0;
  f->k_pad = f->tc ? k : static_cast<int>(align_up(k, 4));
  std::vector<int8_t> wt(static_cast<size_t>(n) * f->k_pad, 0);  // [n][k]: K-major rows
  for (int kk = 0; kk < k; ++kk)
    for (int j = 0; j < n; ++j) wt[static_cast<size_t>(j) * f->k_pad + kk] = w_h[static_cast<size_t>(kk) * n + j];
  {
    long worst = 0;
    for (int j = 0; j < n; ++j) {
      long sum = 0;
      for (int kk = 0; kk < k; ++kk) sum += std::abs(static_cast<int>(wt[static_cast<size_t>(j) * f->k_pad + kk]));
      worst = std::max(worst, sum);
    }
    f->acc_small = worst * 128 < (1L << 22);
  }
  int rc = f->wt.upload(wt.data(), wt.size());
  if (rc) return rc;
  Folded fo = fold(n, wscale_h, n_wscale, bias_h, in_scale, out_dtype == PLB_OUT_I8 ? out_scale : 1.f,
                   act, act_alpha, 0);
  const size_t cb = sizeof(float) * n;
  if ((rc = f->scale_f32.upload(fo.scale_f32.data(), cb))) return rc;
  if ((rc = f->bias_f32.upload(fo.bias_f32.data(), cb))) return rc;
  if ((rc = f->scale_i8.upload(fo.scale_i8.data(), cb))) return rc;
  if ((rc = f->bias_i8.upload(fo.bias_i8.data(), cb))) return rc;
  f->alpha_f32 = fo.alpha_f32;
  f->alpha_i8 = fo.alpha_i8;
  *out = f.release();
  return PLB_OK;
}

static int fc_run_mode(plb_fc* f, const int8_t* x, void* y, int m, int mode) {
  plb_ctx* ctx = f->ctx;
  PLB_CUDA(cudaSetDevice(ctx->device));
  EpiParams e;
  if (mode == OUT_I8) {
    e.scale = f->scale_i8.as<float>(); e.bias = f->bias_i8.as<float>(); e.alpha = f->alpha_i8;
  } else {
    e.scale = f->scale_f32.as<float>(); e.bias = f->bias_f32.as<float>(); e.alpha = f->alpha_f32;
  }
  e.act = f->act;
  e.acc_small = f->acc_small ? 1 : 0;
  if (f->tc && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    IgemmProblem p;
    memset(&p, 0, sizeof(p));
    p.a = x; p.im2col = 0; p.cin_pad = f->k; p.kh = p.kw = 1;
    p.m_total = m; p.b = f->wt.as<int8_t>(); p.cout = f->n;
    p.out_mode = mode; p.y = y; p.ldy = f->n; p.epi = e;
    p.sw = &f->sw;
    return igemm_tc_launch(ctx, p, f->plans);
  }
  // rows of x are not TMA-addressable: CUDA-core kernel on the same operands
  if (f->k_pad != f->k)
    return fail(PLB_E_UNSUPPORTED, "fc with k %% 4 != 0 is not supported (k = %d)", f->k);
  ConvGeom g;
  memset(&g, 0, sizeof(g));
  g.batch = m; g.cin = f->k; g.h = 1; g.w = 1; g.cin_stride = f->k; g.cout = f->n; g.kh = g.kw = 1;
  g.stride_h = g.stride_w = 1; g.dil_h = g.dil_w = 1; g.groups = 1; g.ho = g.wo = 1; g.cg_pad = f->k_pad;
  g.dw_strip = -1;
  OutSpec o;
  memset(&o, 0, sizeof(o));
  o.mode = mode; o.y = y; o.ldy = f->n; o.epi = e;
  return conv_direct_launch(ctx, g, x, f->wt.as<int8_t>(), o);
}

int plb_fc_run(plb_fc* fc, const int8_t* x, void* y, int m) {
  PLB_REQUIRE(fc != nullptr, "null argument");
  PLB_REQUIRE(m >= 0, "negative row count");
  if (m == 0) return PLB_OK;
  PLB_REQUIRE(x && y, "null argument");
  return fc_run_mode(fc, x, y, m, fc->out_dtype == PLB_OUT_I8 ? OUT_I8 : OUT_F32);
}

int plb_fc_acc_i32(plb_fc* fc, const int8_t* x, int32_t* acc, int m) {
  PLB_REQUIRE(fc != nullptr, "null argument");
  PLB_REQUIRE(m >= 0, "negative row count");
  if (m == 0) return PLB_OK;
  PLB_REQUIRE(x && acc, "null argument");
  return fc_run_mode(fc, x, acc, m, OUT_ACC);
}

void plb_fc_destroy(plb_fc* fc) {
  if (!fc) return;
  cudaSetDevice(fc->ctx->device);
  cudaStreamSynchronize(fc->ctx->stream);
  delete fc;
}

// ------------------------------------------------------------------ sparse_conv2d

int plb_sparse_prepare(plb_ctx* ctx, const plb_sparse_desc* desc, const void* nonzero_weights_h,
                       int n_weights, const uint32_t* oc_nonzeros_h, const int32_t* diffs_h,
                       int n_diffs, const float* wscale_h, int n_wscale, const float* bias_h,
                       plb_sparse** out) {
  PLB_REQUIRE(out != nullptr, "out must not be null");
  *out = nullptr;
  PLB_REQUIRE(ctx && desc && oc_nonzeros_h, "ctx, desc and oc_nonzeros are required");
  const plb_sparse_desc& d = *desc;
  PLB_REQUIRE(d.cin > 0 && d.cout > 0 && d.h > 0 && d.w > 0, "bad dims");
  PLB_REQUIRE(n_weights >= 0 && n_diffs >= 0, "negative counts");
  PLB_REQUIRE(n_weights == 0 || (nonzero_weights_h && diffs_h), "weights and diffs are required");
  PLB_REQUIRE(d.act >= PLB_ACT_NONE && d.act <= PLB_ACT_LEAKY, "relu_type must be 0..3");
  if (d.is_int8) {
    // sparse_conv_compute.cc:36-40: weight scale size must be 1 or the channel count
    PLB_REQUIRE(wscale_h && (n_wscale == 1 || n_wscale == d.cout),
                "weight scale size must be 1 or cout (got %d)", n_wscale);
    PLB_REQUIRE(d.in_scale > 0.f && (d.out_dtype == PLB_OUT_F32 || d.out_scale > 0.f), "scales must be positive");
  } else {
    PLB_REQUIRE(d.out_dtype == PLB_OUT_F32, "the fp32 kernel writes fp32");
  }
  PLB_CUDA(cudaSetDevice(ctx->device));
  const int hw = d.h * d.w;
  const long unit = static_cast<long>(d.is_int8 ? 1 : 4) * hw;
  const int pairs = d.flag_semi ? d.cout / 2 : 0;
  const int groups = d.flag_semi ? pairs + d.cout % 2 : d.cout;
  const bool pad4 = !d.is_int8 && !d.flag_semi;
  // Walk the encoding the way the ARM kernels do (start pointers:
  // sparse_conv_impl.cc:3731-3745, :1230-1241; sparse_semi_conv_impl.cc:1788-1823) and
  // collect (input channel, weight) per output channel.
  std::vector<std::vector<std::pair<int, float>>> rows(d.cout);
  const int8_t* w8 = static_cast<const int8_t*>(nonzero_weights_h);
  const float* wf = static_cast<const float*>(nonzero_weights_h);
  auto weight_at = [&](long i) -> float { return d.is_int8 ? static_cast<float>(w8[i]) : wf[i]; };
  for (int g = 0; g < groups; ++g) {
    const uint32_t prev0 = g == 0 ? 0u : oc_nonzeros_h[g - 1];
    const uint32_t skip = pad4 ? ((4u - (prev0 & 3u)) & 3u) : 0u;
    const uint32_t prev = prev0 + skip;
    PLB_REQUIRE(oc_nonzeros_h[g] >= prev0, "oc_nonzeros must be non-decreasing");
    if (oc_nonzeros_h[g] < prev) continue;
    const uint32_t cnt = oc_nonzeros_h[g] - prev;
    PLB_REQUIRE(static_cast<long>(prev) + cnt <= n_diffs, "diffs too short for oc_nonzeros");
    long off = (g == 0 || prev0 == 0) ? 0 : diffs_h[prev0 - 1];
    const bool is_pair = d.flag_semi && g < pairs;
    long wi = d.flag_semi ? static_cast<long>(prev) * 2 : static_cast<long>(prev);
    if (d.flag_semi && !is_pair) wi = static_cast<long>(prev) * 2;  // odd last channel, one value per block
    for (uint32_t t = 0; t < cnt; ++t) {
      PLB_REQUIRE(off % unit == 0, "diff %ld is not a multiple of the channel pitch", off);
      const long ic = d.first_ic + off / unit;
      if (is_pair) {
        PLB_REQUIRE(wi + 1 < n_weights, "nonzero_weights too short");
        const float a = weight_at(wi), b = weight_at(wi + 1);
        if (a != 0.f || b != 0.f) PLB_REQUIRE(ic >= 0 && ic < d.cin, "encoding walks outside the input channels");
        if (a != 0.f) rows[2 * g].push_back({static_cast<int>(ic), a});
        if (b != 0.f) rows[2 * g + 1].push_back({static_cast<int>(ic), b});
        wi += 2;
      } else {
        PLB_REQUIRE(wi < n_weights, "nonzero_weights too short");
        const float a = weight_at(wi);
        const int oc = d.flag_semi ? 2 * pairs + (g - pairs) : g;
        if (a != 0.f) {
          PLB_REQUIRE(ic >= 0 && ic < d.cin, "encoding walks outside the input channels");
          rows[oc].push_back({static_cast<int>(ic), a});
        }
        wi += 1;
      }
      off += diffs_h[prev + t];
    }
  }
  std::unique_ptr<plb_sparse> s(new plb_sparse);
  s->ctx = ctx;
  s->d = d;
  std::vector<int> row_ptr(d.cout + 1, 0), col;
  std::vector<int8_t> val8;
  std::vector<float> valf;
  for (int oc = 0; oc < d.cout; ++oc) {
    for (auto& e : rows[oc]) {
      col.push_back(e.first);
      if (d.is_int8) val8.push_back(static_cast<int8_t>(e.second));
      else valf.push_back(e.second);
    }
    row_ptr[oc + 1] = static_cast<int>(col.size());
  }
  s->nnz = static_cast<int>(col.size());
  int rc;
  if ((rc = s->row_ptr.upload(row_ptr.data(), row_ptr.size() * sizeof(int)))) return rc;
  if ((rc = s->col.upload(col.data(), col.size() * sizeof(int)))) return rc;
  if (d.is_int8) rc = s->val.upload(val8.data(), val8.size());
  else rc = s->val.upload(valf.data(), valf.size() * sizeof(float));
  if (rc) return rc;
  if (!d.is_int8) {
    std::vector<int32_t> cv(2 * col.size());
    for (size_t i = 0; i < col.size(); ++i) {
      cv[2 * i] = col[i];
      memcpy(&cv[2 * i + 1], &valf[i], 4);
    }
    if ((rc = s->col_val.upload(cv.data(), cv.size() * sizeof(int32_t)))) return rc;
  }
  if (d.is_int8) {
    std::vector<int> gptr(d.cout + 1, 0);
    std::vector<uint32_t> gidx, gw;
    for (int oc = 0; oc < d.cout; ++oc) {
      const auto& r = rows[oc];
      for (size_t t = 0; t < r.size(); t += 4) {
        uint32_t ic[4] = {0, 0, 0, 0}, wv = 0;
        for (size_t j = 0; j < 4 && t + j < r.size(); ++j) {
          ic[j] = static_cast<uint32_t>(r[t + j].first);
          wv |= (static_cast<uint32_t>(static_cast<int>(r[t + j].second)) & 0xffu) << (8 * j);
        }
        gidx.push_back(ic[0] | (ic[1] << 16));
        gidx.push_back(ic[2] | (ic[3] << 16));
        gw.push_back(wv);
      }
      gptr[oc + 1] = static_cast<int>(gw.size());
    }
    if ((rc = s->grp_ptr.upload(gptr.data(), gptr.size() * sizeof(int)))) return rc;
    if ((rc = s->grp_idx.upload(gidx.data(), gidx.size() * sizeof(uint32_t)))) return rc;
    if ((rc = s->grp_w.upload(gw.data(), gw.size() * sizeof(uint32_t)))) return rc;
  }
  if (d.is_int8) {
    Folded f = fold(d.cout, wscale_h, n_wscale, bias_h, d.in_scale,
                    d.out_dtype == PLB_OUT_I8 ? d.out_scale : 1.f, d.act, d.act_alpha, d.leaky_compat);
    const bool i8 = d.out_dtype == PLB_OUT_I8;
    if ((rc = s->scale.upload(i8 ? f.scale_i8.data() : f.scale_f32.data(), sizeof(float) * d.cout))) return rc;
    if ((rc = s->bias.upload(i8 ? f.bias_i8.data() : f.bias_f32.data(), sizeof(float) * d.cout))) return rc;
    s->alpha = i8 ? f.alpha_i8 : f.alpha_f32;
    // AUTO: at 20 % density the tensor cores beat walking the non-zeros on CUDA cores from 32
    // channels up (both give the same integer sums, hence the same outputs); DIRECT keeps the walk.
    const bool want_dense = d.impl == PLB_IMPL_TC || (d.impl == PLB_IMPL_AUTO && d.cin >= 32 && d.cout >= 32);
    if (want_dense) {
      // densified variant: the same weights as a dense 1x1 filter on the tensor cores
      std::vector<int8_t> dense(static_cast<size_t>(d.cout) * d.cin, 0);
      for (int oc = 0; oc < d.cout; ++oc)
        for (auto& e : rows[oc]) dense[static_cast<size_t>(oc) * d.cin + e.first] = static_cast<int8_t>(e.second);
      plb_conv_desc cd;
      memset(&cd, 0, sizeof(cd));
      cd.cin = d.cin; cd.h = d.h; cd.w = d.w; cd.cout = d.cout; cd.kh = cd.kw = 1;
      cd.stride_h = cd.stride_w = 1; cd.dil_h = cd.dil_w = 1; cd.groups = 1;
      cd.act = d.act; cd.act_alpha = d.act_alpha; cd.in_scale = d.in_scale; cd.out_scale = d.out_scale;
      cd.out_dtype = d.out_dtype; cd.leaky_compat = d.leaky_compat; cd.impl = PLB_IMPL_TC;
      rc = plb_conv_prepare(ctx, &cd, dense.data(), wscale_h, n_wscale, bias_h, &s->dense);
      if (rc && d.impl == PLB_IMPL_TC) return rc;
      if (rc) s->dense = nullptr;  // AUTO: shapes the tensor-core path cannot take keep the walk
    }
  } else {
    if (bias_h && (rc = s->bias_raw.upload(bias_h, sizeof(float) * d.cout))) return rc;
    s->alpha = d.act_alpha;
    if (d.impl == PLB_IMPL_TC) return fail(PLB_E_UNSUPPORTED, "the fp32 sparse kernel has no tensor-core variant");
  }
  *out = s.release();
  return PLB_OK;
}

int plb_sparse_run(plb_sparse* sp, const void* x, void* y, int batch) {
  PLB_REQUIRE(sp != nullptr, "null argument");
  PLB_REQUIRE(batch >= 0, "negative batch");
  if (batch == 0) return PLB_OK;
  PLB_REQUIRE(x && y, "null argument");
  if (sp->dense) return plb_conv_run(sp->dense, static_cast<const int8_t*>(x), y, batch);
  PLB_CUDA(cudaSetDevice(sp->ctx->device));
  SparseGeom g;
  g.batch = batch; g.cin = sp->d.cin; g.cout = sp->d.cout; g.hw = sp->d.h * sp->d.w;
  g.is_int8 = sp->d.is_int8;
  g.out_mode = sp->d.out_dtype == PLB_OUT_I8 ? OUT_I8 : OUT_F32;
  EpiParams e;
  e.scale = sp->scale.as<float>(); e.bias = sp->bias.as<float>(); e.act = sp->d.act; e.alpha = sp->alpha;
  if (sparse_slab_supported(g, x, y))
    return sparse_slab_launch(sp->ctx, g, static_cast<const int8_t*>(x), sp->grp_ptr.as<int>(), sp->grp_idx.p,
                              sp->grp_w.p, e, y);
  return sparse_csr_launch(sp->ctx, g, x, sp->row_ptr.as<int>(), sp->col.as<int>(), sp->val.p, sp->col_val.p,
                           sp->bias_raw.as<float>(), e, y);
}

void plb_sparse_destroy(plb_sparse* sp) {
  if (!sp) return;
  cudaSetDevice(sp->ctx->device);
  cudaStreamSynchronize(sp->ctx->stream);
  if (sp->dense) plb_conv_destroy(sp->dense);
  delete sp;
}

// ------------------------------------------------------------------ glue

int plb_calib_f32_to_i8(plb_ctx* ctx, const float* x, int8_t* q, size_t n, float scale) {
  PLB_REQUIRE(ctx && (n == 0 || (x && q)), "null argument");
  PLB_REQUIRE(scale > 0.f, "scale must be positive");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return calib_f32_to_i8_launch(ctx, x, q, n, scale);
}

int plb_copy_h2d(plb_ctx* ctx, void* dst_device, const void* src_host, size_t bytes) {
  PLB_REQUIRE(ctx && (bytes == 0 || (dst_device && src_host)), "null argument");
  if (bytes == 0) return PLB_OK;
  PLB_CUDA(cudaSetDevice(ctx->device));
  PLB_CUDA(cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return PLB_OK;
}

int plb_copy_d2h(plb_ctx* ctx, void* dst_host, const void* src_device, size_t bytes) {
  PLB_REQUIRE(ctx && (bytes == 0 || (dst_host && src_device)), "null argument");
  if (bytes == 0) return PLB_OK;
  PLB_CUDA(cudaSetDevice(ctx->device));
  PLB_CUDA(cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  // the bytes are only worth having if no kernel in front of them gave up: same check as plb_ctx_sync
  return wait_and_check_status(ctx);
}

int plb_calib_i8_to_f32(plb_ctx* ctx, const int8_t* q, float* y, size_t n, float scale) {
  PLB_REQUIRE(ctx && (n == 0 || (q && y)), "null argument");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return calib_i8_to_f32_launch(ctx, q, y, n, scale);
}

int plb_nchw_to_nhwc_i8(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w, int cpad) {
  PLB_REQUIRE(ctx && x && y, "null argument");
  PLB_REQUIRE(n >= 0 && c > 0 && h > 0 && w > 0, "bad dims");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return nchw_to_nhwc_i8_launch(ctx, x, y, n, c, h, w, cpad);
}

int plb_nhwc_to_nchw(plb_ctx* ctx, const void* x, void* y, int n, int c, int h, int w, int elem_bytes) {
  PLB_REQUIRE(ctx && x && y, "null argument");
  PLB_REQUIRE(n >= 0 && c > 0 && h > 0 && w > 0, "bad dims");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return nhwc_to_nchw_launch(ctx, x, y, n, c, h, w, elem_bytes);
}

int plb_calib_nchw_f32_to_nhwc_i8(plb_ctx* ctx, const float* x, int8_t* y, int n, int c, int h, int w,
                                  int cpad, float scale) {
  PLB_REQUIRE(ctx && x && y, "null argument");
  PLB_REQUIRE(n >= 0 && c > 0 && h > 0 && w > 0 && scale > 0.f, "bad dims or scale");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return calib_nchw_f32_to_nhwc_i8_launch(ctx, x, y, n, c, h, w, cpad, scale);
}

int plb_maxpool_nhwc_i8(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w, int k,
                        int stride, int pad) {
  PLB_REQUIRE(ctx && x && y, "null argument");
  PLB_REQUIRE(n >= 0 && c > 0 && h > 0 && w > 0 && k > 0 && stride > 0 && pad >= 0, "bad dims");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return maxpool_nhwc_i8_launch(ctx, x, y, n, c, h, w, k, stride, pad);
}

int plb_global_avgpool_nhwc_f32(plb_ctx* ctx, const float* x, float* y, int8_t* q, int n, int hw, int c,
                                float scale) {
  PLB_REQUIRE(ctx && x && (y || q), "null argument");
  PLB_REQUIRE(n >= 0 && hw > 0 && c > 0, "bad dims");
  PLB_REQUIRE(!q || scale > 0.f, "scale must be positive");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return global_avgpool_nhwc_f32_launch(ctx, x, y, q, n, hw, c, q ? scale : 1.f);
}

}  // extern "C"
