// CUDA-core kernels: direct / depthwise / sparse convolutions and the fp32<->int8 glue.
// All of them are bandwidth-oriented: coalesced channel-contiguous (NHWC) or
// pixel-contiguous (NCHW sparse) accesses, packed-byte arithmetic, no atomics.
#include "kernels_simple.cuh"

#include "dw_device.cuh"
#include "igemm_tc.cuh"
#include <cstdlib>

namespace plb {

namespace {

using namespace dw;

constexpr int kBlock = 256;

struct OutDev {
  int mode;
  void* y;
  int ldy;
  const float* scale;
  const float* bias;
  int act;
  float alpha;
  const float* residual;
  float* y_f32;
  int8_t* y_i8;
  float inv_next_scale;
};

OutDev to_dev(const OutSpec& o) {
  OutDev d;
  d.mode = o.mode; d.y = o.y; d.ldy = o.ldy;
  d.scale = o.epi.scale; d.bias = o.epi.bias; d.act = o.epi.act; d.alpha = o.epi.alpha;
  d.residual = o.residual; d.y_f32 = o.y_f32; d.y_i8 = o.y_i8; d.inv_next_scale = o.inv_next_scale;
  return d;
}

// The epilogue of one output value; identical arithmetic to the tensor-core kernel.
__device__ __forceinline__ void emit(const OutDev& o, long row, int col, int acc) {
  const long off = row * o.ldy + col;
  if (o.mode == OUT_ACC) {
    static_cast<int32_t*>(o.y)[off] = acc;
    return;
  }
  float v = fmaf(static_cast<float>(acc), o.scale[col], o.bias[col]);
  if (o.mode == OUT_ADD_RELU) {
    if (o.residual) v += o.residual[off];
    v = v > 0.f ? v : 0.f;
    if (o.y_f32) o.y_f32[off] = v;
    if (o.y_i8) o.y_i8[off] = static_cast<int8_t>(calib_i8(v, o.inv_next_scale));
    return;
  }
  v = act_apply(v, o.act, o.alpha);
  if (o.mode == OUT_F32)
    static_cast<float*>(o.y)[off] = v;
  else
    static_cast<int8_t*>(o.y)[off] = static_cast<int8_t>(requant_i8(v));
}

// ------------------------------------------------------------------ direct convolution
__global__ void __launch_bounds__(kBlock)
    conv_direct_kernel(const ConvGeom g, const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                       const OutDev o, const long total) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total) return;
  const int co = static_cast<int>(idx % g.cout);
  const long m = idx / g.cout;
  const int ow = static_cast<int>(m % g.wo);
  const int oh = static_cast<int>((m / g.wo) % g.ho);
  const long n = m / (static_cast<long>(g.wo) * g.ho);
  const int cog = g.cout / g.groups, cig = g.cin / g.groups;
  const int grp = co / cog;
  const bool vec4 = (cig & 3) == 0 && (g.cin_stride & 3) == 0 && (g.cg_pad & 3) == 0;
  int acc = 0;
  for (int r = 0; r < g.kh; ++r) {
    const int ih = oh * g.stride_h - g.pad_t + r * g.dil_h;
    if (ih < 0 || ih >= g.h) continue;
    for (int s = 0; s < g.kw; ++s) {
      const int iw = ow * g.stride_w - g.pad_l + s * g.dil_w;
      if (iw < 0 || iw >= g.w) continue;
      const int8_t* xp = x + ((n * g.h + ih) * g.w + iw) * g.cin_stride + grp * cig;
      const int8_t* wp = w + (static_cast<long>(co) * g.kh * g.kw + r * g.kw + s) * g.cg_pad;
      if (vec4) {
        const int* xp4 = reinterpret_cast<const int*>(xp);
        const int* wp4 = reinterpret_cast<const int*>(wp);
        for (int c = 0; c < cig / 4; ++c) acc = __dp4a(xp4[c], wp4[c], acc);
      } else {
        for (int c = 0; c < cig; ++c) acc += static_cast<int>(xp[c]) * static_cast<int>(wp[c]);
      }
    }
  }
  emit(o, m, co, acc);
}

// ------------------------------------------------------------------ depthwise convolution
// One thread = one output pixel x 4 consecutive channels (one 32-bit load per tap).
__global__ void __launch_bounds__(kBlock)
    dwconv_kernel(const ConvGeom g, const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                  const OutDev o, const long total, const int cquads) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total) return;
  const int cq = static_cast<int>(idx % cquads);
  const long m = idx / cquads;
  const int ow = static_cast<int>(m % g.wo);
  const int oh = static_cast<int>((m / g.wo) % g.ho);
  const long n = m / (static_cast<long>(g.wo) * g.ho);
  int acc[4] = {0, 0, 0, 0};
  for (int r = 0; r < g.kh; ++r) {
    const int ih = oh * g.stride_h - g.pad_t + r * g.dil_h;
    if (ih < 0 || ih >= g.h) continue;
    for (int s = 0; s < g.kw; ++s) {
      const int iw = ow * g.stride_w - g.pad_l + s * g.dil_w;
      if (iw < 0 || iw >= g.w) continue;
      const uint32_t xv = *reinterpret_cast<const uint32_t*>(
          x + ((n * g.h + ih) * g.w + iw) * g.cin_stride + cq * 4);
      const uint32_t wv =
          *reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * g.kw + s) * g.cg_pad + cq * 4);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        acc[j] += static_cast<int>(static_cast<int8_t>(xv >> (8 * j))) *
                  static_cast<int>(static_cast<int8_t>(wv >> (8 * j)));
    }
  }
  const int c0 = cq * 4;
  if (o.mode == OUT_I8 && c0 + 3 < g.cout && (o.ldy & 3) == 0) {
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      q[j] = requant_i8(act_apply(fmaf(static_cast<float>(acc[j]), o.scale[c0 + j], o.bias[c0 + j]),
                                  o.act, o.alpha));
    *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(o.y) + m * o.ldy + c0) =
        pack4(q[0], q[1], q[2], q[3]);
    return;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c0 + j < g.cout) emit(o, m, c0 + j, acc[j]);
}

// ------------------------------------------------------------------ depthwise 3x3, register tiled
// One thread = 4 consecutive channels (one 32-bit word of an NHWC pixel) x a 2 x 4 (stride 1) or
// 1 x 4 (stride 2) patch of output pixels.  Every input word is loaded once.  The words of four
// neighbouring pixels are byte-transposed, so that a register holds four consecutive pixels of
// ONE channel; a filter row is packed the same way as (w0, w1, w2, 0), and one dp4a then adds a
// whole filter row to an output: 3 dp4a per output instead of 9 multiply-adds plus unpacking.
// The window of output column j starts j*stride bytes into the transposed row (funnel shift).
// |sum| <= 9*127*127 < 2^22, so int -> float goes through the mantissa of 1.5*2^23 exactly,
// without the slow conversion pipe.


template <int ACT>
__device__ __forceinline__ float dw_act(float v, float alpha) {
  if (ACT == PLB_ACT_RELU) return fmaxf(v, 0.f);
  if (ACT == PLB_ACT_RELU6) return fminf(fmaxf(v, 0.f), alpha);
  if (ACT == PLB_ACT_LEAKY) return v <= 0.f ? alpha * v : v;
  return v;
}

template <int S, int ACT, bool OUT_IS_I8>
__global__ void __launch_bounds__(kBlock)
    dwconv3x3_kernel(const ConvGeom g, const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                     const OutDev o, const int cquads, const int tiles_x, const int tiles_y, const long total) {
  pdl_sync_with_previous_kernel();
  constexpr int TH = S == 1 ? 2 : 1, TW = 4;
  constexpr int IH = (TH - 1) * S + 3, IW = (TW - 1) * S + 3;  // 4 x 6 or 3 x 9 input pixels
  // grid = (channel quads x tile columns, tile rows, images): one division per thread
  const int idx = blockIdx.x * kBlock + threadIdx.x;
  if (idx >= cquads * tiles_x) return;
  const int tx = idx / cquads;
  const int cq = idx - tx * cquads;
  const int ty = blockIdx.y;
  const long n = blockIdx.z;
  (void)tiles_y;
  (void)total;
  const int oh0 = ty * TH, ow0 = tx * TW;
  const int c0 = cq * 4;

  // filter rows as (w0, w1, w2, 0) per channel
  uint32_t wr[3][4];
#pragma unroll
  for (int r = 0; r < 3; ++r)
    transpose4x4(__ldg(reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * 3 + 0) * g.cg_pad + c0)),
                 __ldg(reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * 3 + 1) * g.cg_pad + c0)),
                 __ldg(reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * 3 + 2) * g.cg_pad + c0)), 0u, wr[r]);

  int acc[TH][TW][4];
#pragma unroll
  for (int a = 0; a < TH; ++a)
#pragma unroll
    for (int b = 0; b < TW; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0;

  const int ih0 = oh0 * S - g.pad_t, iw0 = ow0 * S - g.pad_l;
  const int8_t* xn = x + n * g.h * static_cast<long>(g.w) * g.cin_stride + c0;
  // all loads of the patch are issued before any arithmetic: one register per 4 input bytes
  uint32_t raw[IH][IW];
  if (ih0 >= 0 && ih0 + IH <= g.h && iw0 >= 0 && iw0 + IW <= g.w) {
    // interior patch: no bounds tests, one pointer per row
    const int8_t* row = xn + (static_cast<long>(ih0) * g.w + iw0) * g.cin_stride;
    const long row_step = static_cast<long>(g.w) * g.cin_stride;
#pragma unroll
    for (int iy = 0; iy < IH; ++iy, row += row_step) {
#pragma unroll
      for (int ix = 0; ix < IW; ++ix)
        raw[iy][ix] = __ldg(reinterpret_cast<const uint32_t*>(row + ix * g.cin_stride));
    }
  } else {
#pragma unroll
    for (int iy = 0; iy < IH; ++iy) {
      const int ih = ih0 + iy;
      const bool row_ok = ih >= 0 && ih < g.h;
#pragma unroll
      for (int ix = 0; ix < IW; ++ix) {
        const int iw = iw0 + ix;
        raw[iy][ix] = 0;
        if (row_ok && iw >= 0 && iw < g.w)
          raw[iy][ix] = __ldg(reinterpret_cast<const uint32_t*>(xn + (static_cast<long>(ih) * g.w + iw) * g.cin_stride));
      }
    }
  }
#pragma unroll
  for (int iy = 0; iy < IH; ++iy) {
    // win[j][c]: bytes = the three input pixels under output column j (fourth byte meets weight 0)
    uint32_t win[TW][4];
    uint32_t ta[4];
    transpose4x4(raw[iy][0], raw[iy][1], raw[iy][2], raw[iy][3], ta);
    if (S == 1) {
      // pixels 4 and 5 of the row: only their two low bytes per channel are ever multiplied
      const uint32_t t0 = __byte_perm(raw[iy][4], raw[iy][5], 0x5140), t1 = __byte_perm(raw[iy][4], raw[iy][5], 0x7362);
      const uint32_t tb[4] = {t0, t0 >> 16, t1, t1 >> 16};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        win[0][c] = ta[c];
        win[1][c] = __funnelshift_r(ta[c], tb[c], 8);
        win[2][c] = __funnelshift_r(ta[c], tb[c], 16);
        win[3][c] = __funnelshift_r(ta[c], tb[c], 24);
      }
    } else {
      uint32_t tb[4];
      transpose4x4(raw[iy][4], raw[iy][5], raw[iy][6], raw[iy][7], tb);
      const uint32_t last = raw[iy][IW - 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        win[0][c] = ta[c];
        win[1][c] = __funnelshift_r(ta[c], tb[c], 16);
        win[2][c] = tb[c];
        win[3][c] = __funnelshift_r(tb[c], last >> (8 * c), 16);
      }
    }
#pragma unroll
    for (int oy = 0; oy < TH; ++oy) {
      const int r = iy - oy * S;  // filter row this input row meets for output row oy
      if (r < 0 || r > 2) continue;
#pragma unroll
      for (int ox = 0; ox < TW; ++ox)
#pragma unroll
        for (int c = 0; c < 4; ++c)
          acc[oy][ox][c] = __dp4a(static_cast<int>(win[ox][c]), static_cast<int>(wr[r][c]), acc[oy][ox][c]);
    }
  }

  const float4 sc = *reinterpret_cast<const float4*>(o.scale + c0);
  const float4 bi = *reinterpret_cast<const float4*>(o.bias + c0);
  const float alpha = OUT_IS_I8 && ACT == PLB_ACT_RELU6 ? fmaxf(fminf(o.alpha, 127.f), -127.f) : o.alpha;
#pragma unroll
  for (int oy = 0; oy < TH; ++oy) {
    const int oh = oh0 + oy;
    if (oh >= g.ho) continue;
#pragma unroll
    for (int ox = 0; ox < TW; ++ox) {
      const int ow = ow0 + ox;
      if (ow >= g.wo) continue;
      const long m = (n * g.ho + oh) * g.wo + ow;
      float f[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) f[c] = __int_as_float(acc[oy][ox][c] + 0x4B400000) - 12582912.f;  // exact (float)acc
      float v[4] = {fmaf(f[0], sc.x, bi.x), fmaf(f[1], sc.y, bi.y), fmaf(f[2], sc.z, bi.z), fmaf(f[3], sc.w, bi.w)};
      if (OUT_IS_I8) {
        uint32_t q[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float t = v[c];
          if (ACT == PLB_ACT_NONE) t = fminf(fmaxf(t, -127.f), 127.f);
          else if (ACT == PLB_ACT_RELU) t = fminf(fmaxf(t, 0.f), 127.f);
          else if (ACT == PLB_ACT_RELU6) t = fminf(fmaxf(t, 0.f), alpha);
          else { t = t <= 0.f ? alpha * t : t; t = fminf(fmaxf(t, -127.f), 127.f); }
          q[c] = __float_as_uint(t + 12582912.f);  // round to nearest even, result in the low byte
        }
        *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(o.y) + m * o.ldy + c0) =
            __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
      } else {
        *reinterpret_cast<float4*>(static_cast<float*>(o.y) + m * o.ldy + c0) =
            make_float4(dw_act<ACT>(v[0], alpha), dw_act<ACT>(v[1], alpha), dw_act<ACT>(v[2], alpha),
                        dw_act<ACT>(v[3], alpha));
      }
    }
  }
}

typedef void (*DwKernel)(const ConvGeom, const int8_t*, const int8_t*, const OutDev, const int, const int,
                         const int, const long);
template <int S, bool I8>
DwKernel pick_dw_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return dwconv3x3_kernel<S, PLB_ACT_RELU, I8>;
    case PLB_ACT_RELU6: return dwconv3x3_kernel<S, PLB_ACT_RELU6, I8>;
    case PLB_ACT_LEAKY: return dwconv3x3_kernel<S, PLB_ACT_LEAKY, I8>;
    default: return dwconv3x3_kernel<S, PLB_ACT_NONE, I8>;
  }
}

// ------------------------------------------------------------------ depthwise 3x3, column strips
// Same arithmetic as dwconv3x3_kernel, other traversal: a thread owns 4 channels x 4 output columns
// and slides DOWN a strip of output rows.  Every input row of the strip is loaded, transposed and
// shifted once and meets all three filter rows (stride 1) in the same step; accumulator rows rotate
// through registers with compile-time indices, and the row completed by a step is requantised and
// stored in that step.  Column predicates, pointers and the filter are set up once per strip, so
// that the per-output cost is the 3 dp4a, the 5-instruction requantiser and little else.
// Accumulators start at the bit pattern of 1.5*2^23: the integer sum then IS the float 1.5*2^23 + sum.


// fp32 work is done two channels at a time with the packed f32x2 instructions (same IEEE results per lane).
template <int ACT, bool OUT_IS_I8>
__device__ __forceinline__ void dw_emit_row(int (&a)[4][4], const float4 sc, const float4 bi, const float alpha,
                                            const float ub, void* __restrict__ y, const long yoff, const int ldy,
                                            const int ncols) {
  const float2 magic = make_float2(12582912.f, 12582912.f), neg_magic = make_float2(-12582912.f, -12582912.f);
#pragma unroll
  for (int ox = 0; ox < 4; ++ox) {
    const float2 v01 = __ffma2_rn(__fadd2_rn(make_float2(__int_as_float(a[ox][0]), __int_as_float(a[ox][1])), neg_magic),
                                  make_float2(sc.x, sc.y), make_float2(bi.x, bi.y));
    const float2 v23 = __ffma2_rn(__fadd2_rn(make_float2(__int_as_float(a[ox][2]), __int_as_float(a[ox][3])), neg_magic),
                                  make_float2(sc.z, sc.w), make_float2(bi.z, bi.w));
    float v[4] = {v01.x, v01.y, v23.x, v23.y};
#pragma unroll
    for (int c = 0; c < 4; ++c) a[ox][c] = kDwMagic;
    if (ox >= ncols) continue;
    if (OUT_IS_I8) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float t = v[c];
        if (ACT == PLB_ACT_NONE) t = fminf(fmaxf(t, -127.f), 127.f);
        else if (ACT == PLB_ACT_RELU) t = fminf(fmaxf(t, 0.f), 127.f);
        else if (ACT == PLB_ACT_RELU6) t = fminf(fmaxf(t, 0.f), ub);
        else { t = t <= 0.f ? alpha * t : t; t = fminf(fmaxf(t, -127.f), 127.f); }
        v[c] = t;
      }
      // + 1.5*2^23 (after the clamp, where the add is exact): round to nearest even, result in the low byte
      const float2 q01 = __fadd2_rn(make_float2(v[0], v[1]), magic), q23 = __fadd2_rn(make_float2(v[2], v[3]), magic);
      *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(y) + yoff + static_cast<long>(ox) * ldy) =
          __byte_perm(__byte_perm(__float_as_uint(q01.x), __float_as_uint(q01.y), 0x0040),
                      __byte_perm(__float_as_uint(q23.x), __float_as_uint(q23.y), 0x0040), 0x5410);
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(y) + yoff + static_cast<long>(ox) * ldy) =
          make_float4(dw_act<ACT>(v[0], alpha), dw_act<ACT>(v[1], alpha), dw_act<ACT>(v[2], alpha),
                      dw_act<ACT>(v[3], alpha));
    }
  }
}

constexpr int kDwBlock = 128;  // four blocks per SM at <= 128 registers: finer scheduling than two of 256

template <int S, int ACT, bool OUT_IS_I8, int CS>
__global__ void __launch_bounds__(kDwBlock, 4)
    dwconv3x3_strip_kernel(const ConvGeom g, const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                           const OutDev o, const int cquads, const int tiles_x, const int strip_rows) {
  pdl_sync_with_previous_kernel();
  constexpr int IW = 3 * S + 3;
  const int idx = blockIdx.x * kDwBlock + threadIdx.x;
  if (idx >= cquads * tiles_x) return;
  const int tx = idx / cquads;
  const int cq = idx - tx * cquads;
  const int oh0 = blockIdx.y * strip_rows;
  const int rows = min(strip_rows, g.ho - oh0);
  const long n = blockIdx.z;
  const int ow0 = tx * 4, c0 = cq * 4;
  // CS != 0: pixel pitch of input and output known at compile time (immediate load / store offsets)
  const int cs = CS ? CS : g.cin_stride;
  const int ldy = CS ? CS : o.ldy;

  uint32_t wr[3][4];
#pragma unroll
  for (int r = 0; r < 3; ++r)
    transpose4x4(__ldg(reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * 3 + 0) * g.cg_pad + c0)),
                 __ldg(reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * 3 + 1) * g.cg_pad + c0)),
                 __ldg(reinterpret_cast<const uint32_t*>(w + static_cast<long>(r * 3 + 2) * g.cg_pad + c0)), 0u, wr[r]);
  const float4 sc = *reinterpret_cast<const float4*>(o.scale + c0);
  const float4 bi = *reinterpret_cast<const float4*>(o.bias + c0);
  const float alpha = o.alpha;
  const float ub = ACT == PLB_ACT_RELU6 ? fmaxf(fminf(o.alpha, 127.f), -127.f) : 127.f;

  const int ih0 = oh0 * S - g.pad_t, iw0 = ow0 * S - g.pad_l;
  uint32_t colmask = 0;
#pragma unroll
  for (int ix = 0; ix < IW; ++ix)
    if (iw0 + ix >= 0 && iw0 + ix < g.w) colmask |= 1u << ix;
  const long row_step = static_cast<long>(g.w) * cs;
  // byte offset of (image n, input row ih0, column iw0, channel c0); rows / columns outside the image
  // are never dereferenced
  const int8_t* xrow = x + (((n * g.h + ih0) * g.w + iw0) * static_cast<long>(cs) + c0);
  const int ncols = g.wo - ow0;
  long yoff = ((n * g.ho + oh0) * g.wo + ow0) * static_cast<long>(ldy) + c0;
  const long yrow = static_cast<long>(g.wo) * ldy;
  const int in_rows = (rows - 1) * S + 3;  // input rows this strip touches

  uint32_t win[4][4];
  if (S == 1) {
    // step iy (P = iy % 3): filter row 0 -> output row iy, row 1 -> iy-1, row 2 -> iy-2 (then complete)
    int acc[3][4][4];
#pragma unroll
    for (int p = 0; p < 3; ++p)
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[p][a][c] = kDwMagic;
    // the three rows of the next iteration are fetched while this iteration's rows are used
    uint32_t cur[3][6], nxt[3][6];
#pragma unroll
    for (int P = 0; P < 3; ++P) {
      dw_load_raw<1>(xrow, cs, P < in_rows && static_cast<unsigned>(ih0 + P) < static_cast<unsigned>(g.h), colmask, cur[P]);
      xrow += row_step;
    }
    // unrolled by two: the copy of the prefetched rows into the current ones becomes a renaming
#pragma unroll 2
    for (int iy = 0; iy < in_rows; iy += 3) {
#pragma unroll
      for (int P = 0; P < 3; ++P) {
        const int ir = iy + 3 + P;
        dw_load_raw<1>(xrow, cs, ir < in_rows && static_cast<unsigned>(ih0 + ir) < static_cast<unsigned>(g.h), colmask, nxt[P]);
        xrow += row_step;
      }
#pragma unroll
      for (int P = 0; P < 3; ++P) {
        const int ir = iy + P;
        dw_make_win<1>(cur[P], win);
        dw_mac(acc[P], win, wr[0]);
        dw_mac(acc[(P + 2) % 3], win, wr[1]);
        dw_mac(acc[(P + 1) % 3], win, wr[2]);
        const int oy = ir - 2;
        if (oy >= 0 && oy < rows) {
          dw_emit_row<ACT, OUT_IS_I8>(acc[(P + 1) % 3], sc, bi, alpha, ub, o.y, yoff, ldy, ncols);
          yoff += yrow;
        } else {
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[(P + 1) % 3][a][c] = kDwMagic;
        }
      }
#pragma unroll
      for (int P = 0; P < 3; ++P)
#pragma unroll
        for (int ix = 0; ix < 6; ++ix) cur[P][ix] = nxt[P][ix];
    }
  } else {
    // input row 2k: filter row 0 of output k and filter row 2 of output k-1 (then complete); row 2k+1: filter row 1
    int acc[2][4][4];
#pragma unroll
    for (int p = 0; p < 2; ++p)
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[p][a][c] = kDwMagic;
    // two rows (one output row) are fetched ahead of the two in use
    uint32_t cur[2][9], nxt[2][9];
#pragma unroll
    for (int P = 0; P < 2; ++P) {
      dw_load_raw<2>(xrow, cs, P < in_rows && static_cast<unsigned>(ih0 + P) < static_cast<unsigned>(g.h), colmask, cur[P]);
      xrow += row_step;
    }
    for (int iy = 0; iy < in_rows; iy += 4) {
#pragma unroll
      for (int P = 0; P < 2; ++P) {
        const int ir = iy + 2 * P;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int in = ir + 2 + q;
          dw_load_raw<2>(xrow, cs, in < in_rows && static_cast<unsigned>(ih0 + in) < static_cast<unsigned>(g.h), colmask, nxt[q]);
          xrow += row_step;
        }
        dw_make_win<2>(cur[0], win);
        dw_mac(acc[P], win, wr[0]);
        dw_mac(acc[P ^ 1], win, wr[2]);
        const int oy = (ir >> 1) - 1;
        if (oy >= 0 && oy < rows) {
          dw_emit_row<ACT, OUT_IS_I8>(acc[P ^ 1], sc, bi, alpha, ub, o.y, yoff, ldy, ncols);
          yoff += yrow;
        } else {
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[P ^ 1][a][c] = kDwMagic;
        }
        dw_make_win<2>(cur[1], win);
        dw_mac(acc[P], win, wr[1]);
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
          for (int ix = 0; ix < 9; ++ix) cur[q][ix] = nxt[q][ix];
      }
    }
  }
}

typedef void (*DwStripKernel)(const ConvGeom, const int8_t*, const int8_t*, const OutDev, const int, const int,
                              const int);
template <int S, bool I8, int CS>
DwStripKernel pick_dw_strip_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return dwconv3x3_strip_kernel<S, PLB_ACT_RELU, I8, CS>;
    case PLB_ACT_RELU6: return dwconv3x3_strip_kernel<S, PLB_ACT_RELU6, I8, CS>;
    case PLB_ACT_LEAKY: return dwconv3x3_strip_kernel<S, PLB_ACT_LEAKY, I8, CS>;
    default: return dwconv3x3_strip_kernel<S, PLB_ACT_NONE, I8, CS>;
  }
}
// int8 output with the usual channel counts as pixel pitch gets the compile-time-pitch variants
template <int S>
DwStripKernel pick_dw_strip(bool i8, int act, int pitch) {
  if (!i8) return pick_dw_strip_act<S, false, 0>(act);
  switch (pitch) {
    case 32: return pick_dw_strip_act<S, true, 32>(act);
    case 64: return pick_dw_strip_act<S, true, 64>(act);
    case 128: return pick_dw_strip_act<S, true, 128>(act);
    case 256: return pick_dw_strip_act<S, true, 256>(act);
    case 512: return pick_dw_strip_act<S, true, 512>(act);
    case 1024: return pick_dw_strip_act<S, true, 1024>(act);
    default: return pick_dw_strip_act<S, true, 0>(act);
  }
}

// ------------------------------------------------------------------ sparse 1x1 convolution
// NCHW.  grid = (pixel blocks, cout, batch).  Each thread owns VEC consecutive pixels of one
// output channel and walks that channel's non-zero weights in ascending input channel, the
// order the reference kernels use.
template <int VEC>
__global__ void __launch_bounds__(kBlock)
    sparse_i8_kernel(const SparseGeom g, const int8_t* __restrict__ x, const int* __restrict__ row_ptr,
                     const int* __restrict__ col, const int8_t* __restrict__ val, const EpiParams e,
                     void* __restrict__ y) {
  pdl_sync_with_previous_kernel();
  const int p = (blockIdx.x * kBlock + threadIdx.x) * VEC;
  if (p >= g.hw) return;
  const int oc = blockIdx.y;
  const long n = blockIdx.z;
  const int8_t* xb = x + n * g.cin * static_cast<long>(g.hw) + p;
  int acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0;
  const int t1 = row_ptr[oc + 1];
  for (int t = row_ptr[oc]; t < t1; ++t) {
    const int wv = val[t];
    const int8_t* xp = xb + static_cast<long>(col[t]) * g.hw;
    if (VEC == 4) {
      const uint32_t xv = *reinterpret_cast<const uint32_t*>(xp);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += wv * static_cast<int>(static_cast<int8_t>(xv >> (8 * j)));
    } else {
      acc[0] += wv * static_cast<int>(xp[0]);
    }
  }
  const float sc = e.scale[oc], bi = e.bias[oc];
  const long off = (n * g.cout + oc) * static_cast<long>(g.hw) + p;
  if (g.out_mode == OUT_I8) {
    int q[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      q[j] = requant_i8(act_apply(fmaf(static_cast<float>(acc[j]), sc, bi), e.act, e.alpha));
    if (VEC == 4)
      *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(y) + off) = pack4(q[0], q[1], q[2], q[3]);
    else
      static_cast<int8_t*>(y)[off] = static_cast<int8_t>(q[0]);
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      static_cast<float*>(y)[off + j] =
          act_apply(fmaf(static_cast<float>(acc[j]), sc, bi), e.act, e.alpha);
  }
}

// ---- int8 sparse 1x1, shared-memory slab + dp4a.
// A block owns 1024 consecutive pixels of one image: it stages x[all cin][1024] in shared memory
// once, then each thread produces every output channel for its 4 pixels.  Non-zeros are walked in
// groups of four (ascending input channel, zero padded): four 32-bit shared loads fetch 4 pixels
// of the 4 input channels, a 4x4 byte transpose turns them into one word per pixel, and one dp4a
// per pixel accumulates the 4 products.  Integer sums, so the order does not matter.
__global__ void __launch_bounds__(kBlock)
    sparse_i8_slab_kernel(const SparseGeom g, const int8_t* __restrict__ x, const int* __restrict__ grp_ptr,
                          const uint2* __restrict__ grp_idx, const uint32_t* __restrict__ grp_w,
                          const EpiParams e, void* __restrict__ y) {
  pdl_sync_with_previous_kernel();
  extern __shared__ uint32_t slab[];  // [cin][256 words]
  const long n = blockIdx.y;
  const int p0 = blockIdx.x * 1024;
  const int8_t* xb = x + n * g.cin * static_cast<long>(g.hw);
  for (int c = 0; c < g.cin; ++c) {
    const int p = p0 + threadIdx.x * 4;
    uint32_t v = 0;
    if (p < g.hw) v = __ldg(reinterpret_cast<const uint32_t*>(xb + static_cast<long>(c) * g.hw + p));
    slab[c * 256 + threadIdx.x] = v;
  }
  __syncthreads();
  const int p = p0 + threadIdx.x * 4;
  if (p >= g.hw) return;
  const uint32_t* col = slab + threadIdx.x;
  const bool relu6 = e.act == PLB_ACT_RELU6, i8 = g.out_mode == OUT_I8;
  for (int oc = 0; oc < g.cout; ++oc) {
    int acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
    const int g1 = grp_ptr[oc + 1];
    for (int t = grp_ptr[oc]; t < g1; ++t) {
      const uint2 idx = __ldg(grp_idx + t);
      const uint32_t wv = __ldg(grp_w + t);
      uint32_t px[4];
      transpose4x4(col[(idx.x & 0xffffu) * 256], col[(idx.x >> 16) * 256], col[(idx.y & 0xffffu) * 256],
                   col[(idx.y >> 16) * 256], px);
      acc0 = __dp4a(static_cast<int>(px[0]), static_cast<int>(wv), acc0);
      acc1 = __dp4a(static_cast<int>(px[1]), static_cast<int>(wv), acc1);
      acc2 = __dp4a(static_cast<int>(px[2]), static_cast<int>(wv), acc2);
      acc3 = __dp4a(static_cast<int>(px[3]), static_cast<int>(wv), acc3);
    }
    const float sc = e.scale[oc], bi = e.bias[oc];
    float v0 = act_apply(fmaf(static_cast<float>(acc0), sc, bi), e.act, e.alpha);
    float v1 = act_apply(fmaf(static_cast<float>(acc1), sc, bi), e.act, e.alpha);
    float v2 = act_apply(fmaf(static_cast<float>(acc2), sc, bi), e.act, e.alpha);
    float v3 = act_apply(fmaf(static_cast<float>(acc3), sc, bi), e.act, e.alpha);
    (void)relu6;
    const long off = (n * g.cout + oc) * static_cast<long>(g.hw) + p;
    if (i8) {
      // clamp, then round to nearest even with the 1.5*2^23 trick (result in the low byte)
      v0 = fminf(fmaxf(v0, -127.f), 127.f) + 12582912.f;
      v1 = fminf(fmaxf(v1, -127.f), 127.f) + 12582912.f;
      v2 = fminf(fmaxf(v2, -127.f), 127.f) + 12582912.f;
      v3 = fminf(fmaxf(v3, -127.f), 127.f) + 12582912.f;
      *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(y) + off) =
          __byte_perm(__byte_perm(__float_as_uint(v0), __float_as_uint(v1), 0x0040),
                      __byte_perm(__float_as_uint(v2), __float_as_uint(v3), 0x0040), 0x5410);
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(y) + off) = make_float4(v0, v1, v2, v3);
    }
  }
}

// fp32: accumulator starts at the bias, one fused multiply-add per non-zero weight.
__global__ void __launch_bounds__(kBlock)
    sparse_f32_kernel(const SparseGeom g, const float* __restrict__ x, const int* __restrict__ row_ptr,
                      const int* __restrict__ col, const float* __restrict__ val,
                      const float* __restrict__ bias, const int act, const float alpha,
                      float* __restrict__ y) {
  pdl_sync_with_previous_kernel();
  const int p = blockIdx.x * kBlock + threadIdx.x;
  if (p >= g.hw) return;
  const int oc = blockIdx.y;
  const long n = blockIdx.z;
  const float* xb = x + n * g.cin * static_cast<long>(g.hw) + p;
  float v = bias ? bias[oc] : 0.f;
  const int t1 = row_ptr[oc + 1];
  for (int t = row_ptr[oc]; t < t1; ++t) v = fmaf(val[t], xb[static_cast<long>(col[t]) * g.hw], v);
  y[(n * g.cout + oc) * static_cast<long>(g.hw) + p] = act_apply(v, act, alpha);
}

// fp32, pixel tiles: a block stages x[all cin][P = 4 * PG pixels] of one image in shared memory.  PG lanes cover the
// tile with one float4 each, so a warp walks 32 / PG output channels at a time; its 8 warps share the channels.  Per
// non-zero a lane group reads one packed {input channel, weight} pair (the same address in all its lanes: a
// broadcast), one float4 of the staged tile and does four fused multiply-adds -- the per-pixel sum is formed exactly as
// in sparse_f32_kernel: bias first, then one fmaf per non-zero in stored (ascending input channel) order.  The loads
// of a tile and the stores of its outputs are full 512-byte rows.
template <int PG>
__global__ void __launch_bounds__(kBlock)
    sparse_f32_tile_kernel(const SparseGeom g, const float* __restrict__ x, const int* __restrict__ row_ptr,
                           const int2* __restrict__ col_val, const float* __restrict__ bias, const int act,
                           const float alpha, float* __restrict__ y) {
  pdl_sync_with_previous_kernel();
  extern __shared__ uint32_t slab[];
  float4* sl = reinterpret_cast<float4*>(slab);  // [cin][PG] float4
  constexpr int P = 4 * PG;
  const long n = blockIdx.y;
  const int p0 = blockIdx.x * P;
  const float* xb = x + n * g.cin * static_cast<long>(g.hw) + p0;
  const int valid = min(P, g.hw - p0);  // a multiple of 4
  for (int i = threadIdx.x; i < g.cin * PG; i += kBlock) {
    const int c = i / PG, q = i - c * PG;
    sl[i] = 4 * q < valid ? __ldg(reinterpret_cast<const float4*>(xb + static_cast<long>(c) * g.hw) + q)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kPerWarp = 32 / PG;             // output channels a warp walks at once
  const int q = lane % PG, sub = lane / PG;
  const bool store = 4 * q < valid;
  for (int oc0 = warp * kPerWarp; oc0 < g.cout; oc0 += (kBlock / 32) * kPerWarp) {
    const int oc = oc0 + sub;
    const bool live = oc < g.cout;
    const float b = (live && bias) ? __ldg(bias + oc) : 0.f;
    float4 acc = make_float4(b, b, b, b);
    int t = live ? __ldg(row_ptr + oc) : 0;
    const int t1 = live ? __ldg(row_ptr + oc + 1) : 0;
    for (; t + 1 < t1; t += 2) {
      const int2 cv0 = __ldg(col_val + t), cv1 = __ldg(col_val + t + 1);
      const float4 x0 = sl[cv0.x * PG + q], x1 = sl[cv1.x * PG + q];
      const float w0 = __int_as_float(cv0.y), w1 = __int_as_float(cv1.y);
      acc.x = fmaf(w0, x0.x, acc.x); acc.y = fmaf(w0, x0.y, acc.y); acc.z = fmaf(w0, x0.z, acc.z); acc.w = fmaf(w0, x0.w, acc.w);
      acc.x = fmaf(w1, x1.x, acc.x); acc.y = fmaf(w1, x1.y, acc.y); acc.z = fmaf(w1, x1.z, acc.z); acc.w = fmaf(w1, x1.w, acc.w);
    }
    if (t < t1) {
      const int2 cv = __ldg(col_val + t);
      const float4 xv = sl[cv.x * PG + q];
      const float w = __int_as_float(cv.y);
      acc.x = fmaf(w, xv.x, acc.x); acc.y = fmaf(w, xv.y, acc.y); acc.z = fmaf(w, xv.z, acc.z); acc.w = fmaf(w, xv.w, acc.w);
    }
    if (live && store)
      *reinterpret_cast<float4*>(y + (n * g.cout + oc) * static_cast<long>(g.hw) + p0 + 4 * q) =
          make_float4(act_apply(acc.x, act, alpha), act_apply(acc.y, act, alpha), act_apply(acc.z, act, alpha),
                      act_apply(acc.w, act, alpha));
  }
}

// fp32 with the input slab in shared memory: a block stages x[all cin][256*VEC pixels] of one
// image and each thread walks every output channel for VEC consecutive pixels.  Per pixel the
// sum is formed exactly as above: bias first, then one fmaf per non-zero in stored order.
template <int VEC>
__global__ void __launch_bounds__(kBlock)
    sparse_f32_slab_kernel(const SparseGeom g, const float* __restrict__ x, const int* __restrict__ row_ptr,
                           const int* __restrict__ col, const float* __restrict__ val,
                           const float* __restrict__ bias, const int act, const float alpha,
                           float* __restrict__ y) {
  pdl_sync_with_previous_kernel();
  extern __shared__ uint32_t slab[];
  float* sl = reinterpret_cast<float*>(slab);  // [cin][256*VEC]
  constexpr int kPix = kBlock * VEC;
  const long n = blockIdx.y;
  const int p = blockIdx.x * kPix + threadIdx.x * VEC;
  const float* xb = x + n * g.cin * static_cast<long>(g.hw);
  for (int c = 0; c < g.cin; ++c) {
    float v[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = 0.f;
    if (p < g.hw) {
      const float* src = xb + static_cast<long>(c) * g.hw + p;
      if (VEC == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(src));
        v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
      } else if (VEC == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2*>(src));
        v[0] = t.x; v[1 % VEC] = t.y;
      } else {
        v[0] = __ldg(src);
      }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) sl[c * kPix + threadIdx.x * VEC + i] = v[i];
  }
  __syncthreads();
  if (p >= g.hw) return;
  const float* colp = sl + threadIdx.x * VEC;
  for (int oc = 0; oc < g.cout; ++oc) {
    float acc[VEC];
    const float b = bias ? bias[oc] : 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = b;
    const int t1 = row_ptr[oc + 1];
    for (int t = row_ptr[oc]; t < t1; ++t) {
      const float wv = __ldg(val + t);
      const float* xs = colp + __ldg(col + t) * kPix;
      if (VEC == 4) {
        const float4 xv = *reinterpret_cast<const float4*>(xs);
        acc[0] = fmaf(wv, xv.x, acc[0]); acc[1 % VEC] = fmaf(wv, xv.y, acc[1 % VEC]);
        acc[2 % VEC] = fmaf(wv, xv.z, acc[2 % VEC]); acc[3 % VEC] = fmaf(wv, xv.w, acc[3 % VEC]);
      } else if (VEC == 2) {
        const float2 xv = *reinterpret_cast<const float2*>(xs);
        acc[0] = fmaf(wv, xv.x, acc[0]); acc[1 % VEC] = fmaf(wv, xv.y, acc[1 % VEC]);
      } else {
        acc[0] = fmaf(wv, xs[0], acc[0]);
      }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = act_apply(acc[i], act, alpha);
    float* dst = y + (n * g.cout + oc) * static_cast<long>(g.hw) + p;
    if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
    else if (VEC == 2) *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1 % VEC]);
    else dst[0] = acc[0];
  }
}

// ------------------------------------------------------------------ glue
__global__ void calib_f32_to_i8_kernel(const float* __restrict__ x, int8_t* __restrict__ q, size_t n,
                                       float inv) {
  pdl_sync_with_previous_kernel();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    q[i] = static_cast<int8_t>(calib_i8(x[i], inv));
}
__global__ void calib_i8_to_f32_kernel(const int8_t* __restrict__ q, float* __restrict__ y, size_t n,
                                       float scale) {
  pdl_sync_with_previous_kernel();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = static_cast<float>(q[i]) * scale;
}

// [n,c,hw] -> [n,hw,cpad]; a block moves a 32-channel x 64-pixel tile through shared memory.
// T = int8_t copies, T = float quantises on the way (calib).
template <typename T>
__global__ void __launch_bounds__(kBlock)
    to_nhwc_i8_kernel(const T* __restrict__ x, int8_t* __restrict__ y, int c, int hw, int cpad,
                      float inv) {
  pdl_sync_with_previous_kernel();
  __shared__ int8_t tile[32][64 + 4];
  const long n = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 64;
  for (int i = threadIdx.x; i < 32 * 64; i += kBlock) {
    const int cc = i >> 6, pp = i & 63;
    int8_t v = 0;
    if (c0 + cc < c && p0 + pp < hw) {
      const T raw = x[(n * c + c0 + cc) * static_cast<long>(hw) + p0 + pp];
      if (sizeof(T) == 1) v = static_cast<int8_t>(raw);
      else v = static_cast<int8_t>(calib_i8(static_cast<float>(raw), inv));
    }
    tile[cc][pp] = v;
  }
  __syncthreads();
  const int pp = threadIdx.x >> 2, cg = threadIdx.x & 3;  // 64 pixels x 4 groups of 8 channels
  if (p0 + pp < hw && c0 + cg * 8 < cpad) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= static_cast<uint32_t>(static_cast<uint8_t>(tile[cg * 8 + j][pp])) << (8 * j);
      hi |= static_cast<uint32_t>(static_cast<uint8_t>(tile[cg * 8 + 4 + j][pp])) << (8 * j);
    }
    *reinterpret_cast<uint2*>(y + (n * hw + p0 + pp) * static_cast<long>(cpad) + c0 + cg * 8) =
        make_uint2(lo, hi);
  }
}

// ---- fast int8 layout staging: 128-pixel x CT-channel tiles through shared memory, 128-bit
// global accesses on the pixel-contiguous (NCHW) side, 4x4 byte transposes with prmt in registers.
// The shared tile is [pixel][17 words] (CT <= 64 channels): odd pitch keeps the row-wise phase
// conflict-free and the strided phase at four-way conflicts.
constexpr int kTilePix = 128;
constexpr int kTilePitchW = 17;  // words per pixel row of the shared tile

// x [n,c,hw] -> y [n,hw,cpad].  grid = (pixel strips, channel tiles, n); block = 256 threads =
// 8 warps; a warp handles 4 channel quads x 8 segments of 16 pixels.  hw % 16 == 0.
__global__ void __launch_bounds__(kBlock)
    nchw_to_nhwc_i8_fast_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int c, int hw, int cpad,
                                int ct) {
  pdl_sync_with_previous_kernel();
  extern __shared__ uint32_t tile_smem[];
  const int cquads = ct / 4;                 // channel quads per tile (8 or 16)
  const int warps_per_strip = cquads / 4;    // 2 or 4
  const int strips = 8 / warps_per_strip;    // 128-pixel strips per block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long n = blockIdx.z;
  const int c0 = blockIdx.y * ct;
  const int p_block = blockIdx.x * strips * kTilePix;
  {
    const int strip = warp / warps_per_strip;
    const int cq = (warp % warps_per_strip) * 4 + (lane >> 3);
    const int seg = lane & 7;
    const int p = p_block + strip * kTilePix + seg * 16;
    uint4 rows[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ch = c0 + cq * 4 + j;
      rows[j] = make_uint4(0, 0, 0, 0);
      if (ch < c && p < hw) rows[j] = __ldg(reinterpret_cast<const uint4*>(x + (n * c + ch) * static_cast<long>(hw) + p));
    }
    const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&rows[0]);
    const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&rows[1]);
    const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&rows[2]);
    const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&rows[3]);
    uint32_t* dst = tile_smem + (strip * kTilePix + seg * 16) * kTilePitchW + cq;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w[4];
      transpose4x4(r0[g], r1[g], r2[g], r3[g], w);
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[(g * 4 + i) * kTilePitchW] = w[i];
    }
  }
  __syncthreads();
  const int words = strips * kTilePix * cquads;
  for (int wi = threadIdx.x; wi < words; wi += kBlock) {
    const int pix = wi / cquads, q = wi - pix * cquads;
    const int p = p_block + pix;
    if (p < hw && c0 + q * 4 < cpad)
      *reinterpret_cast<uint32_t*>(y + (n * hw + p) * static_cast<long>(cpad) + c0 + q * 4) =
          tile_smem[pix * kTilePitchW + q];
  }
}

// x [n,hw,c] -> y [n,c,hw], int8, c % 4 == 0, hw % 16 == 0: the inverse of the kernel above.
__global__ void __launch_bounds__(kBlock)
    nhwc_to_nchw_i8_fast_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int c, int hw, int ct) {
  pdl_sync_with_previous_kernel();
  extern __shared__ uint32_t tile_smem[];
  const int cquads = ct / 4;
  const int warps_per_strip = cquads / 4;
  const int strips = 8 / warps_per_strip;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long n = blockIdx.z;
  const int c0 = blockIdx.y * ct;
  const int p_block = blockIdx.x * strips * kTilePix;
  const int words = strips * kTilePix * cquads;
  for (int wi = threadIdx.x; wi < words; wi += kBlock) {
    const int pix = wi / cquads, q = wi - pix * cquads;
    const int p = p_block + pix;
    uint32_t v = 0;
    if (p < hw && c0 + q * 4 < c)
      v = __ldg(reinterpret_cast<const uint32_t*>(x + (n * hw + p) * static_cast<long>(c) + c0 + q * 4));
    tile_smem[pix * kTilePitchW + q] = v;
  }
  __syncthreads();
  const int strip = warp / warps_per_strip;
  const int cq = (warp % warps_per_strip) * 4 + (lane >> 3);
  const int seg = lane & 7;
  const int p = p_block + strip * kTilePix + seg * 16;
  const uint32_t* src = tile_smem + (strip * kTilePix + seg * 16) * kTilePitchW + cq;
  uint32_t out[4][4];  // [channel j][group g] = 4 pixels of channel j
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t w[4];
    transpose4x4(src[(g * 4 + 0) * kTilePitchW], src[(g * 4 + 1) * kTilePitchW], src[(g * 4 + 2) * kTilePitchW],
                 src[(g * 4 + 3) * kTilePitchW], w);
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j][g] = w[j];
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int ch = c0 + cq * 4 + j;
    if (ch < c && p < hw)
      *reinterpret_cast<uint4*>(y + (n * c + ch) * static_cast<long>(hw) + p) =
          make_uint4(out[j][0], out[j][1], out[j][2], out[j][3]);
  }
}

// Folded staging for stem layers with few input channels (cin * kw <= 32).  One staged pixel
// (t, q) holds, for fh = stride_h consecutive input rows, the kw taps of the filter row and the
// input channels:  y[n][t][q][e*32 + s*cin + c] = x[n][c][t*fh - pad_t + e][q*stride_w - pad_l + s*dil_w]
// (0 outside the image and in the unused tail of each 32-byte group).  The convolution then
// becomes ceil(kh/fh) x 1, stride 1, no padding, over fh*32 "channels": output row p reads
// staged rows p .. p + ceil(kh/fh) - 1.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    fold_rows_kernel(const T* __restrict__ x, int8_t* __restrict__ y, int c, int h, int w, int ht, int wo,
                     int kw, int fh, int stride_w, int pad_t, int pad_l, int dil_w, float inv, long total) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total) return;  // one thread per (n, t, q, e)
  const int e = static_cast<int>(idx % fh);
  const long pix = idx / fh;
  const int q = static_cast<int>(pix % wo);
  const int t = static_cast<int>((pix / wo) % ht);
  const long n = pix / (static_cast<long>(wo) * ht);
  uint32_t words[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int hh = t * fh - pad_t + e;
  if (hh >= 0 && hh < h) {
    const int w0 = q * stride_w - pad_l;
    for (int s = 0; s < kw; ++s) {
      const int iw = w0 + s * dil_w;
      if (iw < 0 || iw >= w) continue;
      for (int cc = 0; cc < c; ++cc) {
        const T raw = x[((n * c + cc) * h + hh) * static_cast<long>(w) + iw];
        const int v = sizeof(T) == 1 ? static_cast<int>(raw) : calib_i8(static_cast<float>(raw), inv);
        const int j = s * c + cc;
        words[j >> 2] |= static_cast<uint32_t>(v & 0xff) << (8 * (j & 3));
      }
    }
  }
  uint4* dst = reinterpret_cast<uint4*>(y + idx * 32);
  dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
  dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
}

// Same layout through shared memory: a block takes kFoldGroup staged rows of one image, i.e.
// kFoldGroup * fh input rows of every channel, quantises them once into row buffers laid out as
// [pixel][channel] bytes (with the left/right zero padding), where the kw*cin bytes a staged pixel
// needs are contiguous, and then copies one unaligned 32-byte window per (staged pixel, folded
// row).  Lanes are ordered so that a warp writes 1 KiB of consecutive staged bytes.  dil_w == 1.
constexpr int kFoldGroup = 4;

__device__ __forceinline__ int8_t fold_quant(float v, float inv) {
  // calib: sat(rne(max(x * inv, -127))); rounding by adding 1.5 * 2^23
  const float f = fminf(fmaxf(v * inv, -127.f), 127.f) + 12582912.f;
  return static_cast<int8_t>(__float_as_uint(f) & 0xffu);
}
__device__ __forceinline__ int8_t fold_quant(int8_t v, float) { return v; }

template <typename T>
__global__ void __launch_bounds__(kBlock)
    fold_rows_fast_kernel(const T* __restrict__ x, int8_t* __restrict__ y, int c, int h, int w, int ht, int wo,
                          int kw, int fh, int stride_w, int pad_t, int pad_l, float inv, int row_words, int vec4) {
  pdl_sync_with_previous_kernel();
  extern __shared__ uint32_t rowbuf[];  // [rows][row_words]
  int8_t* rb = reinterpret_cast<int8_t*>(rowbuf);
  const int t0 = blockIdx.x * kFoldGroup;
  const long n = blockIdx.y;
  const int rows = min(kFoldGroup, ht - t0) * fh;  // folded input rows this block stages
  const int hh0 = t0 * fh - pad_t;
  for (int i = threadIdx.x; i < rows * row_words; i += kBlock) rowbuf[i] = 0;
  __syncthreads();
  const int pix = (wo - 1) * stride_w + kw;  // padded pixels a row buffer holds
  if (vec4 && sizeof(T) == 4) {
    const int w4 = w >> 2;
    const int items = rows * c * w4;
    for (int i = threadIdx.x; i < items; i += kBlock) {
      const int v4 = i % w4;
      const int rc = i / w4;
      const int cc = rc % c, r = rc / c;
      const int hh = hh0 + r;
      if (hh < 0 || hh >= h) continue;
      const float4 v = __ldg(reinterpret_cast<const float4*>(x + ((n * c + cc) * h + hh) * static_cast<long>(w)) + v4);
      const float f[4] = {v.x, v.y, v.z, v.w};
      int8_t* dst = rb + r * row_words * 4 + cc;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int pos = v4 * 4 + k + pad_l;
        if (pos < pix) dst[pos * c] = fold_quant(f[k], inv);
      }
    }
  } else {
    const int items = rows * c * w;
    for (int i = threadIdx.x; i < items; i += kBlock) {
      const int iw = i % w;
      const int rc = i / w;
      const int cc = rc % c, r = rc / c;
      const int hh = hh0 + r;
      const int pos = iw + pad_l;
      if (hh < 0 || hh >= h || pos >= pix) continue;
      rb[r * row_words * 4 + pos * c + cc] = fold_quant(x[((n * c + cc) * h + hh) * static_cast<long>(w) + iw], inv);
    }
  }
  __syncthreads();
  const int gb = kw * c;  // meaningful bytes of a 32-byte group
  const int per_t = wo * fh;
  const int outs = (rows / fh) * per_t;
  for (int i = threadIdx.x; i < outs; i += kBlock) {
    const int tl = i / per_t;
    const int qe = i - tl * per_t;
    const int q = qe / fh, e = qe - q * fh;
    const int off = q * stride_w * c;
    const uint32_t* src = rowbuf + (tl * fh + e) * row_words + (off >> 2);
    const int sh = (off & 3) * 8;
    uint32_t a[9], o[8];
#pragma unroll
    for (int k = 0; k < 9; ++k) a[k] = src[k];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t v = __funnelshift_r(a[k], a[k + 1], sh);
      const int rem = gb - 4 * k;  // bytes of this word that belong to the group
      o[k] = rem >= 4 ? v : (rem <= 0 ? 0u : (v & ((1u << (8 * rem)) - 1u)));
    }
    uint4* dst = reinterpret_cast<uint4*>(y + (((n * ht + t0 + tl) * wo + q) * static_cast<long>(fh) + e) * 32);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// [n,hw,c] -> [n,c,hw], 32x32 element tiles.
template <typename T>
__global__ void nhwc_to_nchw_kernel(const T* __restrict__ x, T* __restrict__ y, int c, int hw) {
  pdl_sync_with_previous_kernel();
  __shared__ T tile[32][33];
  const long n = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  for (int k = threadIdx.y; k < 32; k += 8) {
    const int p = p0 + k, cc = c0 + threadIdx.x;
    if (p < hw && cc < c) tile[k][threadIdx.x] = x[(n * hw + p) * static_cast<long>(c) + cc];
  }
  __syncthreads();
  for (int k = threadIdx.y; k < 32; k += 8) {
    const int cc = c0 + k, p = p0 + threadIdx.x;
    if (p < hw && cc < c) y[(n * c + cc) * static_cast<long>(hw) + p] = tile[threadIdx.x][k];
  }
}

__global__ void __launch_bounds__(kBlock)
    maxpool_nhwc_i8_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int c4, int h, int w,
                           int ho, int wo, int k, int stride, int pad, long total) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total) return;
  const int cq = static_cast<int>(idx % c4);
  const long m = idx / c4;
  const int ow = static_cast<int>(m % wo);
  const int oh = static_cast<int>((m / wo) % ho);
  const long n = m / (static_cast<long>(wo) * ho);
  uint32_t best = 0x80808080u;  // four times -128
  for (int r = 0; r < k; ++r) {
    const int ih = oh * stride - pad + r;
    if (ih < 0 || ih >= h) continue;
    for (int s = 0; s < k; ++s) {
      const int iw = ow * stride - pad + s;
      if (iw < 0 || iw >= w) continue;
      const uint32_t v = reinterpret_cast<const uint32_t*>(x)[((n * h + ih) * w + iw) * c4 + cq];
      best = __vmaxs4(best, v);
    }
  }
  reinterpret_cast<uint32_t*>(y)[m * c4 + cq] = best;
}

// 16 channels (one 128-bit word) per thread
__global__ void __launch_bounds__(kBlock)
    maxpool_nhwc_i8_v16_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int c16, int h, int w,
                               int ho, int wo, int k, int stride, int pad, long total) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total) return;
  const int cq = static_cast<int>(idx % c16);
  const long m = idx / c16;
  const int ow = static_cast<int>(m % wo);
  const int oh = static_cast<int>((m / wo) % ho);
  const long n = m / (static_cast<long>(wo) * ho);
  uint4 best = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
  for (int r = 0; r < k; ++r) {
    const int ih = oh * stride - pad + r;
    if (ih < 0 || ih >= h) continue;
    for (int s = 0; s < k; ++s) {
      const int iw = ow * stride - pad + s;
      if (iw < 0 || iw >= w) continue;
      const uint4 v = reinterpret_cast<const uint4*>(x)[((n * h + ih) * w + iw) * c16 + cq];
      best.x = __vmaxs4(best.x, v.x);
      best.y = __vmaxs4(best.y, v.y);
      best.z = __vmaxs4(best.z, v.z);
      best.w = __vmaxs4(best.w, v.w);
    }
  }
  reinterpret_cast<uint4*>(y)[m * c16 + cq] = best;
}

// The same for the usual 3 x 3 window: the nine loads are issued together (the generic kernel's loops with a run-time
// window serialise them, one memory latency each).
__global__ void __launch_bounds__(kBlock)
    maxpool3x3_nhwc_i8_v16_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int c16, int h, int w, int ho,
                                  int wo, int stride, int pad, long total) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total) return;
  const int cq = static_cast<int>(idx % c16);
  const long m = idx / c16;
  const int ow = static_cast<int>(m % wo);
  const int oh = static_cast<int>((m / wo) % ho);
  const long n = m / (static_cast<long>(wo) * ho);
  const int ih0 = oh * stride - pad, iw0 = ow * stride - pad;
  const uint4* base = reinterpret_cast<const uint4*>(x) + ((n * h + ih0) * w + iw0) * c16 + cq;
  uint4 v[9];
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const bool inside = static_cast<unsigned>(ih0 + r) < static_cast<unsigned>(h) &&
                          static_cast<unsigned>(iw0 + s) < static_cast<unsigned>(w);
      v[r * 3 + s] = inside ? __ldg(base + (static_cast<long>(r) * w + s) * c16)
                            : make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
    }
  uint4 best = v[0];
#pragma unroll
  for (int i = 1; i < 9; ++i) {
    best.x = __vmaxs4(best.x, v[i].x);
    best.y = __vmaxs4(best.y, v[i].y);
    best.z = __vmaxs4(best.z, v[i].z);
    best.w = __vmaxs4(best.w, v[i].w);
  }
  reinterpret_cast<uint4*>(y)[m * c16 + cq] = best;
}

// x [n,hw,c] -> y [n,c] = (sum over hw in ascending order) / hw; optional calib to int8.
__global__ void global_avgpool_kernel(const float* __restrict__ x, float* __restrict__ y,
                                      int8_t* __restrict__ q, int hw, int c, float inv, long total) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long n = idx / c;
  const int cc = static_cast<int>(idx % c);
  const float* xp = x + n * hw * static_cast<long>(c) + cc;
  // the sum runs in ascending pixel order (the reference's order); the loads of 16 pixels are issued together
  float s = 0.f;
  int p = 0;
  for (; p + 16 <= hw; p += 16) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __ldg(xp + static_cast<long>(p + i) * c);
#pragma unroll
    for (int i = 0; i < 16; ++i) s += v[i];
  }
  for (; p < hw; ++p) s += __ldg(xp + static_cast<long>(p) * c);
  const float v = s / static_cast<float>(hw);
  if (y) y[idx] = v;
  if (q) q[idx] = static_cast<int8_t>(calib_i8(v, inv));
}

unsigned blocks_for(long total) { return static_cast<unsigned>((total + kBlock - 1) / kBlock); }

// ---------------------------------------------------------------- row pitch changes for TMA
// TMA needs rows that start on 16-byte boundaries.  NCHW images whose pixel count is not a multiple of 16
// (14 x 14, 7 x 7 ...) are therefore copied once into rows of `pitch` bytes (a multiple of 16) in front of
// the NCHW-native tensor-core kernel and its output is copied back; both copies are small enough to be
// served by the L2.

// 16 bytes starting at any byte address, from aligned 32-bit loads; words that lie wholly at or beyond `end`
// are not read.
__device__ __forceinline__ uint4 load16_unaligned(const uint8_t* p, const uint8_t* end) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(a & ~static_cast<uintptr_t>(3));
  const uint32_t shift = static_cast<uint32_t>(a & 3) * 8;
  uint32_t v[5];
#pragma unroll
  for (int i = 0; i < 5; ++i) v[i] = reinterpret_cast<const uint8_t*>(w + i) < end ? __ldg(w + i) : 0u;
  return make_uint4(__funnelshift_r(v[0], v[1], shift), __funnelshift_r(v[1], v[2], shift),
                    __funnelshift_r(v[2], v[3], shift), __funnelshift_r(v[3], v[4], shift));
}

// src rows of `len` bytes back to back -> dst rows of `pitch` bytes (16-byte chunks; the tail of a row's last
// chunk holds bytes of the following row, which the consumer's tensor map never reads as data).
__global__ void __launch_bounds__(kBlock) pitch_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                            long rows, int len, int pitch, long total_chunks) {
  pdl_sync_with_previous_kernel();
  const long idx = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (idx >= total_chunks) return;
  const int cpr = pitch / 16;
  const long row = idx / cpr;
  const int j = static_cast<int>(idx - row * cpr);
  const uint8_t* end = src + rows * len;
  *reinterpret_cast<uint4*>(dst + row * pitch + 16 * j) = load16_unaligned(src + row * len + 16 * j, end);
}

// src rows of `pitch` bytes -> dst rows of `len` bytes back to back.  One thread per aligned 16 bytes of dst (the
// rows of dst have no alignment of their own, so a thread's bytes may come from several rows); each aligned
// 32-bit word of dst that lies inside one row is an unaligned 32-bit read of src.
__global__ void __launch_bounds__(kBlock) unpitch_rows_i8_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                                 unsigned len, unsigned pitch, unsigned long long total_bytes) {
  pdl_sync_with_previous_kernel();
  const unsigned long long f0 = 16ull * (static_cast<unsigned long long>(blockIdx.x) * kBlock + threadIdx.x);
  if (f0 >= total_bytes) return;
  unsigned long long row = f0 / len;
  unsigned p = static_cast<unsigned>(f0 - row * len);
  uint32_t out[4];
  int full_words = 0;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const unsigned long long f = f0 + 4ull * w;
    if (f + 4 <= total_bytes && p + 4 <= len) {
      const uint8_t* sp = src + row * pitch + p;
      const uintptr_t a = reinterpret_cast<uintptr_t>(sp);
      const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~static_cast<uintptr_t>(3));
      const uint32_t shift = static_cast<uint32_t>(a & 3) * 8;
      const uint32_t lo = __ldg(q), hi = shift ? __ldg(q + 1) : 0u;  // a shifted read ends inside the row's pitch
      out[w] = __funnelshift_r(lo, hi, shift);
      ++full_words;
      p += 4;
      if (p == len) {
        p = 0;
        ++row;
      }
    } else {
      uint32_t v = 0;
      for (int e = 0; e < 4; ++e) {
        if (f + e < total_bytes) v |= static_cast<uint32_t>(src[row * pitch + p]) << (8 * e);
        if (++p == len) {
          p = 0;
          ++row;
        }
      }
      out[w] = v;
      if (f + 4 <= total_bytes) ++full_words;
    }
  }
  if (full_words == 4) {
    *reinterpret_cast<uint4*>(dst + f0) = make_uint4(out[0], out[1], out[2], out[3]);
  } else {
    for (int e = 0; e < 16 && f0 + e < total_bytes; ++e) dst[f0 + e] = static_cast<uint8_t>(out[e >> 2] >> (8 * (e & 3)));
  }
}

__global__ void __launch_bounds__(kBlock) unpitch_rows_b32_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                                                  int len, int pitch, long total) {
  pdl_sync_with_previous_kernel();
  const long f = static_cast<long>(blockIdx.x) * kBlock + threadIdx.x;
  if (f >= total) return;
  const long row = f / len;
  dst[f] = __ldg(src + row * pitch + (f - row * len));
}

}  // namespace

int pitch_rows_i8_launch(plb_ctx* ctx, const void* src, void* dst, long rows, int len, int pitch) {
  if (rows == 0) return PLB_OK;
  if (pitch % 16 || pitch < len || (reinterpret_cast<uintptr_t>(dst) & 15))
    return fail(PLB_E_INVALID, "row pitch must be a multiple of 16 bytes and the destination 16-byte aligned");
  const long chunks = rows * (pitch / 16);
  PLB_CUDA(launch_kernel(pitch_rows_kernel, dim3(blocks_for(chunks)), dim3(kBlock), 0, ctx->stream,
                         static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, len, pitch, chunks));
  ctx->launches++;
  return PLB_OK;
}

int unpitch_rows_launch(plb_ctx* ctx, const void* src, void* dst, long rows, int len, int pitch, int elem_bytes) {
  if (rows == 0) return PLB_OK;
  const long total = rows * len;
  if (elem_bytes == 1) {
    if (reinterpret_cast<uintptr_t>(dst) & 15) return fail(PLB_E_INVALID, "destination must be 16-byte aligned");
    PLB_CUDA(launch_kernel(unpitch_rows_i8_kernel, dim3(blocks_for((total + 15) / 16)), dim3(kBlock), 0, ctx->stream,
                           static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), static_cast<unsigned>(len),
                           static_cast<unsigned>(pitch), static_cast<unsigned long long>(total)));
  } else if (elem_bytes == 4) {
    PLB_CUDA(launch_kernel(unpitch_rows_b32_kernel, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream,
                           static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), len, pitch, total));
  } else {
    return fail(PLB_E_INVALID, "element size must be 1 or 4");
  }
  ctx->launches++;
  return PLB_OK;
}

int conv_direct_launch(plb_ctx* ctx, const ConvGeom& g, const int8_t* x, const int8_t* w_rsc,
                       const OutSpec& out) {
  const long total = static_cast<long>(g.batch) * g.ho * g.wo * g.cout;
  if (total == 0) return PLB_OK;
  PLB_CUDA(launch_kernel(conv_direct_kernel, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream, g, x, w_rsc, to_dev(out), total));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int dwconv_launch(plb_ctx* ctx, const ConvGeom& g, const int8_t* x, const int8_t* w_tc,
                  const OutSpec& out) {
  const bool tiled = g.kh == 3 && g.kw == 3 && g.dil_h == 1 && g.dil_w == 1 && g.stride_h == g.stride_w &&
                     (g.stride_h == 1 || g.stride_h == 2) && (out.mode == OUT_I8 || out.mode == OUT_F32) &&
                     g.cout % 4 == 0 && out.ldy % 4 == 0 && g.cin_stride % 4 == 0 && g.cg_pad % 4 == 0;
  if (tiled) {
    const int cq = g.cout / 4;
    const int tiles_x = (g.wo + 3) / 4, tiles_y = g.stride_h == 1 ? (g.ho + 1) / 2 : g.ho;
    const long total = static_cast<long>(g.batch) * tiles_y * tiles_x * cq;
    if (total == 0) return PLB_OK;
    const bool i8 = out.mode == OUT_I8;
    // column-strip kernel (default): long strips (few halo rows) as long as every SM still gets two blocks
    int strip = g.dw_strip;  // PLB_DW_STRIP as read when the layer was prepared; -1 = cost model
    const long bx = (static_cast<long>(cq) * tiles_x + kDwBlock - 1) / kDwBlock;
    if (strip < 0) {
      // rows per strip: a block costs (input rows it reads) and the blocks run in waves of four per SM
      const long slots = 4L * ctx->sm_count;
      long best = -1;
      for (int ns = 1; ns <= g.ho; ++ns) {
        const int rows = (g.ho + ns - 1) / ns;
        if (rows > 32 && ns < g.ho) continue;
        if ((g.ho + rows - 1) / rows != ns) continue;
        const long waves = (bx * ns * g.batch + slots - 1) / slots;
        // + a block's fixed part (filter transposes, pointers, the first rows' latency): worth about six rows, measured
        // inside MobileNetV1 (256 images: 0.923 ms per step with two rows, 0.911 - 0.912 with four to sixteen)
        const long cost = waves * ((rows - 1) * g.stride_h + 3 + 6);
        if (best < 0 || cost < best) best = cost, strip = rows;
        if (rows <= 2) break;
      }
    }
    if (strip > 0) {
      const int strips = (g.ho + strip - 1) / strip;
      if (strips > 65535 || g.batch > 65535) return fail(PLB_E_UNSUPPORTED, "depthwise 3x3: more than 65535 strips or images");
      const int pitch = g.cin_stride == static_cast<int>(out.ldy) ? g.cin_stride : 0;
      DwStripKernel ks = g.stride_h == 1 ? pick_dw_strip<1>(i8, out.epi.act, pitch) : pick_dw_strip<2>(i8, out.epi.act, pitch);
      dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(strips), static_cast<unsigned>(g.batch));
      PLB_CUDA(launch_kernel(ks, grid, dim3(kDwBlock), 0, ctx->stream, g, x, w_tc, to_dev(out), cq, tiles_x, strip));
      ctx->launches++;
      return PLB_OK;
    }
    DwKernel k = g.stride_h == 1 ? (i8 ? pick_dw_act<1, true>(out.epi.act) : pick_dw_act<1, false>(out.epi.act))
                                 : (i8 ? pick_dw_act<2, true>(out.epi.act) : pick_dw_act<2, false>(out.epi.act));
    if (tiles_y > 65535 || g.batch > 65535) return fail(PLB_E_UNSUPPORTED, "depthwise 3x3: more than 65535 tile rows or images");
    dim3 grid(static_cast<unsigned>((static_cast<long>(cq) * tiles_x + kBlock - 1) / kBlock), static_cast<unsigned>(tiles_y),
              static_cast<unsigned>(g.batch));
    PLB_CUDA(launch_kernel(k, grid, dim3(kBlock), 0, ctx->stream, g, x, w_tc, to_dev(out), cq, tiles_x, tiles_y, total));
    ctx->launches++;
    return PLB_OK;
  }
  const int cquads = (g.cout + 3) / 4;
  const long total = static_cast<long>(g.batch) * g.ho * g.wo * cquads;
  if (total == 0) return PLB_OK;
  PLB_CUDA(launch_kernel(dwconv_kernel, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream, g, x, w_tc, to_dev(out), total, cquads));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int sparse_slab_supported(const SparseGeom& g, const void* x, const void* y) {
  return g.is_int8 && g.hw % 4 == 0 && g.cin <= 160 && g.cin < 65536 && g.batch <= 65535 &&
         (reinterpret_cast<uintptr_t>(x) & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
}

int sparse_slab_launch(plb_ctx* ctx, const SparseGeom& g, const int8_t* x, const int* grp_ptr,
                       const void* grp_idx, const void* grp_w, const EpiParams& epi, void* y) {
  if (g.batch == 0 || g.hw == 0) return PLB_OK;
  const size_t smem = static_cast<size_t>(g.cin) * 1024;
  PLB_CUDA(cudaFuncSetAttribute(sparse_i8_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 164 * 1024));
  dim3 grid((g.hw + 1023) / 1024, g.batch);
  PLB_CUDA(launch_kernel(sparse_i8_slab_kernel, grid, dim3(kBlock), smem, ctx->stream, g, x, grp_ptr,
                         static_cast<const uint2*>(grp_idx), static_cast<const uint32_t*>(grp_w), epi, y));
  ctx->launches++;
  return PLB_OK;
}

int sparse_csr_launch(plb_ctx* ctx, const SparseGeom& g, const void* x, const int* row_ptr,
                      const int* col, const void* val, const void* col_val, const float* bias_raw,
                      const EpiParams& epi, void* y) {
  if (g.batch == 0 || g.hw == 0) return PLB_OK;
  if (!g.is_int8 && col_val && g.hw % 4 == 0 && g.cin <= 512 && g.batch <= 65535 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    // pixel-tile kernel: the widest tile whose slab stays at 64 KiB, so that two blocks share an SM
    const int pg = g.cin <= 128 ? 32 : (g.cin <= 256 ? 16 : 8);
    auto kern = pg == 32 ? sparse_f32_tile_kernel<32> : (pg == 16 ? sparse_f32_tile_kernel<16> : sparse_f32_tile_kernel<8>);
    const size_t smem = static_cast<size_t>(g.cin) * pg * 16;
    PLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    dim3 grid((g.hw + 4 * pg - 1) / (4 * pg), g.batch);
    PLB_CUDA(launch_kernel(kern, grid, dim3(kBlock), smem, ctx->stream, g, static_cast<const float*>(x), row_ptr,
                           static_cast<const int2*>(col_val), bias_raw, epi.act, epi.alpha, static_cast<float*>(y)));
    ctx->launches++;
    return PLB_OK;
  }
  if (g.cout > 65535 || g.batch > 65535) return fail(PLB_E_UNSUPPORTED, "sparse grid too large");
  if (g.is_int8) {
    const bool vec4 = (g.hw & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 3) == 0 &&
                      (reinterpret_cast<uintptr_t>(y) & 3) == 0;
    if (vec4) {
      dim3 grid((g.hw / 4 + kBlock - 1) / kBlock, g.cout, g.batch);
      PLB_CUDA(launch_kernel(sparse_i8_kernel<4>, dim3(grid), dim3(kBlock), 0, ctx->stream, g, static_cast<const int8_t*>(x), row_ptr, col, static_cast<const int8_t*>(val), epi, y));
    } else {
      dim3 grid((g.hw + kBlock - 1) / kBlock, g.cout, g.batch);
      PLB_CUDA(launch_kernel(sparse_i8_kernel<1>, dim3(grid), dim3(kBlock), 0, ctx->stream, g, static_cast<const int8_t*>(x), row_ptr, col, static_cast<const int8_t*>(val), epi, y));
    }
  } else if (g.cin <= 160 && g.batch <= 65535 && g.hw > 0) {
    // shared-memory slab variant: as many pixels per thread as 160 KB of slab and the alignment allow
    int vec = g.cin <= 40 ? 4 : g.cin <= 80 ? 2 : 1;
    const uintptr_t align = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y);
    while (vec > 1 && (g.hw % vec || (align & (4 * vec - 1)))) vec >>= 1;
    const size_t smem = static_cast<size_t>(g.cin) * kBlock * vec * 4;
    auto kern = vec == 4 ? sparse_f32_slab_kernel<4> : vec == 2 ? sparse_f32_slab_kernel<2> : sparse_f32_slab_kernel<1>;
    PLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 164 * 1024));
    dim3 grid((g.hw + kBlock * vec - 1) / (kBlock * vec), g.batch);
    PLB_CUDA(launch_kernel(kern, grid, dim3(kBlock), smem, ctx->stream, g, static_cast<const float*>(x), row_ptr, col, static_cast<const float*>(val), bias_raw, epi.act, epi.alpha, static_cast<float*>(y)));
  } else {
    dim3 grid((g.hw + kBlock - 1) / kBlock, g.cout, g.batch);
    PLB_CUDA(launch_kernel(sparse_f32_kernel, dim3(grid), dim3(kBlock), 0, ctx->stream, g, static_cast<const float*>(x), row_ptr, col, static_cast<const float*>(val), bias_raw, epi.act, epi.alpha, static_cast<float*>(y)));
  }
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

// Row softmax over the last axis: y = exp(max(x - rowmax, -64)) / sum.  One block per row; the
// row lives in registers between the passes (up to 8 values per thread), longer rows re-read it.
__global__ void __launch_bounds__(kBlock)
    softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int cols) {
  pdl_sync_with_previous_kernel();
  __shared__ float red[kBlock / 32];
  __shared__ float bcast;
  const float* xr = x + static_cast<long>(blockIdx.x) * cols;
  float* yr = y + static_cast<long>(blockIdx.x) * cols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -3.402823466e38f;
  for (int i = threadIdx.x; i < cols; i += kBlock) m = fmaxf(m, xr[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int i = 1; i < kBlock / 32; ++i) t = fmaxf(t, red[i]);
    bcast = t;
  }
  __syncthreads();
  m = bcast;
  float s = 0.f;
  for (int i = threadIdx.x; i < cols; i += kBlock) {
    const float e = expf(fmaxf(xr[i] - m, -64.f));
    yr[i] = e;
    s += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncthreads();  // everyone has read bcast
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < kBlock / 32; ++i) t += red[i];
    bcast = 1.f / t;
  }
  __syncthreads();
  const float inv = bcast;
  for (int i = threadIdx.x; i < cols; i += kBlock) yr[i] *= inv;
}

int softmax_rows_launch(plb_ctx* ctx, const float* x, float* y, int rows, int cols) {
  if (rows == 0) return PLB_OK;
  PLB_CUDA(launch_kernel(softmax_rows_kernel, dim3(static_cast<unsigned>(rows)), dim3(kBlock), 0, ctx->stream, x, y, cols));
  ctx->launches++;
  return PLB_OK;
}

int calib_f32_to_i8_launch(plb_ctx* ctx, const float* x, int8_t* q, size_t n, float scale) {
  if (n == 0) return PLB_OK;
  const unsigned blocks = static_cast<unsigned>(std::min<size_t>((n + kBlock - 1) / kBlock, 148 * 16));
  PLB_CUDA(launch_kernel(calib_f32_to_i8_kernel, dim3(blocks), dim3(kBlock), 0, ctx->stream, x, q, n, 1.f / scale));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int calib_i8_to_f32_launch(plb_ctx* ctx, const int8_t* q, float* y, size_t n, float scale) {
  if (n == 0) return PLB_OK;
  const unsigned blocks = static_cast<unsigned>(std::min<size_t>((n + kBlock - 1) / kBlock, 148 * 16));
  PLB_CUDA(launch_kernel(calib_i8_to_f32_kernel, dim3(blocks), dim3(kBlock), 0, ctx->stream, q, y, n, scale));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int nchw_to_nhwc_i8_launch(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w,
                           int cpad) {
  if (n == 0) return PLB_OK;
  if (cpad % 8 || cpad < c) return fail(PLB_E_INVALID, "cpad must be a multiple of 8 and >= c");
  const int hw = h * w;
  if (hw % 16 == 0 && cpad % 32 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(y) & 3) == 0) {
    const int ct = cpad % 64 == 0 ? 64 : 32;
    const int strips = 8 / (ct / 16);
    dim3 fgrid((hw + strips * kTilePix - 1) / (strips * kTilePix), cpad / ct, n);
    const size_t smem = static_cast<size_t>(strips) * kTilePix * kTilePitchW * 4;
    PLB_CUDA(launch_kernel(nchw_to_nhwc_i8_fast_kernel, fgrid, dim3(kBlock), smem, ctx->stream, x, y, c, hw, cpad, ct));
    ctx->launches++;
    return PLB_OK;
  }
  dim3 grid((hw + 63) / 64, (cpad + 31) / 32, n);
  PLB_CUDA(launch_kernel(to_nhwc_i8_kernel<int8_t>, dim3(grid), dim3(kBlock), 0, ctx->stream, x, y, c, hw, cpad, 1.f));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int calib_nchw_f32_to_nhwc_i8_launch(plb_ctx* ctx, const float* x, int8_t* y, int n, int c, int h,
                                     int w, int cpad, float scale) {
  if (n == 0) return PLB_OK;
  if (cpad % 8 || cpad < c) return fail(PLB_E_INVALID, "cpad must be a multiple of 8 and >= c");
  const int hw = h * w;
  dim3 grid((hw + 63) / 64, (cpad + 31) / 32, n);
  PLB_CUDA(launch_kernel(to_nhwc_i8_kernel<float>, dim3(grid), dim3(kBlock), 0, ctx->stream, x, y, c, hw, cpad, 1.f / scale));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int fold_rows_launch(plb_ctx* ctx, const void* x, int x_is_f32, int8_t* y, int n, int c, int h, int w,
                     int ht, int wo, int kw, int fh, int stride_w, int pad_t, int pad_l, int dil_w,
                     float scale) {
  const long total = static_cast<long>(n) * ht * wo * fh;
  if (total == 0) return PLB_OK;
  if (c * kw > 32) return fail(PLB_E_INVALID, "row folding needs cin * kw <= 32");
  // row buffer: the padded pixels of one input row plus 9 words of slack for the window reads
  const int row_words = (((wo - 1) * stride_w + kw) * c + 3) / 4 + 9;
  if (dil_w == 1 && static_cast<size_t>(row_words) * 4 * kFoldGroup * fh <= 40 * 1024 && n <= 65535) {
    dim3 grid(static_cast<unsigned>((ht + kFoldGroup - 1) / kFoldGroup), static_cast<unsigned>(n));
    const size_t smem = static_cast<size_t>(row_words) * 4 * kFoldGroup * fh;
    const int vec4 = w % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (x_is_f32)
      PLB_CUDA(launch_kernel(fold_rows_fast_kernel<float>, grid, dim3(kBlock), smem, ctx->stream,
                             static_cast<const float*>(x), y, c, h, w, ht, wo, kw, fh, stride_w, pad_t, pad_l,
                             1.f / scale, row_words, vec4));
    else
      PLB_CUDA(launch_kernel(fold_rows_fast_kernel<int8_t>, grid, dim3(kBlock), smem, ctx->stream,
                             static_cast<const int8_t*>(x), y, c, h, w, ht, wo, kw, fh, stride_w, pad_t, pad_l, 1.f,
                             row_words, 0));
    ctx->launches++;
    return PLB_OK;
  }
  if (x_is_f32)
    PLB_CUDA(launch_kernel(fold_rows_kernel<float>, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream,
                           static_cast<const float*>(x), y, c, h, w, ht, wo, kw, fh, stride_w, pad_t, pad_l,
                           dil_w, 1.f / scale, total));
  else
    PLB_CUDA(launch_kernel(fold_rows_kernel<int8_t>, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream,
                           static_cast<const int8_t*>(x), y, c, h, w, ht, wo, kw, fh, stride_w, pad_t, pad_l,
                           dil_w, 1.f, total));
  ctx->launches++;
  return PLB_OK;
}

int nhwc_to_nchw_launch(plb_ctx* ctx, const void* x, void* y, int n, int c, int h, int w,
                        int elem_bytes) {
  if (n == 0) return PLB_OK;
  const int hw = h * w;
  if (elem_bytes == 1 && hw % 16 == 0 && c % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 3) == 0) {
    const int ct = c >= 64 ? 64 : 32;
    const int strips = 8 / (ct / 16);
    dim3 fgrid((hw + strips * kTilePix - 1) / (strips * kTilePix), (c + ct - 1) / ct, n);
    const size_t smem = static_cast<size_t>(strips) * kTilePix * kTilePitchW * 4;
    PLB_CUDA(launch_kernel(nhwc_to_nchw_i8_fast_kernel, fgrid, dim3(kBlock), smem, ctx->stream,
                           static_cast<const int8_t*>(x), static_cast<int8_t*>(y), c, hw, ct));
    ctx->launches++;
    return PLB_OK;
  }
  dim3 grid((hw + 31) / 32, (c + 31) / 32, n), block(32, 8);
  if (elem_bytes == 1)
    PLB_CUDA(launch_kernel(nhwc_to_nchw_kernel<int8_t>, dim3(grid), dim3(block), 0, ctx->stream, static_cast<const int8_t*>(x), static_cast<int8_t*>(y), c, hw));
  else if (elem_bytes == 4)
    PLB_CUDA(launch_kernel(nhwc_to_nchw_kernel<int32_t>, dim3(grid), dim3(block), 0, ctx->stream, static_cast<const int32_t*>(x), static_cast<int32_t*>(y), c, hw));
  else
    return fail(PLB_E_INVALID, "element size must be 1 or 4");
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int maxpool_nhwc_i8_launch(plb_ctx* ctx, const int8_t* x, int8_t* y, int n, int c, int h, int w,
                           int k, int stride, int pad) {
  if (c % 4) return fail(PLB_E_UNSUPPORTED, "max pool needs a channel count that is a multiple of 4");
  const int ho = (h + 2 * pad - k) / stride + 1, wo = (w + 2 * pad - k) / stride + 1;
  if (c % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    const long total16 = static_cast<long>(n) * ho * wo * (c / 16);
    if (total16 == 0) return PLB_OK;
    if (k == 3)
      PLB_CUDA(launch_kernel(maxpool3x3_nhwc_i8_v16_kernel, dim3(blocks_for(total16)), dim3(kBlock), 0, ctx->stream, x, y,
                             c / 16, h, w, ho, wo, stride, pad, total16));
    else
      PLB_CUDA(launch_kernel(maxpool_nhwc_i8_v16_kernel, dim3(blocks_for(total16)), dim3(kBlock), 0, ctx->stream,
                             x, y, c / 16, h, w, ho, wo, k, stride, pad, total16));
    ctx->launches++;
    return PLB_OK;
  }
  const long total = static_cast<long>(n) * ho * wo * (c / 4);
  if (total == 0) return PLB_OK;
  PLB_CUDA(launch_kernel(maxpool_nhwc_i8_kernel, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream, x, y, c / 4, h, w, ho, wo, k, stride, pad, total));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int global_avgpool_nhwc_f32_launch(plb_ctx* ctx, const float* x, float* y, int8_t* q, int n, int hw,
                                   int c, float scale) {
  const long total = static_cast<long>(n) * c;
  if (total == 0) return PLB_OK;
  PLB_CUDA(launch_kernel(global_avgpool_kernel, dim3(blocks_for(total)), dim3(kBlock), 0, ctx->stream, x, y, q, hw, c, 1.f / scale, total));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

}  // namespace plb
