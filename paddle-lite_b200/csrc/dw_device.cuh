// Per-thread building blocks of the depthwise 3x3 convolution, shared by the stand-alone kernels
// (kernels_simple.cu) and the fused depthwise + pointwise kernel (fused_dwpw.cu): a thread owns 4 consecutive
// channels (one 32-bit word of a channels-last pixel) x 4 output columns, turns the words of neighbouring pixels
// into per-channel 3-pixel windows by byte transposes and funnel shifts, and adds one filter row to one output
// with one dp4a.
#pragma once
#include "common.cuh"

namespace plb {
namespace dw {

// Accumulators start at the bit pattern of 1.5*2^23: the integer sum then IS the float 1.5*2^23 + sum.
constexpr int kDwMagic = 0x4B400000;

// Bytes a,b,c,d[i] -> w[i] = {a[i], b[i], c[i], d[i]}: a 4x4 byte transpose in 6 permutes.
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&w)[4]) {
  const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(a, b, 0x7362);
  const uint32_t t2 = __byte_perm(c, d, 0x5140), t3 = __byte_perm(c, d, 0x7362);
  w[0] = __byte_perm(t0, t2, 0x5410);
  w[1] = __byte_perm(t0, t2, 0x7632);
  w[2] = __byte_perm(t1, t3, 0x5410);
  w[3] = __byte_perm(t1, t3, 0x7632);
}

// One input row of a strip: IW words.  rok is the same for all threads of a block (a uniform branch);
// the column mask is per thread.
template <int S>
__device__ __forceinline__ void dw_load_raw(const int8_t* __restrict__ p, const int cs, const bool rok,
                                            const uint32_t colmask, uint32_t (&raw)[3 * S + 3]) {
  constexpr int IW = 3 * S + 3;
#pragma unroll
  for (int ix = 0; ix < IW; ++ix) raw[ix] = 0;
  if (rok) {
#pragma unroll
    for (int ix = 0; ix < IW; ++ix)
      if ((colmask >> ix) & 1u) raw[ix] = __ldg(reinterpret_cast<const uint32_t*>(p + ix * cs));
  }
}

// The words of a row -> the four 3-pixel windows of every channel (win[ox][c]).
template <int S>
__device__ __forceinline__ void dw_make_win(const uint32_t (&raw)[3 * S + 3], uint32_t (&win)[4][4]) {
  constexpr int IW = 3 * S + 3;
  uint32_t ta[4];
  transpose4x4(raw[0], raw[1], raw[2], raw[3], ta);
  if (S == 1) {
    const uint32_t t0 = __byte_perm(raw[4], raw[5], 0x5140), t1 = __byte_perm(raw[4], raw[5], 0x7362);
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
    transpose4x4(raw[4], raw[5], raw[6], raw[7], tb);
    const uint32_t last = raw[IW - 1];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      win[0][c] = ta[c];
      win[1][c] = __funnelshift_r(ta[c], tb[c], 16);
      win[2][c] = tb[c];
      win[3][c] = __funnelshift_r(tb[c], last >> (8 * c), 16);
    }
  }
}

__device__ __forceinline__ void dw_mac(int (&a)[4][4], const uint32_t (&win)[4][4], const uint32_t (&wr)[4]) {
#pragma unroll
  for (int ox = 0; ox < 4; ++ox)
#pragma unroll
    for (int c = 0; c < 4; ++c) a[ox][c] = __dp4a(static_cast<int>(win[ox][c]), static_cast<int>(wr[c]), a[ox][c]);
}

}  // namespace dw
}  // namespace plb
