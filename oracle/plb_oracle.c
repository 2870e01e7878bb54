/*
 * CPU oracle for the int8 conv / depthwise / fc / sparse_conv hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing the library ships may call into this file;
 * it exists so the parity tests, the smoke check and the CPU-baseline leg of the
 * benchmark have an independent statement of the arithmetic.
 *
 * Every function restates, in plain C with exact integer accumulation, what the
 * reference (PaddlePaddle/Paddle-Lite) computes on its x86 int8 path:
 *
 *   conv2d / depthwise_conv2d  lite/kernels/x86/conv_compute.cc:216-472
 *       = im2col<int8_t>       lite/backends/x86/math/avx/conv_utils.cc:1349-1398
 *       + gemm_s8u8            lite/backends/x86/math/gemm_s8u8_compute.h:65-106
 *   epilogue                   lite/backends/x86/math/gemm_s8u8_kernel.cc:31-55,
 *                              :276-290 (int8 store, RNE + clamp to [-127,127]),
 *                              :610-622 (fp32 store)
 *   scale / bias preparation   lite/backends/x86/math/gemm_s8u8_compute.cc:26-98
 *   fc                         lite/kernels/x86/fc_compute.cc:176-269 (GEMM) with the
 *                              per-output-feature scale/bias orientation of
 *                              lite/kernels/arm/fc_compute.cc:207-260
 *   sparse weight encoders     lite/core/optimizer/mir/sparse_conv_detect_pass.cc:35-368
 *   sparse walk (start ptr)    lite/backends/arm/math/sparse_conv_impl.cc:3731-3745,
 *                              lite/backends/arm/math/sparse_semi_conv_impl.cc:1788-1823
 *   calib fp32<->int8          lite/backends/x86/math/calib.cc:25-239
 *
 * Where the AVX2 GEMM differs from exact arithmetic (vpmaddubsw saturates the
 * int16 pair sum, gemm_s8u8_kernel.cc:122-125) this oracle keeps the exact int32
 * sum: the reference's own test keeps operands small enough that the two agree
 * (lite/tests/math/x86_gemm_s8u8_compute_test.cc:131).
 *
 * Canonical epilogue (c = output channel, acc = exact int32 sum):
 *   fp32 out : y = act(fmaf((float)acc, ws[c]*in_s, bias[c]))
 *   int8 out : q = clamp(rne(act'(fmaf((float)acc, ws[c]*in_s/out_s, bias[c]/out_s))), -127, 127)
 *              relu6 bound = alpha/out_s; leaky slope = alpha (or alpha/out_s when
 *              leaky_compat != 0, which mirrors conv_compute.cc:394)
 * The reference evaluates float(acc + 128*sumA)*s + (bias - 128*s*sumA), which is the
 * same value up to fp32 rounding.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_ACT_NONE 0
#define ORC_ACT_RELU 1
#define ORC_ACT_RELU6 2
#define ORC_ACT_LEAKY 3

static int out_size(int in, int pad_a, int pad_b, int k, int dil, int stride) {
  /* lite/operators/conv_op.cc:42-53 */
  return (in + pad_a + pad_b - (dil * (k - 1) + 1)) / stride + 1;
}

int orc_conv_out_hw(int h, int w, int kh, int kw, int sh, int sw, int pt, int pb, int pl,
                    int pr, int dh, int dw, int* ho, int* wo) {
  *ho = out_size(h, pt, pb, kh, dh, sh);
  *wo = out_size(w, pl, pr, kw, dw, sw);
  return (*ho > 0 && *wo > 0) ? 0 : -1;
}

/* Exact int32 accumulators of a grouped NCHW convolution.
 * x [N,Cin,H,W] int8, w [Cout,Cin/groups,kh,kw] int8, acc [N,Cout,Ho,Wo] int32.
 * Same index arithmetic as im2col<int8_t> followed by an exact GEMM. */
int orc_conv_acc_i32(const int8_t* x, const int8_t* w, int32_t* acc, int n, int cin, int h,
                     int wd, int cout, int kh, int kw, int sh, int sw, int pt, int pb, int pl,
                     int pr, int dh, int dw, int groups) {
  int ho, wo;
  if (groups <= 0 || cin % groups || cout % groups) return -1;
  if (orc_conv_out_hw(h, wd, kh, kw, sh, sw, pt, pb, pl, pr, dh, dw, &ho, &wo)) return -1;
  const int cig = cin / groups, cog = cout / groups;
  const long total = (long)n * cout;
#pragma omp parallel for schedule(dynamic, 1)
  for (long idx = 0; idx < total; ++idx) {
    const int b = (int)(idx / cout), co = (int)(idx % cout);
    const int g = co / cog;
    int32_t* out = acc + idx * (long)ho * wo;
    memset(out, 0, sizeof(int32_t) * (size_t)ho * wo);
    for (int ci = 0; ci < cig; ++ci) {
      const int8_t* xin = x + ((long)b * cin + (long)g * cig + ci) * h * wd;
      const int8_t* wk = w + ((long)co * cig + ci) * kh * kw;
      for (int r = 0; r < kh; ++r) {
        for (int s = 0; s < kw; ++s) {
          const int32_t wv = wk[r * kw + s];
          if (wv == 0) continue;
          for (int oh = 0; oh < ho; ++oh) {
            const int ih = oh * sh - pt + r * dh;
            if (ih < 0 || ih >= h) continue;
            const int8_t* xrow = xin + (long)ih * wd;
            int32_t* orow = out + (long)oh * wo;
            /* valid ow range: 0 <= ow*sw - pl + s*dw < wd */
            const int off = s * dw - pl;
            int ow0 = 0;
            if (off < 0) ow0 = (-off + sw - 1) / sw;
            int ow1 = wo;
            if (off + (wo - 1) * sw >= wd) ow1 = (wd - 1 - off) / sw + 1;
            if (ow1 > wo) ow1 = wo;
            for (int ow = ow0; ow < ow1; ++ow) orow[ow] += wv * (int32_t)xrow[ow * sw + off];
          }
        }
      }
    }
  }
  return 0;
}

/* Exact int32 accumulators of fc: x [M,K] int8, w [K,N] int8 (FcParam layout,
 * lite/operators/op_params.h:100-118), acc [M,N]. */
int orc_fc_acc_i32(const int8_t* x, const int8_t* w, int32_t* acc, int m, int k, int n) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    int32_t* out = acc + (long)i * n;
    memset(out, 0, sizeof(int32_t) * (size_t)n);
    for (int kk = 0; kk < k; ++kk) {
      const int32_t xv = x[(long)i * k + kk];
      if (xv == 0) continue;
      const int8_t* wrow = w + (long)kk * n;
      for (int j = 0; j < n; ++j) out[j] += xv * (int32_t)wrow[j];
    }
  }
  return 0;
}

static inline float act_apply(float v, int act, float alpha) {
  /* gemm_fuse_relu_bias, gemm_s8u8_kernel.cc:31-55 */
  switch (act) {
    case ORC_ACT_RELU:
      return v > 0.f ? v : 0.f;
    case ORC_ACT_RELU6:
      v = v > 0.f ? v : 0.f;
      return v < alpha ? v : alpha;
    case ORC_ACT_LEAKY:
      return v <= 0.f ? alpha * v : v;
    default:
      return v;
  }
}

static inline int8_t requant(float v) {
  /* cvtps_epi32 (RNE) -> packs (saturate) -> max(.,-127): gemm_s8u8_kernel.cc:133-145,276-290 */
  float r = nearbyintf(v); /* default rounding mode is to-nearest-even */
  if (r > 127.f) r = 127.f;
  if (r < -127.f) r = -127.f;
  if (r != r) r = 0.f;
  return (int8_t)r;
}

/* Epilogue over acc laid out [outer][C][inner] (NCHW conv: outer=N, inner=Ho*Wo;
 * fc: outer=M, C=N, inner=1).  out is float* or int8_t* depending on out_is_int8. */
int orc_epilogue(const int32_t* acc, void* out, long outer, int c, long inner,
                 const float* wscale, int n_wscale, float in_scale, float out_scale,
                 const float* bias, int act, float alpha, int out_is_int8, int leaky_compat) {
  if (n_wscale != 1 && n_wscale != c) return -1; /* conv_compute.cc:242-244 */
  for (long o = 0; o < outer; ++o) {
    for (int ch = 0; ch < c; ++ch) {
      const float ws = wscale[n_wscale == 1 ? 0 : ch];
      float scale = ws * in_scale; /* calc_scale, gemm_s8u8_compute.cc:85-98 */
      float b = bias ? bias[ch] : 0.f;
      float a = alpha;
      if (out_is_int8) {
        scale = scale / out_scale;
        b = b / out_scale;
        if (act == ORC_ACT_RELU6) a = alpha / out_scale;             /* conv_compute.cc:390 */
        if (act == ORC_ACT_LEAKY && leaky_compat) a = alpha / out_scale; /* :394 */
      }
      const int32_t* src = acc + ((long)o * c + ch) * inner;
      if (out_is_int8) {
        int8_t* dst = (int8_t*)out + ((long)o * c + ch) * inner;
        for (long i = 0; i < inner; ++i)
          dst[i] = requant(act_apply(fmaf((float)src[i], scale, b), act, a));
      } else {
        float* dst = (float*)out + ((long)o * c + ch) * inner;
        for (long i = 0; i < inner; ++i) dst[i] = act_apply(fmaf((float)src[i], scale, b), act, a);
      }
    }
  }
  return 0;
}

/* fp64 shadow of the fp32-out epilogue, for reporting how far fp32 rounding moves a value. */
int orc_epilogue_f64(const int32_t* acc, double* out, long outer, int c, long inner,
                     const float* wscale, int n_wscale, float in_scale, const float* bias,
                     int act, float alpha) {
  if (n_wscale != 1 && n_wscale != c) return -1;
  for (long o = 0; o < outer; ++o)
    for (int ch = 0; ch < c; ++ch) {
      const double scale = (double)wscale[n_wscale == 1 ? 0 : ch] * (double)in_scale;
      const double b = bias ? bias[ch] : 0.0;
      const int32_t* src = acc + ((long)o * c + ch) * inner;
      double* dst = out + ((long)o * c + ch) * inner;
      for (long i = 0; i < inner; ++i) {
        double v = (double)src[i] * scale + b;
        if (act == ORC_ACT_RELU) v = v > 0 ? v : 0;
        if (act == ORC_ACT_RELU6) { v = v > 0 ? v : 0; v = v < alpha ? v : alpha; }
        if (act == ORC_ACT_LEAKY) v = v <= 0 ? alpha * v : v;
        dst[i] = v;
      }
    }
  return 0;
}

/* ------------------------------------------------------------------ calib */

/* fp32 -> int8, lite/backends/x86/math/calib.cc:25-151 (vector body):
 * q = sat8(rne(max(x * (1/scale), -127))). */
void orc_calib_f32_to_i8(const float* x, int8_t* q, long n, float scale) {
  const float inv = 1.f / scale;
  for (long i = 0; i < n; ++i) {
    float v = x[i] * inv;
    if (!(v > -127.f)) v = -127.f;
    float r = nearbyintf(v);
    if (r > 127.f) r = 127.f;
    q[i] = (int8_t)r;
  }
}

/* int8 -> fp32, calib.cc:153-239: y = q * scale. */
void orc_calib_i8_to_f32(const int8_t* q, float* y, long n, float scale) {
  for (long i = 0; i < n; ++i) y[i] = (float)q[i] * scale;
}

/* ------------------------------------------------- sparse weight encoders */

/* ComputeSemiSparseZeros, sparse_conv_detect_pass.cc:303-368.
 * Returns the number of zero entries; fills count_nonzeroes / count_channels /
 * count_blocks / flag_semi exactly as the pass does. */
#define DEF_SPARSE_ZEROS(NAME, T)                                                             \
  int NAME(const T* data, int height, int width, int* count_nonzeroes, int* count_channels,   \
           int* count_blocks, int* flag_semi) {                                               \
    long nnz = 0, blocks2 = 0;                                                                \
    const int align2 = height & (-2);                                                         \
    for (int oc = 0; oc < align2; oc += 2)                                                    \
      for (int ic = 0; ic < width; ++ic) {                                                    \
        const int r0 = data[(long)oc * width + ic] != (T)0;                                   \
        const int r1 = data[(long)(oc + 1) * width + ic] != (T)0;                             \
        nnz += r0 + r1;                                                                       \
        blocks2 += (r0 | r1);                                                                 \
      }                                                                                       \
    const long block2_nnz = nnz;                                                              \
    for (int oc = align2; oc < height; ++oc)                                                  \
      for (int ic = 0; ic < width; ++ic) nnz += data[(long)oc * width + ic] != (T)0;          \
    *flag_semi = 0;                                                                           \
    *count_channels = height;                                                                 \
    *count_nonzeroes = (int)nnz;                                                              \
    *count_blocks = (int)nnz;                                                                 \
    if (block2_nnz * 5 >= blocks2 * 9) {                                                      \
      *count_channels = height / 2 + height % 2;                                              \
      *flag_semi = 1;                                                                         \
      const long rem = nnz - block2_nnz;                                                      \
      *count_nonzeroes = (int)(blocks2 * 2 + rem);                                            \
      *count_blocks = (int)(blocks2 + rem);                                                   \
    }                                                                                         \
    return (int)((long)height * width - *count_nonzeroes);                                    \
  }
DEF_SPARSE_ZEROS(orc_sparse_zeros_i8, int8_t)
DEF_SPARSE_ZEROS(orc_sparse_zeros_f32, float)

/* Replace the last diff of every output-channel group by the running sum of all diffs
 * so far (sparse_conv_detect_pass.cc:70-85 and the identical loops at :172-192, :262-295). */
static void diffs_running_sum(int32_t* diffs, const uint32_t* cum, int groups) {
  long run = 0;
  long ik = 0;
  for (int g = 0; g < groups; ++g) {
    const uint32_t cnt = g == 0 ? cum[0] : cum[g] - cum[g - 1];
    for (uint32_t t = 0; t < cnt; ++t) run += diffs[ik++];
    if (ik != 0) diffs[ik - 1] = (int32_t)run;
  }
}

/* ComputeSparseWeight<T> without padding (used for int8 weights, :35-91, call site :769-776).
 * w [M,K]; hw = Ho*Wo of the layer.  nonzero_out [nnz], oc_nonzeros [M] cumulative,
 * diffs [nnz].  Returns first_ic. */
#define DEF_SPARSE_ENCODE(NAME, T)                                                         \
  int NAME(const T* w, int m, int k, int hw, T* nonzero_out, uint32_t* oc_nonzeros,        \
           int32_t* diffs) {                                                               \
    int first_ic = 0, last_ic = 0, first = 1;                                              \
    long ni = 0, di = 0;                                                                   \
    for (int oc = 0; oc < m; ++oc) {                                                       \
      for (int ic = 0; ic < k; ++ic) {                                                     \
        const T v = w[(long)oc * k + ic];                                                  \
        if (v != (T)0) {                                                                   \
          nonzero_out[ni++] = v;                                                           \
          if (first) first_ic = ic;                                                        \
          else diffs[di++] = (int32_t)((ic - last_ic) * (int)sizeof(T)) * hw;              \
          first = 0;                                                                       \
          last_ic = ic;                                                                    \
        }                                                                                  \
      }                                                                                    \
      oc_nonzeros[oc] = (uint32_t)ni;                                                      \
    }                                                                                      \
    /* the pass runs the running-sum loop BEFORE it writes the wrap-around diff; the slot \
     * it reads early (diffs[nnz-1]) is then overwritten, so zero it first for a defined  \
     * value and finish with the wrap diff as the pass does. */                            \
    if (ni > 0) diffs[ni - 1] = 0;                                                         \
    diffs_running_sum(diffs, oc_nonzeros, m);                                              \
    if (!first) diffs[di++] = (int32_t)((first_ic - last_ic) * (int)sizeof(T)) * hw;       \
    return first_ic;                                                                       \
  }
DEF_SPARSE_ENCODE(orc_sparse_encode_i8, int8_t)
DEF_SPARSE_ENCODE(orc_sparse_encode_unpadded_f32, float)

/* ComputeSparseWeight<T> padded to multiples of 4 per channel (fp32 weights, :93-194,
 * call site :746-754).  Buffers must hold sum over channels of roundup4(nnz_c) entries.
 * Returns first_ic; *n_stored receives the stored (padded) count. */
int orc_sparse_encode_pad4_f32(const float* w, int m, int k, int hw, float* nonzero_out,
                               uint32_t* oc_nonzeros, int32_t* diffs, int* n_stored) {
  long nnz_total = 0;
  for (long i = 0; i < (long)m * k; ++i) nnz_total += w[i] != 0.f;
  int32_t* act = (int32_t*)calloc((size_t)nnz_total + 1, sizeof(int32_t));
  int first_ic = 0, last_ic = 0, first = 1;
  long ni = 0, di = 0;
  for (int oc = 0; oc < m; ++oc) {
    uint32_t cnt = 0;
    for (int ic = 0; ic < k; ++ic) {
      const float v = w[(long)oc * k + ic];
      if (v != 0.f) {
        nonzero_out[ni++] = v;
        if (first) first_ic = ic;
        else act[di++] = (int32_t)((ic - last_ic) * (int)sizeof(float)) * hw;
        first = 0;
        last_ic = ic;
        ++cnt;
      }
    }
    if (cnt % 4) for (uint32_t j = 0; j < 4 - cnt % 4; ++j) nonzero_out[ni++] = 0.f;
    if (oc == 0) {
      oc_nonzeros[0] = cnt;
    } else {
      const uint32_t rem = oc_nonzeros[oc - 1] & 3u;
      oc_nonzeros[oc] = rem == 0 ? cnt + oc_nonzeros[oc - 1] : cnt + oc_nonzeros[oc - 1] + 4 - rem;
    }
  }
  if (!first) act[di++] = (int32_t)((first_ic - last_ic) * (int)sizeof(float)) * hw;
  long li = 0, ri = 0;
  for (int oc = 0; oc < m; ++oc) {
    uint32_t cur;
    if (oc == 0) {
      cur = oc_nonzeros[0];
    } else {
      const uint32_t rem = oc_nonzeros[oc - 1] & 3u;
      cur = rem == 0 ? oc_nonzeros[oc] - oc_nonzeros[oc - 1]
                     : oc_nonzeros[oc] - (oc_nonzeros[oc - 1] + 4 - rem);
    }
    for (uint32_t i = 0; i < cur; ++i) diffs[ri++] = act[li++];
    if (cur % 4) for (uint32_t j = 0; j < 4 - cur % 4; ++j) diffs[ri++] = 0;
  }
  free(act);
  *n_stored = (int)ri;
  /* running sum over the stored (padded) counts: cum[] as the kernel will see them */
  {
    long run = 0, ik = 0;
    for (int oc = 0; oc < m; ++oc) {
      const uint32_t cnt = oc == 0 ? oc_nonzeros[0] : oc_nonzeros[oc] - oc_nonzeros[oc - 1];
      for (uint32_t t = 0; t < cnt; ++t) run += diffs[ik++];
      if (ik != 0) diffs[ik - 1] = (int32_t)run;
    }
  }
  return first_ic;
}

/* ComputeSemiSparseWeight<T> (:196-301).  Pairs of output channels share one diff per
 * stored 2x1 block; an odd last channel is stored one value per block.
 * oc_nonzeros has ceil(M/2) meaningful cumulative block counts. */
#define DEF_SPARSE_ENCODE_SEMI(NAME, T)                                                     \
  int NAME(const T* w, int m, int k, int hw, T* nonzero_out, uint32_t* oc_nonzeros,         \
           int32_t* diffs) {                                                                \
    const int align2 = m & (-2);                                                            \
    int first_ic = 0, last_ic = 0, first = 1;                                               \
    long ni = 0, di = 0;                                                                    \
    uint32_t block_n = 0;                                                                   \
    int bi = 0;                                                                             \
    for (int oc = 0; oc < align2; oc += 2) {                                                \
      for (int ic = 0; ic < k; ++ic) {                                                      \
        const T a = w[(long)oc * k + ic], b = w[(long)(oc + 1) * k + ic];                   \
        if (a != (T)0 || b != (T)0) {                                                       \
          nonzero_out[ni++] = a;                                                            \
          nonzero_out[ni++] = b;                                                            \
          if (first) first_ic = ic;                                                         \
          else diffs[di++] = (int32_t)((ic - last_ic) * (int)sizeof(T)) * hw;               \
          first = 0;                                                                        \
          last_ic = ic;                                                                     \
          ++block_n;                                                                        \
        }                                                                                   \
      }                                                                                     \
      oc_nonzeros[bi++] = block_n;                                                          \
    }                                                                                       \
    for (int oc = align2; oc < m; ++oc) {                                                   \
      for (int ic = 0; ic < k; ++ic) {                                                      \
        const T a = w[(long)oc * k + ic];                                                   \
        if (a != (T)0) {                                                                    \
          nonzero_out[ni++] = a;                                                            \
          if (first) first_ic = ic;                                                         \
          else diffs[di++] = (int32_t)((ic - last_ic) * (int)sizeof(T)) * hw;               \
          first = 0;                                                                        \
          last_ic = ic;                                                                     \
          ++block_n;                                                                        \
        }                                                                                   \
      }                                                                                     \
      oc_nonzeros[bi++] = block_n;                                                          \
    }                                                                                       \
    if (block_n > 0) diffs[block_n - 1] = 0;                                                \
    diffs_running_sum(diffs, oc_nonzeros, bi);                                              \
    if (!first) diffs[di++] = (int32_t)((first_ic - last_ic) * (int)sizeof(T)) * hw;        \
    return first_ic;                                                                        \
  }
DEF_SPARSE_ENCODE_SEMI(orc_sparse_encode_semi_i8, int8_t)
DEF_SPARSE_ENCODE_SEMI(orc_sparse_encode_semi_f32, float)

/* Walk an encoding the way the ARM kernels do and rebuild the dense [M,K] matrix.
 * Start of group g: weights at A + cum[g-1]*(semi?2:1); input pointer at
 * B + (cum[g-1]==0 ? 0 : diffs[cum[g-1]-1]) with B = x + first_ic*hw
 * (sparse_conv_impl.cc:3738-3745, sparse_semi_conv_impl.cc:1788-1823,
 * sparse_conv_compute.cc:181).  Returns 0, or -1 if a walk leaves [0,K). */
/* pad4 != 0 selects the fp32 unstructured layout whose channels are padded to multiples of 4. */
#define DEF_SPARSE_DECODE(NAME, T)                                                            \
  int NAME(const T* nz, const uint32_t* cum, const int32_t* diffs, int m, int k, int hw,      \
           int first_ic, int flag_semi, int pad4, T* dense) {                                 \
    memset(dense, 0, sizeof(T) * (size_t)m * k);                                              \
    const long unit = (long)sizeof(T) * hw;                                                   \
    const int pairs = flag_semi ? m / 2 : 0;                                                  \
    const int groups = flag_semi ? pairs + (m % 2) : m;                                       \
    for (int g = 0; g < groups; ++g) {                                                        \
      const uint32_t prev0 = g == 0 ? 0 : cum[g - 1];                                         \
      /* padded fp32 encoding: a channel starts at the next multiple of 4 after the previous \
       * channel's last real entry (sparse_conv_impl.cc:1230-1241) */                         \
      const uint32_t skip = (pad4 && !flag_semi) ? ((4u - (prev0 & 3u)) & 3u) : 0u;           \
      const uint32_t prev = prev0 + skip;                                                     \
      const uint32_t cnt = cum[g] - prev;                                                     \
      long off = (g == 0 || prev0 == 0) ? 0 : diffs[prev0 - 1];                               \
      const int is_pair = flag_semi && g < pairs;                                             \
      const T* wp = nz + (flag_semi ? (g < pairs ? (long)prev * 2                             \
                                                 : (long)(pairs ? cum[pairs - 1] : 0) * 2 +   \
                                                       (prev - (pairs ? cum[pairs - 1] : 0))) \
                                    : (long)prev);                                            \
      for (uint32_t t = 0; t < cnt; ++t) {                                                    \
        if (off % unit) return -1;                                                            \
        const long ic = first_ic + off / unit;                                                \
        if (is_pair) {                                                                        \
          if (ic < 0 || ic >= k) { if (wp[0] != (T)0 || wp[1] != (T)0) return -1; }           \
          else { dense[(long)(2 * g) * k + ic] += wp[0]; dense[(long)(2 * g + 1) * k + ic] += wp[1]; } \
          wp += 2;                                                                            \
        } else {                                                                              \
          const int oc = flag_semi ? 2 * pairs + (g - pairs) : g;                             \
          if (ic < 0 || ic >= k) { if (wp[0] != (T)0) return -1; }                            \
          else dense[(long)oc * k + ic] += wp[0];                                             \
          wp += 1;                                                                            \
        }                                                                                     \
        off += diffs[prev + t];                                                               \
      }                                                                                       \
    }                                                                                         \
    return 0;                                                                                 \
  }
DEF_SPARSE_DECODE(orc_sparse_decode_i8, int8_t)
DEF_SPARSE_DECODE(orc_sparse_decode_f32, float)

/* fp32 1x1 conv on dense weights: bias first, then fused multiply-adds in ascending
 * input-channel order over the non-zero weights (the ARM kernel's order,
 * sparse_conv_impl.cc:1486-1496), then the activation.  x [N,K,HW], y [N,M,HW]. */
int orc_sparse_conv_f32(const float* x, const float* dense, const float* bias, float* y, int n,
                        int m, int k, int hw, int act, float alpha) {
#pragma omp parallel for schedule(static)
  for (long idx = 0; idx < (long)n * m; ++idx) {
    const int b = (int)(idx / m), oc = (int)(idx % m);
    float* out = y + idx * hw;
    const float b0 = bias ? bias[oc] : 0.f;
    for (int p = 0; p < hw; ++p) out[p] = b0;
    for (int ic = 0; ic < k; ++ic) {
      const float wv = dense[(long)oc * k + ic];
      if (wv == 0.f) continue;
      const float* xin = x + ((long)b * k + ic) * hw;
      for (int p = 0; p < hw; ++p) out[p] = fmaf(wv, xin[p], out[p]);
    }
    for (int p = 0; p < hw; ++p) out[p] = act_apply(out[p], act, alpha);
  }
  return 0;
}

/* fp64 version of the above, for tolerance reporting. */
int orc_sparse_conv_f64(const float* x, const float* dense, const float* bias, double* y, int n,
                        int m, int k, int hw, int act, float alpha) {
#pragma omp parallel for schedule(static)
  for (long idx = 0; idx < (long)n * m; ++idx) {
    const int b = (int)(idx / m), oc = (int)(idx % m);
    double* out = y + idx * hw;
    for (int p = 0; p < hw; ++p) out[p] = bias ? bias[oc] : 0.0;
    for (int ic = 0; ic < k; ++ic) {
      const double wv = dense[(long)oc * k + ic];
      if (wv == 0.0) continue;
      const float* xin = x + ((long)b * k + ic) * hw;
      for (int p = 0; p < hw; ++p) out[p] += wv * xin[p];
    }
    for (int p = 0; p < hw; ++p) {
      double v = out[p];
      if (act == ORC_ACT_RELU) v = v > 0 ? v : 0;
      if (act == ORC_ACT_RELU6) { v = v > 0 ? v : 0; v = v < alpha ? v : alpha; }
      if (act == ORC_ACT_LEAKY) v = v <= 0 ? alpha * v : v;
      out[p] = v;
    }
  }
  return 0;
}

/* ------------------------------------------------ fp32 glue between layers */

/* softmax over the last axis, the x86 form (lite/backends/x86/math/softmax_impl.h:110-131):
 * shift by the row maximum, clip the shifted logits at -64, exponentiate, scale by 1/sum.
 * exp and the sum are evaluated in double here; the CUDA kernel and the reference's polynomial
 * vec_exp both stay within 1e-5 relative of this. */
int orc_softmax_f32(const float* x, float* y, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (long)r * cols;
    float* yr = y + (long)r * cols;
    float m = xr[0];
    for (int i = 1; i < cols; ++i) m = xr[i] > m ? xr[i] : m;
    double s = 0.0;
    for (int i = 0; i < cols; ++i) {
      float d = xr[i] - m;
      d = d < -64.f ? -64.f : d;
      s += exp((double)d);
    }
    for (int i = 0; i < cols; ++i) {
      float d = xr[i] - m;
      d = d < -64.f ? -64.f : d;
      yr[i] = (float)(exp((double)d) / s);
    }
  }
  return 0;
}

/* max pool on int8 NCHW (pool2d max, exclusive padding = ignore out-of-range taps). */
int orc_maxpool_i8(const int8_t* x, int8_t* y, int n, int c, int h, int w, int k, int s, int p) {
  const int ho = (h + 2 * p - k) / s + 1, wo = (w + 2 * p - k) / s + 1;
  for (long pc = 0; pc < (long)n * c; ++pc)
    for (int oh = 0; oh < ho; ++oh)
      for (int ow = 0; ow < wo; ++ow) {
        int best = -128;
        for (int r = 0; r < k; ++r)
          for (int q = 0; q < k; ++q) {
            const int ih = oh * s - p + r, iw = ow * s - p + q;
            if (ih < 0 || ih >= h || iw < 0 || iw >= w) continue;
            const int v = x[(pc * h + ih) * w + iw];
            if (v > best) best = v;
          }
        y[(pc * ho + oh) * wo + ow] = (int8_t)best;
      }
  return 0;
}
