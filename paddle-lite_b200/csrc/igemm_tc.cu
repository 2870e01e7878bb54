// int8 x int8 -> int32 implicit GEMM on the sm_100a tensor cores (tcgen05.mma kind::i8,
// accumulators in tensor memory), operands staged through shared memory by TMA
// (cp.async.bulk.tensor, tiled for flat GEMMs and filters, im2col mode for convolutions;
// never cluster multicast), fused dequant / bias / activation / requant epilogue.
//
// This is the B200 replacement for the reference's im2col<int8_t> + gemm_s8u8 pair
// (lite/backends/x86/math/avx/conv_utils.cc:1349-1398,
//  lite/backends/x86/math/gemm_s8u8_compute.h:65-106, gemm_s8u8_kernel.cc:353-891).
//
// Persistent CTA (one per SM) of 18 warps:
//   warps 0-15 epilogue, four groups of four warps (warp w reads TMEM lane quadrant w%4).
//              With channel tiles of up to 128 there are four accumulator buffers and each
//              group drains every fourth tile; with 256-wide tiles there are two buffers and
//              two groups share a tile by 32-column chunks;
//   warp 16    TMA producer (one elected lane) filling a ring of operand stages;
//   warp 17    TMEM allocation + MMA issue (one elected lane); the epilogue of one tile
//              overlaps the main loops of the following ones.
// Tile = 128 output pixels x BN output channels, K consumed KC bytes per pipeline stage
// (KC = 32/64/128 = the TMA swizzle span), 32 bytes of K per tcgen05.mma.
// Every mbarrier wait is bounded; a wait that runs out records a fault in the ctx status
// word and the CTA drains and exits instead of hanging.
#include "igemm_tc.cuh"
#include "igemm_pair.cuh"
#include "tc_device.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <utility>

namespace plb {

namespace {

using namespace tc;

constexpr int kTileM = 128;
constexpr int kMaxStages = 16;
constexpr int kEpilogueGroups = 4;              // groups of 4 warps (one per TMEM lane quadrant)
constexpr int kEpilogueWarps = 4 * kEpilogueGroups;
constexpr int kProducerWarp = kEpilogueWarps;
constexpr int kMmaWarp = kEpilogueWarps + 1;
constexpr int kThreads = 32 * (kEpilogueWarps + 2);
constexpr int kMaxAccBufs = 8;
constexpr int kCtrlBytes = 1024;                // barriers + tmem slot
constexpr int kMaxResidentB = 56 * 1024;        // filters up to this size stay in shared memory for the whole kernel

struct IgemmArgs {
  int im2col;
  int m_total, cout;
  int bn, kc, cchunks, ksteps, stages;
  int taps, kw;
  int ho, wo, stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int tiles_n, num_tiles;
  int staging_bytes, staging_w_bytes;  // epilogue staging in front of the operand ring
  int stage_b_warp;                    // bytes of int8 staging per epilogue warp
  int res_prefetch;                    // OUT_ADD_RELU: two residual staging tiles per warp, one chunk fetched ahead
  int acc_bufs;                        // TMEM accumulator buffers: 2, 4 or 8 (epilogue groups per buffer = max(1, 4 / acc_bufs))
  int resident_b;                      // whole filter of this CTA's channel tile kept in shared memory
  int resident_bytes;                  // its size, rounded up to 1 KiB
  // slab mode (stride-1 filters with several taps): a pipeline stage holds the input window of a
  // 16 x 8 pixel output tile once and every tap reads it through a shifted matrix descriptor
  int slab, kh;
  int slab_w;                          // window width in pixels = 8 + (kw-1)*dil_w
  int slab_rows;                       // window pixels = slab_w * (16 + (kh-1)*dil_h)
  int plane_bytes;                     // one channel chunk of the window, rounded up to 1 KiB
  int tiles_x, tiles_y;                // output tiles per image
  // dual mode (OUT_ADD_RELU): a second 1x1 GEMM (the shortcut convolution of a residual block)
  // accumulates into the columns next to the main accumulator; the epilogue turns it into the
  // residual value fma(acc2, scale2, bias2) instead of reading a residual tensor
  int dual, ksteps2, cchunks2, im2col2, stride2_h, stride2_w;
  const float* scale2;
  const float* bias2;
  int out_mode, ldy;
  void* y;
  const float* scale;
  const float* bias;
  int act;
  float alpha;
  int acc_small;                       // every |accumulator| < 2^22 (proven from the filter by the host)
  int fast_window;                     // window tiles of a row-folded stem layer (shapes 4x1 / 2x1, two MMAs per tap): short role loops
  int fast_flat;                       // flat tiles without a shortcut GEMM: short producer loop
  int fast_im2col, cin_bytes;          // im2col tiles without a shortcut GEMM: short producer loop; cchunks * kc
  int fast_mma;                        // flat or im2col tiles without a shortcut GEMM: short MMA loop
  int sb_off, sb_cols;                 // scale / bias tables copied to shared memory (offset in the staging area; 0 columns = not)
  const float* residual;
  float* y_f32;
  int8_t* y_i8;
  float inv_next_scale;
  int* status;
#ifdef PLB_TC_FAULT_TEST
  int test_skip_load;                  // test build: CTA 0 drops the copies of one pipeline stage
#endif
};

// Residual values of one 32-column chunk, fetched before the accumulator is read so that
// the global-memory latency overlaps the wait for the tensor cores.
__device__ __forceinline__ void load_residual32(const IgemmArgs& a, long row, int col, float (&res)[32]) {
  const int ncols = a.cout - col < 32 ? a.cout - col : 32;
  const float* src = a.residual + row * a.ldy + col;
  if (ncols == 32 && (a.ldy & 7) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) ld_global_v8f(src + 8 * j, &res[8 * j]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) res[j] = j < ncols ? src[j] : 0.f;
  }
}

template <int MODE, int ACT>
__device__ __forceinline__ void epilogue_store32(const IgemmArgs& a, const uint32_t (&r)[32],
                                                 const float (&res)[32], long row, int col) {
  const int ncols = a.cout - col < 32 ? a.cout - col : 32;
  const bool full = ncols == 32;
  if (MODE == OUT_ACC) {
    int32_t* dst = static_cast<int32_t*>(a.y) + row * a.ldy + col;
    if (full && (a.ldy & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<int4*>(dst + j) =
            make_int4((int)r[j], (int)r[j + 1], (int)r[j + 2], (int)r[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = (int)r[j];
    }
    return;
  }
  // per-channel scale and bias: every lane reads the same addresses (one broadcast request);
  // the arrays are padded so that a ragged last tile may read past cout
  const float4* sc4 = reinterpret_cast<const float4*>(a.scale + col);
  const float4* bi4 = reinterpret_cast<const float4*>(a.bias + col);
  if (MODE == OUT_I8) {
    const float ub = quant_upper_bound<ACT>(a.alpha);
    uint32_t q[8];
    if (a.acc_small) {
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = quant4<ACT, true>(&r[4 * j], __ldg(sc4 + j), __ldg(bi4 + j), a.alpha, ub);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = quant4<ACT, false>(&r[4 * j], __ldg(sc4 + j), __ldg(bi4 + j), a.alpha, ub);
    }
    int8_t* dst = static_cast<int8_t*>(a.y) + row * a.ldy + col;
    if (full && (a.ldy & 31) == 0) {
      st_global_v8(dst, q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
    } else if (full && (a.ldy & 15) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(q[0], q[1], q[2], q[3]);
      *reinterpret_cast<uint4*>(dst + 16) = make_uint4(q[4], q[5], q[6], q[7]);
    } else if (full && (a.ldy & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<uint32_t*>(dst + 4 * j) = q[j];
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = static_cast<int8_t>(q[j >> 2] >> (8 * (j & 3)));
    }
    return;
  }
  if (MODE == OUT_F32) {
    float* dst = static_cast<float*>(a.y) + row * a.ldy + col;
    const bool vec8 = full && (a.ldy & 7) == 0;
    const bool vec4 = full && (a.ldy & 3) == 0;
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float4 v[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 sc = __ldg(sc4 + j + h), bi = __ldg(bi4 + j + h);
        v[h].x = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * (j + h)]), sc.x, bi.x), a.alpha);
        v[h].y = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * (j + h) + 1]), sc.y, bi.y), a.alpha);
        v[h].z = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * (j + h) + 2]), sc.z, bi.z), a.alpha);
        v[h].w = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * (j + h) + 3]), sc.w, bi.w), a.alpha);
      }
      if (vec8) {
        st_global_v8f(dst + 4 * j, v[0], v[1]);
      } else if (vec4) {
        *reinterpret_cast<float4*>(dst + 4 * j) = v[0];
        *reinterpret_cast<float4*>(dst + 4 * j + 4) = v[1];
      } else {
        const float t[8] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w};
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (4 * j + e < ncols) dst[4 * j + e] = t[e];
      }
    }
    return;
  }
  // OUT_ADD_RELU: fp32 value + residual, ReLU, optional fp32 store, optional calib to int8
  {
    const long off = row * a.ldy + col;
    const bool vec8 = full && (a.ldy & 7) == 0;
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float4 v[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 sc = __ldg(sc4 + j + h), bi = __ldg(bi4 + j + h);
        const int b = 4 * (j + h);
        v[h].x = fmaxf(fmaf(__int2float_rn((int)r[b]), sc.x, bi.x) + res[b], 0.f);
        v[h].y = fmaxf(fmaf(__int2float_rn((int)r[b + 1]), sc.y, bi.y) + res[b + 1], 0.f);
        v[h].z = fmaxf(fmaf(__int2float_rn((int)r[b + 2]), sc.z, bi.z) + res[b + 2], 0.f);
        v[h].w = fmaxf(fmaf(__int2float_rn((int)r[b + 3]), sc.w, bi.w) + res[b + 3], 0.f);
        // calib of the next layer: sat(rne(max(v * inv_scale, -127))); v >= 0 here
        q[j + h] = pack_low_bytes(__float_as_uint(fminf(v[h].x * a.inv_next_scale, 127.f) + kRoundMagic),
                                  __float_as_uint(fminf(v[h].y * a.inv_next_scale, 127.f) + kRoundMagic),
                                  __float_as_uint(fminf(v[h].z * a.inv_next_scale, 127.f) + kRoundMagic),
                                  __float_as_uint(fminf(v[h].w * a.inv_next_scale, 127.f) + kRoundMagic));
      }
      if (a.y_f32 != nullptr) {
        float* dst = a.y_f32 + off + 4 * j;
        if (vec8) {
          st_global_v8f(dst, v[0], v[1]);
        } else {
          const float t[8] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w};
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (4 * j + e < ncols) dst[e] = t[e];
        }
      }
    }
    if (a.y_i8 != nullptr) {
      int8_t* dst = a.y_i8 + off;
      if (full && (a.ldy & 31) == 0) {
        st_global_v8(dst, q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) dst[j] = static_cast<int8_t>(q[j >> 2] >> (8 * (j & 3)));
      }
    }
  }
}

// ---------------------------------------------------------------- epilogue through shared memory
// With one lane per output row every global access of a warp touches 32 different lines, which
// makes the load/store unit (32 wavefronts per instruction) the limit of the fp32 epilogues.
// When the output geometry allows it the epilogue therefore moves its global traffic with
// TMA: the fp32 residual tile of a chunk is fetched by cp.async.bulk.tensor into a 128-byte
// swizzled staging tile, results are written to staging tiles and leave with TMA stores
// (bulk async-group), which also clip ragged rows at the end of the tensor.
// One 32-column chunk of one row, staged.  st_w: this warp's 32 x 128-byte fp32 tile (128-byte
// swizzle: 16-byte chunk j of row r lives at chunk j ^ (r & 7)), holding the residual on entry
// for OUT_ADD_RELU and the fp32 / int32 result on exit.  st_b_row: address of this lane's row in
// the int8 staging tile, byte_chunk0 the index of the first 16-byte chunk to write and
// b_swz_mask the xor mask of that row in the tile's swizzle (see b_swz at the call site).
template <int MODE, int ACT>
__device__ __forceinline__ void epilogue_chunk_staged(const IgemmArgs& a, const float* scale, const float* bias,
                                                      const uint32_t (&r)[32], int lane, int col, uint32_t st_w,
                                                      uint32_t st_b_row, int byte_chunk0, int b_swz_mask, bool have_res) {
  const uint32_t w_row = st_w + lane * 128;
  const int sw = lane & 7;
  if (MODE == OUT_ACC) {
#pragma unroll
    for (int j = 0; j < 8; ++j) sts128(w_row + ((j ^ sw) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    return;
  }
  // scale / bias: the CTA's shared-memory copy (all lanes read the same address: a broadcast) or global memory
  const float4* sc4 = reinterpret_cast<const float4*>(scale + col);
  const float4* bi4 = reinterpret_cast<const float4*>(bias + col);
  if (MODE == OUT_F32) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 sc = sc4[j], bi = bi4[j];
      const float x = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j]), sc.x, bi.x), a.alpha);
      const float y = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j + 1]), sc.y, bi.y), a.alpha);
      const float z = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j + 2]), sc.z, bi.z), a.alpha);
      const float w = act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j + 3]), sc.w, bi.w), a.alpha);
      sts128(w_row + ((j ^ sw) << 4), __float_as_uint(x), __float_as_uint(y), __float_as_uint(z), __float_as_uint(w));
    }
    return;
  }
  uint32_t q[8];
  if (MODE == OUT_I8) {
    const float ub = quant_upper_bound<ACT>(a.alpha);
    // two halves of 16 columns, each stored as soon as it is packed; the compiler barrier keeps the
    // second half's scale / bias loads from being hoisted (they would cost 32 registers)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (a.acc_small) {
#pragma unroll
        for (int j = 4 * h; j < 4 * h + 4; ++j) q[j] = quant4<ACT, true>(&r[4 * j], sc4[j], bi4[j], a.alpha, ub);
      } else {
#pragma unroll
        for (int j = 4 * h; j < 4 * h + 4; ++j) q[j] = quant4<ACT, false>(&r[4 * j], sc4[j], bi4[j], a.alpha, ub);
      }
      sts128(st_b_row + (((byte_chunk0 + h) ^ b_swz_mask) << 4), q[4 * h], q[4 * h + 1], q[4 * h + 2], q[4 * h + 3]);
      asm volatile("" ::: "memory");
    }
    return;
  } else {  // OUT_ADD_RELU
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 sc = sc4[j], bi = bi4[j];
      const uint32_t addr = w_row + ((j ^ sw) << 4);
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (have_res) t = lds128f(addr);
      const float x = fmaxf(fmaf(__int2float_rn((int)r[4 * j]), sc.x, bi.x) + t.x, 0.f);
      const float y = fmaxf(fmaf(__int2float_rn((int)r[4 * j + 1]), sc.y, bi.y) + t.y, 0.f);
      const float z = fmaxf(fmaf(__int2float_rn((int)r[4 * j + 2]), sc.z, bi.z) + t.z, 0.f);
      const float w = fmaxf(fmaf(__int2float_rn((int)r[4 * j + 3]), sc.w, bi.w) + t.w, 0.f);
      if (a.y_f32 != nullptr)
        sts128(addr, __float_as_uint(x), __float_as_uint(y), __float_as_uint(z), __float_as_uint(w));
      q[j] = pack_low_bytes(__float_as_uint(fminf(x * a.inv_next_scale, 127.f) + kRoundMagic),
                            __float_as_uint(fminf(y * a.inv_next_scale, 127.f) + kRoundMagic),
                            __float_as_uint(fminf(z * a.inv_next_scale, 127.f) + kRoundMagic),
                            __float_as_uint(fminf(w * a.inv_next_scale, 127.f) + kRoundMagic));
    }
    if (a.y_i8 == nullptr) return;
  }
  sts128(st_b_row + (((byte_chunk0) ^ b_swz_mask) << 4), q[0], q[1], q[2], q[3]);
  sts128(st_b_row + (((byte_chunk0 + 1) ^ b_swz_mask) << 4), q[4], q[5], q[6], q[7]);
}

// ---------------------------------------------------------------- MMA issue sequences
// A 128 x 64 x 32 MMA keeps the tensor core busy for under 60 cycles, so the issuing warp can
// afford only a handful of instructions per MMA: the sequences below are fully unrolled for the
// common shapes, which turns every descriptor into "loop-invariant base + constant".

// MPS MMAs covering one K step (MPS * 32 bytes of K) of one pair of operand tiles.
template <int MPS>
__device__ __forceinline__ void issue_kstep(uint32_t d_tmem, uint32_t a_lo, uint32_t hi_a, uint32_t b_lo,
                                            uint32_t hi_b, uint32_t idesc, uint32_t accumulate, bool leader) {
  tc_mma_i8_halves(d_tmem, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
#pragma unroll
  for (int j = 1; j < MPS; ++j) tc_mma_i8_halves(d_tmem, a_lo + 2u * j, hi_a, b_lo + 2u * j, hi_b, idesc, 1u, leader);
}

// All taps of one window-mode tile: KH x KW taps, CC channel chunks, MPS MMAs per chunk.
template <int KH, int KW, int CC, int MPS>
__device__ __forceinline__ void issue_window(uint32_t d_tmem, uint32_t slab_lo, uint32_t row_lo, uint32_t col_lo,
                                             uint32_t plane_lo, uint32_t hi_a, uint32_t b_lo, uint32_t stage_b_lo,
                                             uint32_t hi_b, uint32_t idesc, bool leader) {
#pragma unroll
  for (int r = 0; r < KH; ++r) {
#pragma unroll
    for (int sx = 0; sx < KW; ++sx) {
#pragma unroll
      for (int cc = 0; cc < CC; ++cc) {
        const int ks = (r * KW + sx) * CC + cc;
        issue_kstep<MPS>(d_tmem, slab_lo + r * row_lo + sx * col_lo + cc * plane_lo, hi_a, b_lo + ks * stage_b_lo, hi_b,
                         idesc, ks > 0 ? 1u : 0u, leader);
      }
    }
  }
}

// Any filter size with CC channel chunks and MPS MMAs per chunk unrolled: the loops over the taps
// stay, everything inside a tap is "tap base + constant".
template <int CC, int MPS>
__device__ __forceinline__ void issue_window_taps(int kh, int kw, uint32_t d_tmem, uint32_t slab_lo, uint32_t row_lo,
                                                  uint32_t col_lo, uint32_t plane_lo, uint32_t hi_a, uint32_t b_lo,
                                                  uint32_t stage_b_lo, uint32_t hi_b, uint32_t idesc, bool leader) {
  uint32_t accumulate = 0;
  uint32_t row_a = slab_lo;
  for (int r = 0; r < kh; ++r, row_a += row_lo) {
    uint32_t tap_a = row_a;
    for (int sx = 0; sx < kw; ++sx, tap_a += col_lo, b_lo += CC * stage_b_lo) {
#pragma unroll
      for (int cc = 0; cc < CC; ++cc) {
        issue_kstep<MPS>(d_tmem, tap_a + cc * plane_lo, hi_a, b_lo + cc * stage_b_lo, hi_b, idesc, accumulate, leader);
        accumulate = 1;
      }
    }
  }
}

// Flat GEMM tiles (1x1 convolutions and fc; resident or streamed filter, any number of channel tiles): with
// few channels a tile is only a K step or two of work, so the per-tile instruction count of the two
// single-warp roles decides how fast tiles flow.  These loops keep the bookkeeping to a minimum: no
// divisions, no mode branches.  The MMA warp does not need to know which tile it is working on: with a streamed filter the B tile sits behind the A tile of
// the same stage, with a resident one at K step ks of the resident copy.
template <int MPS>
__device__ __forceinline__ bool mma_loop_flat(const IgemmArgs& a, uint32_t tmem_base, uint32_t acc_stride, int nb_mask,
                                              int nb_shift, uint32_t ring_lo, uint32_t stage_lo, uint32_t stage_a_lo,
                                              uint32_t bres_lo, uint32_t stage_b_lo, uint32_t hi, uint32_t idesc,
                                              uint32_t full0, uint32_t empty0, uint32_t acc_full0, uint32_t acc_empty0,
                                              uint32_t acc2_cols, bool leader, volatile int* abort_flag) {
  int s = 0, it = 0;
  uint32_t full_parity = 0;
  const bool resident = a.resident_b != 0;
  const int ksteps2 = a.dual ? a.ksteps2 : 0;
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x, ++it) {
    const int buf = it & nb_mask;
    if (!mbar_wait(acc_empty0 + 8u * buf, ((it >> nb_shift) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_ACCUM)) return false;
    const uint32_t d_tmem = tmem_base + buf * acc_stride;
    uint32_t b_res = bres_lo;
    for (int ks = 0; ks < a.ksteps; ++ks, b_res += stage_b_lo) {
      if (!mbar_wait(full0 + 8u * s, full_parity, abort_flag, a.status, FAULT_WAIT_FULL)) return false;
      tc_fence_after();
      const uint32_t a_lo = ring_lo + s * stage_lo;
      issue_kstep<MPS>(d_tmem, a_lo, hi, resident ? b_res : a_lo + stage_a_lo, hi, idesc, ks > 0 ? 1u : 0u, leader);
      tc_commit_if(empty0 + 8u * s, leader);
      if (++s == a.stages) {
        s = 0;
        full_parity ^= 1;
      }
    }
    // shortcut GEMM of a fused residual block: its K steps follow in the ring (filter always streamed) and
    // accumulate into the columns next to the main accumulator
    for (int ks = 0; ks < ksteps2; ++ks) {
      if (!mbar_wait(full0 + 8u * s, full_parity, abort_flag, a.status, FAULT_WAIT_FULL)) return false;
      tc_fence_after();
      const uint32_t a_lo = ring_lo + s * stage_lo;
      issue_kstep<MPS>(d_tmem + acc2_cols, a_lo, hi, a_lo + stage_a_lo, hi, idesc, ks > 0 ? 1u : 0u, leader);
      tc_commit_if(empty0 + 8u * s, leader);
      if (++s == a.stages) {
        s = 0;
        full_parity ^= 1;
      }
    }
    tc_commit_if(acc_full0 + 8u * buf, leader);
  }
  return true;
}

// The producer's (row block, channel tile) advance by the decomposition of gridDim.x with a carry.
__device__ __forceinline__ bool producer_loop_flat(const IgemmArgs& a, const CUtensorMap* tmA, const CUtensorMap* tmB,
                                                   const CUtensorMap* tmA2, const CUtensorMap* tmB2, uint32_t smem_base,
                                                   int stage_bytes, int stage_a, uint32_t full0, uint32_t empty0, bool leader,
                                                   volatile int* abort_flag, int& s, uint32_t& empty_parity) {
  const int k2_end = a.dual ? a.ksteps2 * a.kc : 0;
  int tn = static_cast<int>(blockIdx.x) % a.tiles_n, tm = static_cast<int>(blockIdx.x) / a.tiles_n;
  const int dn = static_cast<int>(gridDim.x) % a.tiles_n, dm = static_cast<int>(gridDim.x) / a.tiles_n;
  const int k_end = a.ksteps * a.kc;
  const bool resident = a.resident_b != 0;
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    const int m0 = tm * kTileM, n0 = tn * a.bn;
    for (int kb = 0; kb < k_end; kb += a.kc) {
      if (!mbar_wait(empty0 + 8u * s, empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY)) return false;
      const uint32_t dst = smem_base + s * stage_bytes;
      mbar_expect_tx_if(full0 + 8u * s, static_cast<uint32_t>(stage_bytes), leader);
      tma_load_2d_if(dst, tmA, full0 + 8u * s, kb, m0, leader);
      if (!resident) tma_load_2d_if(dst + stage_a, tmB, full0 + 8u * s, kb, n0, leader);
      if (++s == a.stages) {
        s = 0;
        empty_parity ^= 1;
      }
    }
    if (k2_end > 0) {
      // shortcut GEMM of a fused residual block: 1x1 filter, stride stride2, no padding, on its own input
      int q0 = 0, p0 = 0, cn = 0;
      if (a.im2col2) {
        q0 = m0 % a.wo;
        const int t = m0 / a.wo;
        p0 = t % a.ho;
        cn = t / a.ho;
      }
      for (int kb = 0; kb < k2_end; kb += a.kc) {
        if (!mbar_wait(empty0 + 8u * s, empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY)) return false;
        const uint32_t dst = smem_base + s * stage_bytes;
        mbar_expect_tx_if(full0 + 8u * s, static_cast<uint32_t>(stage_bytes), leader);
        if (a.im2col2) tma_load_im2col_4d_if(dst, tmA2, full0 + 8u * s, kb, q0 * a.stride2_w, p0 * a.stride2_h, cn, 0, 0, leader);
        else tma_load_2d_if(dst, tmA2, full0 + 8u * s, kb, m0, leader);
        tma_load_2d_if(dst + stage_a, tmB2, full0 + 8u * s, kb, n0, leader);
        if (++s == a.stages) {
          s = 0;
          empty_parity ^= 1;
        }
      }
    }
    tn += dn;
    tm += dm;
    if (tn >= a.tiles_n) {
      tn -= a.tiles_n;
      ++tm;
    }
  }
  return true;
}

// im2col tiles: the same bookkeeping, the K steps as nested loops over (filter row, filter column, channel chunk).
__device__ __forceinline__ bool producer_loop_im2col(const IgemmArgs& a, const CUtensorMap* tmA, const CUtensorMap* tmB,
                                                     uint32_t smem_base, int stage_bytes, int stage_a, uint32_t full0,
                                                     uint32_t empty0, bool leader, volatile int* abort_flag, int& s,
                                                     uint32_t& empty_parity) {
  int tn = static_cast<int>(blockIdx.x) % a.tiles_n, tm = static_cast<int>(blockIdx.x) / a.tiles_n;
  const int dn = static_cast<int>(gridDim.x) % a.tiles_n, dm = static_cast<int>(gridDim.x) / a.tiles_n;
  const bool resident = a.resident_b != 0;
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    const int m0 = tm * kTileM, n0 = tn * a.bn;
    const int q0 = m0 % a.wo, t = m0 / a.wo;
    const int p0 = t % a.ho, cn = t / a.ho;
    const int cw = q0 * a.stride_w - a.pad_l, ch = p0 * a.stride_h - a.pad_t;
    int kb = 0;
    for (int r = 0, off_h = 0; r < a.kh; ++r, off_h += a.dil_h) {
      for (int sx = 0, off_w = 0; sx < a.kw; ++sx, off_w += a.dil_w) {
        for (int c = 0; c < a.cin_bytes; c += a.kc, kb += a.kc) {
          if (!mbar_wait(empty0 + 8u * s, empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY)) return false;
          const uint32_t dst = smem_base + s * stage_bytes;
          mbar_expect_tx_if(full0 + 8u * s, static_cast<uint32_t>(stage_bytes), leader);
          tma_load_im2col_4d_if(dst, tmA, full0 + 8u * s, c, cw, ch, cn, static_cast<uint16_t>(off_w),
                                static_cast<uint16_t>(off_h), leader);
          if (!resident) tma_load_2d_if(dst + stage_a, tmB, full0 + 8u * s, kb, n0, leader);
          if (++s == a.stages) {
            s = 0;
            empty_parity ^= 1;
          }
        }
      }
    }
    tn += dn;
    tm += dm;
    if (tn >= a.tiles_n) {
      tn -= a.tiles_n;
      ++tm;
    }
  }
  return true;
}

// Window-mode tiles of the row-folded stem layers (a handful of MMAs per tile, resident filter, one
// channel tile, one window box per tile): the same short loops as for flat tiles.  The window position
// (tx, ty, image) advances by the decomposition of gridDim.x with carries instead of divisions.
__device__ __forceinline__ bool producer_loop_window_resident(const IgemmArgs& a, const CUtensorMap* tmA, uint32_t smem_base,
                                                              int stage_bytes, uint32_t full0, uint32_t empty0, bool leader,
                                                              volatile int* abort_flag, int& s, uint32_t& empty_parity) {
  int tx = static_cast<int>(blockIdx.x) % a.tiles_x;
  int ty = (static_cast<int>(blockIdx.x) / a.tiles_x) % a.tiles_y;
  int img = (static_cast<int>(blockIdx.x) / a.tiles_x) / a.tiles_y;
  const int dtx = static_cast<int>(gridDim.x) % a.tiles_x;
  const int dty = (static_cast<int>(gridDim.x) / a.tiles_x) % a.tiles_y;
  const int dimg = (static_cast<int>(gridDim.x) / a.tiles_x) / a.tiles_y;
  const uint32_t bytes = static_cast<uint32_t>(a.slab_rows * a.kc);
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    if (!mbar_wait(empty0 + 8u * s, empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY)) return false;
    mbar_expect_tx_if(full0 + 8u * s, bytes, leader);
    tma_load_4d_if(smem_base + s * stage_bytes, tmA, full0 + 8u * s, 0, tx * 8 - a.pad_l, ty * 16 - a.pad_t, img, leader);
    if (++s == a.stages) {
      s = 0;
      empty_parity ^= 1;
    }
    tx += dtx;
    ty += dty;
    img += dimg;
    if (tx >= a.tiles_x) {
      tx -= a.tiles_x;
      ++ty;
    }
    if (ty >= a.tiles_y) {
      ty -= a.tiles_y;
      ++img;
    }
  }
  return true;
}

template <int KH, int KW, int MPS>
__device__ __forceinline__ bool mma_loop_window_resident(const IgemmArgs& a, uint32_t tmem_base, uint32_t acc_stride,
                                                         int nb_mask, int nb_shift, uint32_t ring_lo, uint32_t stage_lo,
                                                         uint32_t row_lo, uint32_t col_lo, uint32_t hi_a, uint32_t bres_lo,
                                                         uint32_t stage_b_lo, uint32_t hi_b, uint32_t idesc, uint32_t full0,
                                                         uint32_t empty0, uint32_t acc_full0, uint32_t acc_empty0,
                                                         bool leader, volatile int* abort_flag) {
  int s = 0, it = 0;
  uint32_t full_parity = 0;
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x, ++it) {
    const int buf = it & nb_mask;
    if (!mbar_wait(acc_empty0 + 8u * buf, ((it >> nb_shift) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_ACCUM)) return false;
    if (!mbar_wait(full0 + 8u * s, full_parity, abort_flag, a.status, FAULT_WAIT_FULL)) return false;
    tc_fence_after();
    issue_window<KH, KW, 1, MPS>(tmem_base + buf * acc_stride, ring_lo + s * stage_lo, row_lo, col_lo, 0u, hi_a, bres_lo,
                                 stage_b_lo, hi_b, idesc, leader);
    tc_commit_if(empty0 + 8u * s, leader);
    tc_commit_if(acc_full0 + 8u * buf, leader);
    if (++s == a.stages) {
      s = 0;
      full_parity ^= 1;
    }
  }
  return true;
}

// ---------------------------------------------------------------- the kernel
// Persistent: one CTA per SM walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...;
// consecutive tile ids share the same 128 pixels (channel tile fastest) so that CTAs running
// side by side hit the same activation rows in L2.  The operand ring and the TMEM
// accumulator buffers run across tile boundaries: the producer prefetches the next tiles
// while the epilogue groups drain the previous ones.
template <int MODE, int ACT, bool STAGED>
__global__ void __launch_bounds__(kThreads, 1)
    igemm_i8_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmRes,
                       const __grid_constant__ CUtensorMap tmOutW,
                       const __grid_constant__ CUtensorMap tmOutB,
                       const __grid_constant__ CUtensorMap tmA2,
                       const __grid_constant__ CUtensorMap tmB2, const IgemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem_al = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  // [epilogue staging: wide tiles, byte tiles][resident filter][operand ring][barriers]
  const int stage_a = kTileM * a.kc;
  const int stage_b = a.bn * a.kc;
  uint8_t* smem_bres = smem_al + a.staging_bytes;
  uint8_t* smem = smem_bres + a.resident_bytes;
  const int stage_bytes = a.slab ? a.cchunks * a.plane_bytes : (a.resident_b ? stage_a : stage_a + stage_b);
  uint8_t* ctrl = smem + a.stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;     // [4] accumulator buffer ready for its epilogue group(s)
  uint64_t* acc_empty = acc_full + kMaxAccBufs;    // [4] accumulator buffer drained
  uint64_t* res_bar = acc_empty + kMaxAccBufs;     // [2][16] per epilogue warp and staging tile: residual landed
  uint64_t* bres_bar = res_bar + 2 * kEpilogueWarps;  // resident filter landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bres_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Per-channel scale and bias of all output channels in shared memory: an epilogue chunk then
  // reads them with broadcast shared loads instead of waiting for L2.  The epilogue warps copy the
  // tables at the start of their role (see there), off the path of the producer and MMA warps.
  const float* ep_scale = a.scale;
  const float* ep_bias = a.bias;
  const float* ep_scale2 = a.scale2;
  const float* ep_bias2 = a.bias2;
  if (a.sb_cols > 0) {
    float* sb = reinterpret_cast<float*>(smem_al + a.sb_off);
    ep_scale = sb;
    ep_bias = sb + a.sb_cols;
    if (a.dual) {
      ep_scale2 = sb + 2 * a.sb_cols;
      ep_bias2 = sb + 3 * a.sb_cols;
    }
  }

  // TMEM: nb accumulator buffers of acc_cols columns each (512 columns in total at most)
  uint32_t acc_cols = 32;
  while (acc_cols < static_cast<uint32_t>(a.bn)) acc_cols <<= 1;
  const int nb = a.acc_bufs;  // 8 (tiles of <= 64 columns), 4, or 2 (tile 256 wide, or a CTA has only a tile or two to do)
  // epilogue groups sharing one buffer (split by columns); with 8 buffers (tiles of <= 64 columns) every
  // group alternates between two buffers, so the MMA warp refills one while the group drains the other
  const int gpb = nb >= kEpilogueGroups ? 1 : kEpilogueGroups / nb;
  const uint32_t acc_stride = a.dual ? 2 * acc_cols : acc_cols;  // dual mode: main and shortcut accumulators side by side
  const uint32_t tmem_cols = acc_stride * nb < 32 ? 32 : acc_stride * nb;

  if (warp == kProducerWarp) {
    // All barriers live in one array (full .. bres); the lanes of this warp initialise them in
    // parallel (a single thread took ~1 us for the 89 of them).  Only the "accumulator drained"
    // barriers expect more than one arrival.
    constexpr int kBarriers = 2 * kMaxStages + 2 * kMaxAccBufs + 2 * kEpilogueWarps + 1;
    const int first_acc_empty = 2 * kMaxStages + kMaxAccBufs;
    for (int i = lane; i < kBarriers; i += 32) {
      const bool drained = i >= first_acc_empty && i < first_acc_empty + kMaxAccBufs;
      mbar_init(smem_u32(&full_bar[i]), drained ? 4 * gpb : 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 0) *abort_flag = 0;
    {
      // descriptor prefetch, one map per lane (unused maps are valid copies of the filter map)
      const CUtensorMap* map = lane == 0 ? &tmA : lane == 1 ? &tmB : lane == 2 ? &tmRes : lane == 3 ? &tmOutW
                               : lane == 4 ? &tmOutB : lane == 5 ? &tmA2 : &tmB2;
      if (lane < 7) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
    }
    __syncwarp();
    if (a.resident_b && lane == 0) {
      // small filter, one channel tile: fetch all of it once; the ring then carries activations only.
      // Filters are not written by the preceding kernel, so this copy does not wait for it.
      const uint32_t bar = smem_u32(bres_bar);
      mbar_expect_tx(bar, static_cast<uint32_t>(a.ksteps * stage_b));
      for (int ks = 0; ks < a.ksteps; ++ks) tma_load_2d(smem_u32(smem_bres) + ks * stage_b, &tmB, bar, ks * a.kc, 0);
    }
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the set-up above overlapped the previous kernel's tail; from here on global memory is touched
  pdl_sync_with_previous_kernel();

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp walks the loop (so that addresses and coordinates stay warp-uniform values)
    // and one elected lane issues the copies.  The loop body is free of divisions: ring position,
    // tap and channel-chunk counters advance incrementally.
    const bool leader = elect_one();
    int s = 0;
    uint32_t empty_parity = 1;  // a fresh barrier passes a wait on parity 1
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    if (a.fast_window)
      ok = producer_loop_window_resident(a, &tmA, smem_base, stage_bytes, smem_u32(&full_bar[0]), smem_u32(&empty_bar[0]),
                                         leader, abort_flag, s, empty_parity);
    for (int tile = blockIdx.x; a.slab && !a.fast_window && tile < a.num_tiles && ok; tile += gridDim.x) {
      // one window per tile: rows ty*16 - pad_t ..., columns tx*8 - pad_l ...; cells outside the
      // image are filled with zeros by the copy engine
      const int tile_m = tile / a.tiles_n;
      const int tx = tile_m % a.tiles_x;
      const int t = tile_m / a.tiles_x;
      const int ty = t % a.tiles_y;
      const int img = t / a.tiles_y;
      ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
      if (!ok) break;
      const uint32_t bar = smem_u32(&full_bar[s]);
      const uint32_t dst = smem_base + s * stage_bytes;
      mbar_expect_tx_if(bar, static_cast<uint32_t>(a.cchunks * a.slab_rows * a.kc), leader);
      for (int cc = 0; cc < a.cchunks; ++cc)
        tma_load_4d_if(dst + cc * a.plane_bytes, &tmA, bar, cc * a.kc, tx * 8 - a.pad_l, ty * 16 - a.pad_t, img,
                       leader);
      if (++s == a.stages) {
        s = 0;
        empty_parity ^= 1;
      }
    }
    if (a.fast_flat)  // flat tiles: one box of activations (and one of the filter, unless resident) per K step
      ok = producer_loop_flat(a, &tmA, &tmB, &tmA2, &tmB2, smem_base, stage_bytes, stage_a, smem_u32(&full_bar[0]),
                              smem_u32(&empty_bar[0]), leader, abort_flag, s, empty_parity);
    if (a.fast_im2col)
      ok = producer_loop_im2col(a, &tmA, &tmB, smem_base, stage_bytes, stage_a, smem_u32(&full_bar[0]), smem_u32(&empty_bar[0]),
                                leader, abort_flag, s, empty_parity);
    for (int tile = blockIdx.x; !a.slab && !a.fast_flat && !a.fast_im2col && tile < a.num_tiles && ok; tile += gridDim.x) {
      const int tile_m = tile / a.tiles_n;
      const int m0 = tile_m * kTileM;
      const int n0 = (tile - tile_m * a.tiles_n) * a.bn;
      int q0 = 0, p0 = 0, cn = 0;
      if (a.im2col || (a.dual && a.im2col2)) {
        q0 = m0 % a.wo;
        const int t = m0 / a.wo;
        p0 = t % a.ho;
        cn = t / a.ho;
      }
      const int cw = q0 * a.stride_w - a.pad_l;
      const int ch = p0 * a.stride_h - a.pad_t;
      int r = 0, sx = 0, cc = 0, kb = 0;  // filter row, filter column, channel chunk, K offset in B
      for (int ks = 0; ks < a.ksteps; ++ks) {
        ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
        if (!ok) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t dst_a = smem_base + s * stage_bytes;
        const uint32_t dst_b = dst_a + stage_a;
#ifdef PLB_TC_FAULT_TEST
        // Test build only: CTA 0 "loses" the copies of the first K step of its first tile (neither armed nor
        // issued), so the MMA warp's bounded wait for that stage runs out.  Nothing traps, spins or faults.
        if (a.test_skip_load && blockIdx.x == 0 && tile == 0 && ks == 0) {
          kb += a.kc;
          if (++cc == a.cchunks) {
            cc = 0;
            if (++sx == a.kw) {
              sx = 0;
              ++r;
            }
          }
          if (++s == a.stages) {
            s = 0;
            empty_parity ^= 1;
          }
          continue;
        }
#endif
        mbar_expect_tx_if(bar, static_cast<uint32_t>(stage_bytes), leader);
        if (a.im2col) {
          tma_load_im2col_4d_if(dst_a, &tmA, bar, cc * a.kc, cw, ch, cn, static_cast<uint16_t>(sx * a.dil_w),
                                static_cast<uint16_t>(r * a.dil_h), leader);
        } else {
          tma_load_2d_if(dst_a, &tmA, bar, kb, m0, leader);
        }
        if (!a.resident_b) tma_load_2d_if(dst_b, &tmB, bar, kb, n0, leader);
        kb += a.kc;
        if (++cc == a.cchunks) {
          cc = 0;
          if (++sx == a.kw) {
            sx = 0;
            ++r;
          }
        }
        if (++s == a.stages) {
          s = 0;
          empty_parity ^= 1;
        }
      }
      // dual mode: the K steps of the shortcut GEMM follow (1x1 filter, stride stride2, no padding)
      for (int ks = 0; a.dual && ok && ks < a.ksteps2; ++ks) {
        ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
        if (!ok) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t dst_a = smem_base + s * stage_bytes;
        mbar_expect_tx_if(bar, static_cast<uint32_t>(stage_bytes), leader);
        if (a.im2col2) tma_load_im2col_4d_if(dst_a, &tmA2, bar, ks * a.kc, q0 * a.stride2_w, p0 * a.stride2_h, cn, 0, 0, leader);
        else tma_load_2d_if(dst_a, &tmA2, bar, ks * a.kc, m0, leader);
        tma_load_2d_if(dst_a + stage_a, &tmB2, bar, ks * a.kc, n0, leader);
        if (++s == a.stages) {
          s = 0;
          empty_parity ^= 1;
        }
      }
    }
    if (!ok || *abort_flag) {
      // Some role of this CTA gave up.  Copies this warp has issued may still be in flight into the ring:
      // give each of them a bounded time to land before the CTA frees its tensor memory and exits.  Stages
      // below s were armed in the current round (their phase has parity empty_parity ^ 1), the others in the
      // round before.
      for (int j = 0; j < a.stages; ++j)
        mbar_wait_drain(smem_u32(&full_bar[j]), j < s ? (empty_parity ^ 1u) : empty_parity);
      if (a.resident_b) mbar_wait_drain(smem_u32(bres_bar), 0);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    // Again the whole warp runs the loop and an elected lane issues: matrix descriptors are
    // warp-uniform values, built from 32-bit halves with as few instructions per MMA as possible
    // (a 128 x 64 x 32 MMA occupies the tensor core for only ~57 cycles).
    const bool leader = elect_one();
    // instruction descriptor: D=s32, A=B=s8, both K-major, N=bn, M=128
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a.bn >> 3) << 17) |
                           (static_cast<uint32_t>(kTileM >> 4) << 24);
    const int mma_per_stage = a.kc / 32;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t hi_b = static_cast<uint32_t>(make_smem_desc(0, a.kc) >> 32);  // layout, 8-row group stride
    // window mode: the 8-row groups of A are one window row (slab_w pixels) apart
    const uint32_t hi_a = a.slab ? ((hi_b & 0xFFFFC000u) | ((static_cast<uint32_t>(a.slab_w * a.kc) >> 4) & 0x3FFFu)) : hi_b;
    const uint32_t lo_flags = 1u << 16;  // leading-dimension byte offset field (unused by swizzled K-major tiles)
    const int nb_mask = nb - 1, nb_shift = nb == 8 ? 3 : (nb == 4 ? 2 : 1);
    // window mode: descriptor steps per filter row / filter column / channel chunk
    const uint32_t row_lo = static_cast<uint32_t>(a.slab_w * a.kc * a.dil_h) >> 4;
    const uint32_t col_lo = static_cast<uint32_t>(a.dil_w * a.kc) >> 4;
    const uint32_t plane_lo = static_cast<uint32_t>(a.plane_bytes) >> 4;
    int window_shape = 0;  // which unrolled issue sequence applies
    if (a.slab) {  // other filter sizes: taps in a loop, the inside of a tap unrolled
      if (a.cchunks == 1 && mma_per_stage == 1) window_shape = 11;
      if (a.cchunks == 1 && mma_per_stage == 2) window_shape = 12;
      if (a.cchunks == 1 && mma_per_stage == 4) window_shape = 14;
      if (a.cchunks == 2 && mma_per_stage == 4) window_shape = 24;
    }
    if (a.slab && a.kh == 4 && a.kw == 1 && a.cchunks == 1 && mma_per_stage == 2) window_shape = 4;  // row-folded 7x7 stem
    if (a.slab && a.kh == 2 && a.kw == 1 && a.cchunks == 1 && mma_per_stage == 2) window_shape = 5;  // row-folded 3x3 stem
    if (a.slab && a.kh == 3 && a.kw == 3) {
      if (a.cchunks == 1 && mma_per_stage == 2) window_shape = 1;
      if (a.cchunks == 1 && mma_per_stage == 4) window_shape = 2;
      if (a.cchunks == 2 && mma_per_stage == 4) window_shape = 3;
    }
    int s = 0, it = 0;
    uint32_t full_parity = 0;
    bool ok = true;
    if (a.resident_b) {
      ok = mbar_wait(smem_u32(bres_bar), 0, abort_flag, a.status, FAULT_WAIT_FULL);
      tc_fence_after();
    }
    const uint32_t bres_lo = ((smem_u32(smem_bres) >> 4) & 0x3FFFu) | lo_flags;
    const uint32_t stage_b_lo = static_cast<uint32_t>(stage_b) >> 4;
    const uint32_t stage_lo = static_cast<uint32_t>(stage_bytes) >> 4;
    const uint32_t ring_lo = ((smem_base >> 4) & 0x3FFFu) | lo_flags;
    if (a.fast_mma && ok) {
      const uint32_t f0 = smem_u32(&full_bar[0]), e0 = smem_u32(&empty_bar[0]);
      const uint32_t af0 = smem_u32(&acc_full[0]), ae0 = smem_u32(&acc_empty[0]);
      const uint32_t stage_a_lo = static_cast<uint32_t>(stage_a) >> 4;
      if (mma_per_stage == 4)
        ok = mma_loop_flat<4>(a, tmem_base, acc_stride, nb_mask, nb_shift, ring_lo, stage_lo, stage_a_lo, bres_lo, stage_b_lo,
                              hi_b, idesc, f0, e0, af0, ae0, acc_cols, leader, abort_flag);
      else if (mma_per_stage == 2)
        ok = mma_loop_flat<2>(a, tmem_base, acc_stride, nb_mask, nb_shift, ring_lo, stage_lo, stage_a_lo, bres_lo, stage_b_lo,
                              hi_b, idesc, f0, e0, af0, ae0, acc_cols, leader, abort_flag);
      else
        ok = mma_loop_flat<1>(a, tmem_base, acc_stride, nb_mask, nb_shift, ring_lo, stage_lo, stage_a_lo, bres_lo, stage_b_lo,
                              hi_b, idesc, f0, e0, af0, ae0, acc_cols, leader, abort_flag);
    }
    if (a.fast_window && ok) {
      const uint32_t f0 = smem_u32(&full_bar[0]), e0 = smem_u32(&empty_bar[0]);
      const uint32_t af0 = smem_u32(&acc_full[0]), ae0 = smem_u32(&acc_empty[0]);
      if (a.kh == 4)
        ok = mma_loop_window_resident<4, 1, 2>(a, tmem_base, acc_stride, nb_mask, nb_shift, ring_lo, stage_lo, row_lo, col_lo,
                                               hi_a, bres_lo, stage_b_lo, hi_b, idesc, f0, e0, af0, ae0, leader, abort_flag);
      else
        ok = mma_loop_window_resident<2, 1, 2>(a, tmem_base, acc_stride, nb_mask, nb_shift, ring_lo, stage_lo, row_lo, col_lo,
                                               hi_a, bres_lo, stage_b_lo, hi_b, idesc, f0, e0, af0, ae0, leader, abort_flag);
    }
    for (int tile = blockIdx.x; !a.fast_mma && !a.fast_window && tile < a.num_tiles && ok; tile += gridDim.x, ++it) {
      int buf = it & nb_mask;
      ok = mbar_wait(smem_u32(&acc_empty[buf]), ((it >> nb_shift) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * acc_stride;
      uint32_t accumulate = 0;
      if (a.slab) {
        ok = mbar_wait(smem_u32(&full_bar[s]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        // Tile row g (8 pixels) is window row g + r*dil_h starting at column sx*dil_w.  The swizzle
        // is a function of the shared-memory address, so a start address shifted by whole
        // pixels addresses the same bytes the copy engine wrote.
        const uint32_t slab_lo = ring_lo + s * stage_lo;
        if (window_shape == 1) {
          issue_window<3, 3, 1, 2>(d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 2) {
          issue_window<3, 3, 1, 4>(d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 3) {
          issue_window<3, 3, 2, 4>(d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 4) {
          issue_window<4, 1, 1, 2>(d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 5) {
          issue_window<2, 1, 1, 2>(d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 11) {
          issue_window_taps<1, 1>(a.kh, a.kw, d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 12) {
          issue_window_taps<1, 2>(a.kh, a.kw, d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 14) {
          issue_window_taps<1, 4>(a.kh, a.kw, d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else if (window_shape == 24) {
          issue_window_taps<2, 4>(a.kh, a.kw, d_tmem, slab_lo, row_lo, col_lo, plane_lo, hi_a, bres_lo, stage_b_lo, hi_b, idesc, leader);
        } else {
          uint32_t b_lo = bres_lo;
          uint32_t row_a = slab_lo;
          for (int r = 0; r < a.kh; ++r, row_a += row_lo) {
            uint32_t tap_a = row_a;
            for (int sx = 0; sx < a.kw; ++sx, tap_a += col_lo) {
              uint32_t a_lo = tap_a;
              for (int cc = 0; cc < a.cchunks; ++cc, a_lo += plane_lo, b_lo += stage_b_lo) {
                for (int j = 0; j < mma_per_stage; ++j) {
                  tc_mma_i8_halves(d_tmem, a_lo + 2u * j, hi_a, b_lo + 2u * j, hi_b, idesc, accumulate, leader);
                  accumulate = 1;
                }
              }
            }
          }
        }
        tc_commit_if(smem_u32(&empty_bar[s]), leader);
        if (++s == a.stages) {
          s = 0;
          full_parity ^= 1;
        }
      }
      uint32_t b_res_lo = bres_lo;
      for (int ks = 0; !a.slab && ks < a.ksteps; ++ks, b_res_lo += stage_b_lo) {
        ok = mbar_wait(smem_u32(&full_bar[s]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = ring_lo + s * stage_lo;
        const uint32_t b_lo = a.resident_b ? b_res_lo : a_lo + (static_cast<uint32_t>(stage_a) >> 4);
        // advance 32 bytes of K inside the swizzle span: +2 in the (addr >> 4) field
        if (mma_per_stage == 4) issue_kstep<4>(d_tmem, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
        else if (mma_per_stage == 2) issue_kstep<2>(d_tmem, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
        else issue_kstep<1>(d_tmem, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
        accumulate = 1;
        tc_commit_if(smem_u32(&empty_bar[s]), leader);  // frees the stage when these MMAs retire
        if (++s == a.stages) {
          s = 0;
          full_parity ^= 1;
        }
      }
      // dual mode: the shortcut GEMM accumulates into the columns next to the main accumulator
      accumulate = 0;
      for (int ks = 0; a.dual && ok && ks < a.ksteps2; ++ks) {
        ok = mbar_wait(smem_u32(&full_bar[s]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = ring_lo + s * stage_lo;
        const uint32_t b_lo = a_lo + (static_cast<uint32_t>(stage_a) >> 4);
        if (mma_per_stage == 4) issue_kstep<4>(d_tmem + acc_cols, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
        else if (mma_per_stage == 2) issue_kstep<2>(d_tmem + acc_cols, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
        else issue_kstep<1>(d_tmem + acc_cols, a_lo, hi_a, b_lo, hi_b, idesc, accumulate, leader);
        accumulate = 1;
        tc_commit_if(smem_u32(&empty_bar[s]), leader);
        if (++s == a.stages) {
          s = 0;
          full_parity ^= 1;
        }
      }
      tc_commit_if(smem_u32(&acc_full[buf]), leader);  // accumulator complete (or drained on a fault)
    }
  } else {
    // ------------------------------------------------------------ epilogue groups
    if (a.sb_cols > 0) {
      // The tables are layer constants (not written by the preceding kernel).  Only the epilogue warps
      // need them, and long after this point, so the copy costs the other roles nothing; all 16 epilogue
      // warps reach this barrier exactly once, before any of their exits.
      float* sb = reinterpret_cast<float*>(smem_al + a.sb_off);
      for (int i = threadIdx.x; i < a.sb_cols; i += 32 * kEpilogueWarps) {
        sb[i] = __ldg(a.scale + i);
        sb[a.sb_cols + i] = __ldg(a.bias + i);
        if (a.dual) {
          sb[2 * a.sb_cols + i] = __ldg(a.scale2 + i);
          sb[3 * a.sb_cols + i] = __ldg(a.bias2 + i);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
    }
    const int group = warp >> 2;     // 0..3
    const int quad = warp & 3;       // TMEM lane quadrant this warp may read
    const int first_it = group / gpb;             // this group's first tile of the CTA's sequence
    const int it_stride = kEpilogueGroups / gpb;  // groups that take whole tiles
    const int col_par = group % gpb; // which part of its columns
    const int nb_shift = nb == 8 ? 3 : (nb == 4 ? 2 : 1);
    // staged I/O: this warp's staging tiles and bookkeeping
    const uint32_t st_w = smem_u32(smem_al) + warp * 4096;
    const int wq = a.bn / gpb;       // columns (= int8 bytes per row) this group owns in a tile
    const uint32_t st_b = smem_u32(smem_al) + a.staging_w_bytes + warp * a.stage_b_warp;
    // int8 staging rows are wq bytes long and swizzled with span wq (as the store's tensor map is):
    // 16-byte chunk j of row r lives at j ^ (r & 7), j ^ ((r >> 1) & 3) or j ^ ((r >> 2) & 1)
    const int b_swz = wq == 128 ? (lane & 7) : (wq == 64 ? ((lane >> 1) & 3) : (wq == 32 ? ((lane >> 2) & 1) : 0));
    const uint32_t my_res_bar = smem_u32(&res_bar[warp]);
    uint32_t res_phase = 0;
    // residual prefetch: two staging tiles per warp (8 KiB apart per warp), one barrier each
    const uint32_t pf_tile[2] = {smem_u32(smem_al) + warp * 8192, smem_u32(smem_al) + warp * 8192 + 4096};
    const uint32_t pf_bar[2] = {smem_u32(&res_bar[warp]), smem_u32(&res_bar[kEpilogueWarps + warp])};
    uint32_t pf_phase[2] = {0, 0};
    int pf_cur = 0;
    bool pf_ready = false;
    bool stores_pending = false;
    bool ok = true;
    // one channel tile (flat 1x1 layers with few channels, where a tile is little work): no divisions per tile
    const bool one_n = MODE != OUT_ADD_RELU && !a.slab && a.tiles_n == 1;
    for (int it = first_it; ok; it += it_stride) {
      const int my_buf = it & (nb - 1);  // the accumulator buffer of this tile
      const long tile_l = static_cast<long>(blockIdx.x) + static_cast<long>(it) * gridDim.x;
      if (tile_l >= a.num_tiles) break;
      const int tile = static_cast<int>(tile_l);
      const int m0 = (one_n ? tile : tile / a.tiles_n) * kTileM;
      const int n0 = one_n ? 0 : (tile % a.tiles_n) * a.bn;
      const long row = static_cast<long>(m0) + quad * 32 + lane;
      const uint32_t lane_addr = tmem_base + my_buf * acc_stride + (static_cast<uint32_t>(quad * 32) << 16);
      bool waited = false;
      if (STAGED && MODE == OUT_ADD_RELU && a.res_prefetch) {
        // Residual convolutions are bound by the latency of the residual fetch: each chunk needs
        // its 4 KiB residual tile before it can do anything.  With two staging tiles per warp the
        // tile of the following chunk (of this or the warp's next output tile) is requested
        // while the current one is computed and stored.  Flat GEMM tiles only.
        const int row0 = m0 + quad * 32;
        const bool active = row0 < a.m_total;
        const int cbase = col_par * wq;
        for (int c = cbase; c < cbase + wq; c += 32) {
          if (n0 + c >= a.cout) break;  // warp-uniform
          bool drained = false;
          if (active && !pf_ready) {
            // nothing was requested ahead for this chunk (first chunk of the warp)
            if (stores_pending) {
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
              stores_pending = false;
              drained = true;
            }
            if (lane == 0) {
              mbar_expect_tx(pf_bar[pf_cur], 4096);
              tma_load_2d(pf_tile[pf_cur], &tmRes, pf_bar[pf_cur], n0 + c, row0);
            }
          }
          if (!waited) {
            ok = mbar_wait(smem_u32(&acc_full[my_buf]), (it >> nb_shift) & 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
            tc_fence_after();
            waited = true;
            if (!ok) break;
          }
          uint32_t r[32];
          tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
          tc_wait_ld();
          // where is this warp's next chunk?
          int nc = c + 32, nrow0 = row0, ncol;
          bool nvalid = true;
          if (nc >= cbase + wq || n0 + nc >= a.cout) {
            const long ntile = tile_l + static_cast<long>(nb) * gridDim.x;
            nvalid = ntile < a.num_tiles;
            const int nt = static_cast<int>(nvalid ? ntile : 0);
            nrow0 = (nt / a.tiles_n) * kTileM + quad * 32;
            nc = cbase;
            ncol = (nt % a.tiles_n) * a.bn + nc;
          } else {
            ncol = n0 + nc;
          }
          nvalid = nvalid && ncol < a.cout && nrow0 < a.m_total;
          if (nvalid) {
            // the other staging tile was last read by the stores of the previous chunk
            if (stores_pending && !drained) {
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
              stores_pending = false;
              drained = true;
            }
            if (lane == 0) {
              mbar_expect_tx(pf_bar[pf_cur ^ 1], 4096);
              tma_load_2d(pf_tile[pf_cur ^ 1], &tmRes, pf_bar[pf_cur ^ 1], ncol, nrow0);
            }
          }
          if (active) {
            ok = mbar_wait(pf_bar[pf_cur], pf_phase[pf_cur], abort_flag, a.status, FAULT_WAIT_FULL);
            pf_phase[pf_cur] ^= 1;
            if (!ok) break;
            if (stores_pending && !drained) {  // the int8 staging rows are rewritten below
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
              stores_pending = false;
            }
            epilogue_chunk_staged<MODE, ACT>(a, ep_scale, ep_bias, r, lane, n0 + c, pf_tile[pf_cur], st_b + lane * 32, 0, 0, true);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (a.y_f32 != nullptr) tma_store_2d(&tmOutW, pf_tile[pf_cur], n0 + c, row0);
              if (a.y_i8 != nullptr) tma_store_2d(&tmOutB, st_b, n0 + c, row0);
              bulk_commit();
            }
            stores_pending = true;
          }
          pf_ready = nvalid;
          pf_cur ^= 1;
        }
      } else if (STAGED) {
        const int row0 = m0 + quad * 32;
        // slab tiles are 16 x 8 pixels: this quadrant owns tile rows quad*4 .. quad*4+3
        int s_w = 0, s_h = 0, s_img = 0;
        if (a.slab) {
          const int tile_m = tile / a.tiles_n;
          s_w = (tile_m % a.tiles_x) * 8;
          const int t = tile_m / a.tiles_x;
          s_h = (t % a.tiles_y) * 16 + quad * 4;
          s_img = t / a.tiles_y;
        }
        const bool active = a.slab ? s_h < a.ho : row0 < a.m_total;  // warp-uniform: some row of this quadrant exists
        const bool use_w = MODE == OUT_F32 || MODE == OUT_ACC || (MODE == OUT_ADD_RELU && a.y_f32 != nullptr);
        const bool dual = MODE == OUT_ADD_RELU && a.dual != 0;  // residual = the shortcut GEMM in the next TMEM columns
        const bool have_res = MODE == OUT_ADD_RELU && (a.residual != nullptr || dual);
        const bool use_b = MODE == OUT_I8 || (MODE == OUT_ADD_RELU && a.y_i8 != nullptr);
        const int cbase = col_par * wq;
        bool wrote_b = false;
        for (int c = cbase; c < cbase + wq; c += 32) {
          if (n0 + c >= a.cout) break;  // warp-uniform
          if (active && stores_pending && (use_w || have_res || c == cbase)) {
            // the staging tiles are about to be overwritten: earlier stores must have read them
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
            stores_pending = false;
          }
          if (active && have_res && !dual && lane == 0) {
            mbar_expect_tx(my_res_bar, 4096);
            if (a.slab) tma_load_4d(st_w, &tmRes, my_res_bar, n0 + c, s_w, s_h, s_img);
            else tma_load_2d(st_w, &tmRes, my_res_bar, n0 + c, row0);
          }
          if (!waited) {
            ok = mbar_wait(smem_u32(&acc_full[my_buf]), (it >> nb_shift) & 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
            tc_fence_after();
            waited = true;
            if (!ok) break;
          }
          if (active && dual) {
            // shortcut value of this chunk: fma(acc2, scale2, bias2) exactly as its own fp32-out
            // convolution would have stored it, written where a fetched residual tile would be
            // (done before the main accumulator is read, to keep both out of the registers at once)
            uint32_t r2[32];
            tc_ld32(lane_addr + acc_cols + static_cast<uint32_t>(c), r2);
            tc_wait_ld();
            const float4* sc4 = reinterpret_cast<const float4*>(ep_scale2 + n0 + c);
            const float4* bi4 = reinterpret_cast<const float4*>(ep_bias2 + n0 + c);
            const uint32_t w_row = st_w + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 sc = sc4[j], bi = bi4[j];
              sts128(w_row + ((j ^ (lane & 7)) << 4),
                     __float_as_uint(fmaf(__int2float_rn((int)r2[4 * j]), sc.x, bi.x)),
                     __float_as_uint(fmaf(__int2float_rn((int)r2[4 * j + 1]), sc.y, bi.y)),
                     __float_as_uint(fmaf(__int2float_rn((int)r2[4 * j + 2]), sc.z, bi.z)),
                     __float_as_uint(fmaf(__int2float_rn((int)r2[4 * j + 3]), sc.w, bi.w)));
            }
          }
          uint32_t r[32];
          tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
          tc_wait_ld();
          if (active) {
            if (dual) {
            } else if (have_res) {
              ok = mbar_wait(my_res_bar, res_phase, abort_flag, a.status, FAULT_WAIT_FULL);
              res_phase ^= 1;
              if (!ok) break;
            }
            epilogue_chunk_staged<MODE, ACT>(a, ep_scale, ep_bias, r, lane, n0 + c, st_w, st_b + lane * wq,
                                             (c - cbase) >> 4, b_swz, have_res);
            if (use_w) {  // make this chunk's staging writes visible to the copy engine
              fence_proxy_async_smem();
              __syncwarp();
            }
            if (use_w && lane == 0) {
              if (a.slab) tma_store_4d(&tmOutW, st_w, n0 + c, s_w, s_h, s_img);
              else tma_store_2d(&tmOutW, st_w, n0 + c, row0);
              bulk_commit();
            }
            if (use_w) stores_pending = true;
            wrote_b = use_b;
          }
        }
        if (wrote_b) {
          if (!use_w) {  // int8-only output: one fence per tile instead of one per chunk
            fence_proxy_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            if (a.slab) tma_store_4d(&tmOutB, st_b, n0 + cbase, s_w, s_h, s_img);
            else tma_store_2d(&tmOutB, st_b, n0 + cbase, row0);
            bulk_commit();
          }
          stores_pending = true;
        }
      } else {
        for (int c = col_par * 32; c < a.bn; c += 32 * gpb) {
          if (n0 + c >= a.cout) break;  // warp-uniform
          float res[32];
          if (MODE == OUT_ADD_RELU) {
            if (a.residual != nullptr && row < a.m_total) {
              load_residual32(a, row, n0 + c, res);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) res[j] = 0.f;
            }
          }
          if (!waited) {
            ok = mbar_wait(smem_u32(&acc_full[my_buf]), (it >> nb_shift) & 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
            tc_fence_after();
            waited = true;
            if (!ok) break;
          }
          uint32_t r[32];
          tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
          tc_wait_ld();
          if (row < a.m_total) epilogue_store32<MODE, ACT>(a, r, res, row, n0 + c);
        }
      }
      if (!waited && ok) {  // nothing to do for this group in this tile: still consume the phase
        ok = mbar_wait(smem_u32(&acc_full[my_buf]), (it >> nb_shift) & 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
        tc_fence_after();
      }
      // this warp no longer reads the buffer: let the MMA warp overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[my_buf]));
    }
    if (STAGED && MODE == OUT_ADD_RELU && (!ok || *abort_flag) && lane == 0) {
      // gave up with a residual tile possibly still on its way into this warp's staging memory
      mbar_wait_drain(pf_bar[0], a.res_prefetch ? pf_phase[0] : res_phase);
      if (a.res_prefetch) mbar_wait_drain(pf_bar[1], pf_phase[1]);
    }
    if (STAGED && lane == 0) bulk_wait_all();  // staging memory must outlive the stores reading it
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(tmem_cols)
                 : "memory");
  }
}

typedef void (*IgemmKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const CUtensorMap, const CUtensorMap, const CUtensorMap, const IgemmArgs);

template <int MODE, bool STAGED>
IgemmKernel pick_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return igemm_i8_tc_kernel<MODE, PLB_ACT_RELU, STAGED>;
    case PLB_ACT_RELU6: return igemm_i8_tc_kernel<MODE, PLB_ACT_RELU6, STAGED>;
    case PLB_ACT_LEAKY: return igemm_i8_tc_kernel<MODE, PLB_ACT_LEAKY, STAGED>;
    default: return igemm_i8_tc_kernel<MODE, PLB_ACT_NONE, STAGED>;
  }
}

template <bool STAGED>
IgemmKernel pick_mode(int mode, int act) {
  switch (mode) {
    case OUT_F32: return pick_act<OUT_F32, STAGED>(act);
    case OUT_I8: return pick_act<OUT_I8, STAGED>(act);
    case OUT_ACC: return igemm_i8_tc_kernel<OUT_ACC, PLB_ACT_NONE, STAGED>;
    default: return igemm_i8_tc_kernel<OUT_ADD_RELU, PLB_ACT_NONE, STAGED>;
  }
}

IgemmKernel pick_kernel(int mode, int act, bool staged) {
  return staged ? pick_mode<true>(mode, act) : pick_mode<false>(mode, act);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;

int load_driver_entry_points() {
  if (g_encode_tiled && g_encode_im2col) return PLB_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr)
    return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  fn = nullptr;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr)
    return fail(PLB_E_CUDA, "cuTensorMapEncodeIm2col is not available from this driver");
  g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  return PLB_OK;
}

CUtensorMapSwizzle swizzle_for(int kc) {
  return kc == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : (kc == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// swizzle of a staging tile whose rows are `bytes` long (no swizzle for other lengths)
CUtensorMapSwizzle swizzle_for_bytes(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                      : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                     : (bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
}

int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  return v && *v ? std::atoi(v) : dflt;
}

// A switch value of -1 means "planner's choice".
int sw_or(int value, int dflt) { return value >= 0 ? value : dflt; }

// Everything one launch needs, derived once per (problem, pointers).
struct IgemmPlan {
  IgemmArgs a;
  alignas(64) CUtensorMap tmA, tmB, tmRes, tmOutW, tmOutB, tmA2, tmB2;
  IgemmKernel kernel;
  size_t smem;
  unsigned grid;
};

std::mutex g_configure_mutex;  // guards the driver entry points and the per-(kernel, device) attribute list

int pick_kc(int cin_pad) { return cin_pad % 128 == 0 ? 128 : (cin_pad % 64 == 0 ? 64 : 32); }

}  // namespace

TcSwitches tc_switches_from_env() {
  TcSwitches s;
  s.slab = env_int("PLB_TC_SLAB", -1);
  s.bn = env_int("PLB_TC_BN", -1);
  s.kc = env_int("PLB_TC_KC", -1);
  s.stages = env_int("PLB_TC_STAGES", -1);
  s.acc_bufs = env_int("PLB_TC_ACC_BUFS", -1);
  s.resident = env_int("PLB_TC_RESIDENT", 1);
  s.staged = env_int("PLB_TC_STAGED", 1);
  s.res_prefetch = env_int("PLB_TC_RES_PREFETCH", -1);
  s.acc_small = env_int("PLB_TC_ACC_SMALL", 1);
  s.sb_smem = env_int("PLB_TC_SB_SMEM", 1);
  s.fast_flat = env_int("PLB_TC_FAST_FLAT", 1);
  s.fast_im2col = env_int("PLB_TC_FAST_IM2COL", 1);
  s.fast_mma = env_int("PLB_TC_FAST_MMA", 1);
  s.fast_dual = env_int("PLB_TC_FAST_DUAL", 1);
  s.fast_window = env_int("PLB_TC_FAST_WINDOW", 1);
  s.pair = env_int("PLB_TC_PAIR", -1);
  s.nchw = env_int("PLB_TC_NCHW", -1);
  s.res_prefetch_tiles = env_int("PLB_TC_RES_PREFETCH_TILES", -1);
  s.dw_strip = env_int("PLB_DW_STRIP", -1);
  s.nchw_gather = env_int("PLB_TC_NCHW_GATHER", -1);
  s.nchw_bres = env_int("PLB_TC_NCHW_BRES", -1);
  s.stem = env_int("PLB_STEM", -1);
  s.dwpw = env_int("PLB_DWPW", -1);
  s.dwpw_tw = env_int("PLB_DWPW_TW", -1);
  s.dwpw_seg = env_int("PLB_DWPW_SEG", -1);
  return s;
}

struct IgemmPlanCache {
  struct Entry {
    IgemmProblem key;
    TcSwitches sw;
    int device;
    IgemmPlan plan;
  };
  std::vector<Entry> entries;
  size_t next = 0;  // round-robin replacement
  long hits = 0;
};
IgemmPlanCache* igemm_plan_cache_create() { return new IgemmPlanCache; }
void igemm_plan_cache_destroy(IgemmPlanCache* c) { delete c; }
long igemm_plan_cache_hits(const IgemmPlanCache* c) { return c ? c->hits : 0; }

bool igemm_tc_supported(const IgemmProblem& p, std::string* why) {
  auto no = [&](const char* msg) {
    if (why) *why = msg;
    return false;
  };
  if (p.cin_pad % 32 != 0) return no("row length (padded input channels) must be a multiple of 32");
  if (p.m_total <= 0 || p.cout <= 0) return no("empty problem");
  if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15))
    return no("operand base addresses must be 16-byte aligned");
  if (p.im2col) {
    if (p.stride_h < 1 || p.stride_h > 8 || p.stride_w < 1 || p.stride_w > 8)
      return no("im2col traversal stride must be 1..8");
    const int up_w = p.pad_r - (p.kw - 1) * p.dil_w, up_h = p.pad_b - (p.kh - 1) * p.dil_h;
    if (p.pad_l > 128 || p.pad_t > 128 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127)
      return no("im2col bounding-box corner outside [-128,127]");
    if ((p.kw - 1) * p.dil_w > 65535 || (p.kh - 1) * p.dil_h > 65535) return no("tap offset too large");
  }
  return true;
}

namespace {

// Derives tile shapes, the shared-memory budget, the kernel instance and all tensor maps of one problem.
int igemm_tc_plan(plb_ctx* ctx, const IgemmProblem& p, const TcSwitches& sw_, IgemmPlan* plan) {
  std::string why;
  if (!igemm_tc_supported(p, &why)) return fail(PLB_E_UNSUPPORTED, "tensor-core path: %s", why.c_str());
  {
    std::lock_guard<std::mutex> lock(g_configure_mutex);
    int rc = load_driver_entry_points();
    if (rc) return rc;
  }

  IgemmArgs& a = plan->a;
  CUtensorMap& tmA = plan->tmA;
  CUtensorMap& tmB = plan->tmB;
  memset(&a, 0, sizeof(a));
  a.im2col = p.im2col;
  a.m_total = p.m_total;
  a.cout = p.cout;
  a.kc = pick_kc(p.cin_pad);
  if ((sw_.kc == 32 || sw_.kc == 64) && sw_.kc < a.kc) a.kc = sw_.kc;
  const bool dual = p.a2 != nullptr;
  if (dual) {
    if (p.out_mode != OUT_ADD_RELU || p.residual != nullptr || p.im2col || p.b2 == nullptr || p.cin_pad2 % 32 != 0 ||
        (reinterpret_cast<uintptr_t>(p.a2) & 15) || (reinterpret_cast<uintptr_t>(p.b2) & 15))
      return fail(PLB_E_UNSUPPORTED, "dual mode needs a flat main GEMM in add+relu mode without a residual tensor");
    const int kc2 = pick_kc(p.cin_pad2);
    if (kc2 < a.kc) a.kc = kc2;  // both GEMMs share the stage geometry
  }
  a.cchunks = p.cin_pad / a.kc;
  a.taps = p.im2col ? p.kh * p.kw : 1;
  a.kw = p.im2col ? p.kw : 1;
  a.kh = p.im2col ? p.kh : 1;
  a.ksteps = a.taps * a.cchunks;
  const int cout16 = (p.cout + 15) / 16 * 16;
  int bn = cout16 < 256 ? cout16 : 256;
  if (dual && bn > 128) bn = 128;  // two accumulators per tile and still two tiles in flight
  // small problems: shrink the channel tile until the grid covers the SMs
  const int tiles_m = (p.m_total + kTileM - 1) / kTileM;
  // (the epilogue works in chunks of 32 columns, so a tile that is not the last one of its row of
  // tiles must be a multiple of 32 wide: halve only down to such widths)
  while (bn > 32 && tiles_m * ((cout16 + bn - 1) / bn) < ctx->sm_count && (bn / 2) % 32 == 0) bn /= 2;
  // Measured per layer (ResNet-50, batch 128): a convolution that adds an fp32 residual and writes fp32 + int8 is
  // bound by its epilogue's HBM traffic and runs best with narrow tiles (512 channels on 28 x 28: 81 us at 64
  // columns, 87 at 128, 90 at 256); a layer of 256 output channels has a single 256-wide tile per row of pixels
  // and loses to wave quantisation (196 tiles on 148 SMs: 10.6 us against 9.9 us at 128 columns).
  if (!dual && p.out_mode == OUT_ADD_RELU && p.residual != nullptr && cout16 >= 512 && bn > 64)
    bn = 64;
  else if (!dual && cout16 == 256 && bn == 256 && tiles_m <= 2 * ctx->sm_count)
    bn = 128;  // (with more tiles the wide tile wins again: 3x3 256 -> 256 on 14 x 14 at 512 images, 49 us against 57)
  bn = sw_or(sw_.bn, bn);
  if (dual && bn > 128) bn = 128;  // also after an override: two accumulators per tile must fit the 512 TMEM columns
  if (bn > cout16) bn = cout16;
  if (bn < cout16 && bn % 32) bn = bn / 32 * 32;
  if (bn < 16 || bn > 256 || bn % 16) return fail(PLB_E_INVALID, "bad channel tile %d", bn);
  a.bn = bn;
  a.tiles_n = (p.cout + bn - 1) / bn;
  // Staged (TMA) epilogue I/O needs power-of-two channel tiles, 16-byte aligned rows and bases.
  const bool want_w = p.out_mode == OUT_F32 || p.out_mode == OUT_ACC ||
                      (p.out_mode == OUT_ADD_RELU && (p.y_f32 != nullptr || p.residual != nullptr || dual));
  const bool want_b = p.out_mode == OUT_I8 || (p.out_mode == OUT_ADD_RELU && p.y_i8 != nullptr);
  auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  bool staged = sw_.staged != 0 && (bn == 32 || bn == 64 || bn == 128 || bn == 256);
  if (want_w && (p.ldy % 4 != 0)) staged = false;
  if (want_b && (p.ldy % 16 != 0)) staged = false;
  if (p.out_mode == OUT_ADD_RELU) {
    if (!aligned16(p.residual) || !aligned16(p.y_f32) || !aligned16(p.y_i8)) staged = false;
  } else if (!aligned16(p.y)) {
    staged = false;
  }
  // The residual tile is fetched one chunk ahead of its use.  Measured inside the network (ResNet-50, 128 images, graph
  // replays on one box): 1.799 ms per step with the prefetch in all twelve residual convolutions, 1.842 with it only in
  // the launches of up to 12 tiles per SM, 1.848 with up to 3 (the earlier rule, taken from single-layer loops, in which
  // the residual tensor of the previous iteration is still in L2 and the prefetch measures slower).
  // In launches of 1024 images (170 - 340 tiles per SM) it costs 2 % (80.9k against 82.6k images/s), at 256 images it is
  // neutral: the limit is 50 tiles per SM (PLB_TC_RES_PREFETCH_TILES).
  const bool short_run = static_cast<long>(tiles_m) * ((p.cout + bn - 1) / bn) <=
                         static_cast<long>(sw_or(sw_.res_prefetch_tiles, 50)) * ctx->sm_count;
  a.res_prefetch = staged && p.out_mode == OUT_ADD_RELU && p.residual != nullptr && !p.im2col &&
                   sw_or(sw_.res_prefetch, short_run ? 1 : 0) != 0;
  a.staging_w_bytes = staged && want_w ? kEpilogueWarps * (a.res_prefetch ? 8192 : 4096) : 0;
  // With many tiles per CTA four accumulator buffers keep every epilogue group on its own tile;
  // with one or two tiles the drain of the last tile is what is left exposed, so two groups
  // share a tile (by column halves) and finish it in half the time.
  {
    const long tiles_total = static_cast<long>(tiles_m) * ((p.cout + bn - 1) / bn);
    const bool few = tiles_total <= 2L * ctx->sm_count;
    a.acc_bufs = bn > 128 ? 2 : (few && bn >= 64 ? 2 : 4);  // 8 (tiles of <= 64 columns) is possible and measured equal
    a.acc_bufs = sw_or(sw_.acc_bufs, a.acc_bufs);
    if (dual) a.acc_bufs = 2;
    if (a.acc_bufs != 2 && a.acc_bufs != 4 && a.acc_bufs != 8) return fail(PLB_E_INVALID, "accumulator buffers must be 2, 4 or 8");
    if (a.acc_bufs == 8 && bn > 64) a.acc_bufs = 4;
    if (a.acc_bufs == 4 && bn > 128) a.acc_bufs = 2;
    if (a.acc_bufs == 2 && bn < 64) a.acc_bufs = 4;
  }
  {
    const int wq_h = bn / (a.acc_bufs >= kEpilogueGroups ? 1 : kEpilogueGroups / a.acc_bufs);
    // 32 rows of wq bytes per warp; 128-byte-swizzled tiles (wq = 128) need 1 KiB alignment, which 4 KiB keeps
    a.stage_b_warp = staged && want_b ? (wq_h == 128 ? 4096 : 32 * wq_h) : 0;
    if (a.res_prefetch && want_b) a.stage_b_warp = 1024;  // int8 results leave chunk by chunk (32 rows x 32 bytes)
  }
  a.sb_off = a.staging_w_bytes + kEpilogueWarps * a.stage_b_warp;
  a.sb_cols = 0;
  if (staged && p.out_mode != OUT_ACC && sw_.sb_smem != 0) {
    const int cols = (p.cout + 31) / 32 * 32;  // the device arrays are readable up to the next multiple of 64 floats
    if (cols * 8 * (dual ? 2 : 1) <= 16 * 1024) a.sb_cols = cols;
  }
  a.staging_bytes = (a.sb_off + a.sb_cols * 8 * (dual ? 2 : 1) + 1023) / 1024 * 1024;
  if (a.res_prefetch) {
    // the doubled staging leaves less room for the operand ring: shorter K steps keep three stages
    while (a.kc > 32 && (225 * 1024 - a.staging_bytes - kCtrlBytes) / ((kTileM + bn) * a.kc) < 3) {
      a.kc /= 2;
      a.cchunks = p.cin_pad / a.kc;
      a.ksteps = a.taps * a.cchunks;
    }
  }
  const int tiles_n_h = (p.cout + bn - 1) / bn;
  const int resident_bytes = (a.ksteps * bn * a.kc + 1023) / 1024 * 1024;
  const bool can_resident = sw_.resident != 0 && tiles_n_h == 1 && resident_bytes <= kMaxResidentB && !dual;
  a.resident_b = can_resident && tiles_m > ctx->sm_count;  // worth it only when a CTA walks several tiles
  // Slab mode: stride-1 filters with several taps read each input pixel once per tile instead of
  // once per tap.  Output tiles are 16 x 8 pixels, so images much smaller than that waste too
  // many accumulator rows.
  int tiles_m_eff = tiles_m;
  if (p.im2col && a.taps > 1 && p.stride_h == 1 && p.stride_w == 1 && staged) {
    const int tx = (p.wo + 7) / 8, ty = (p.ho + 15) / 16;
    const int sw_px = 8 + (p.kw - 1) * p.dil_w, sh_px = 16 + (p.kh - 1) * p.dil_h;
    const double waste = static_cast<double>(tx) * 8 * ty * 16 / (static_cast<double>(p.wo) * p.ho);
    const int plane = (sw_px * sh_px * a.kc + 1023) / 1024 * 1024;
    const bool geom_ok = sw_px <= 256 && sh_px <= 256 && sw_px * a.kc <= 0x3FFF * 16;
    const int room = 225 * 1024 - a.staging_bytes - kCtrlBytes - 1024;
    const bool fits = geom_ok && can_resident && 2 * a.cchunks * plane + resident_bytes <= room;
    // (Streaming a filter that does not fit through a ring of its own was measured on 128->128 and 256->256
    // 3x3 layers and was no faster than im2col mode: with 128-wide tiles every MMA reads 8 KiB of shared
    // memory in 64 cycles, the whole shared-memory bandwidth.  Window mode therefore needs a resident filter.)
    const int dflt = waste <= 1.35 && fits && a.resident_b;
    if (fits && sw_or(sw_.slab, dflt) != 0) {
      a.slab = 1;
      a.resident_b = 1;
      a.kh = p.kh;
      a.slab_w = sw_px;
      a.slab_rows = sw_px * sh_px;
      a.plane_bytes = plane;
      a.tiles_x = tx;
      a.tiles_y = ty;
      tiles_m_eff = p.batch * tx * ty;
    }
  }
  a.resident_bytes = a.resident_b ? resident_bytes : 0;
  a.fast_window = a.slab && a.resident_b && a.tiles_n == 1 && a.cchunks == 1 && a.kc == 64 && a.kw == 1 &&
                  (a.kh == 4 || a.kh == 2) && !dual && sw_.fast_window != 0;
  a.fast_flat = !a.slab && !p.im2col && (!dual || sw_.fast_dual != 0) && sw_.fast_flat != 0;
  a.cin_bytes = a.cchunks * a.kc;
  a.fast_im2col = !a.slab && p.im2col && !dual && sw_.fast_im2col != 0;
  // the MMA warp's short loop does not care how the A tile of a stage was fetched: im2col tiles take it too
  a.fast_mma = a.fast_flat || (!a.slab && !dual && sw_.fast_mma != 0);
  const int stage_bytes = (kTileM + bn) * a.kc;
  const int ring_stage_bytes = a.slab ? a.cchunks * a.plane_bytes : (a.resident_b ? kTileM * a.kc : stage_bytes);
  // one CTA per SM: spend (almost) all remaining shared memory on the operand ring
  int stages = (225 * 1024 - a.staging_bytes - kCtrlBytes - a.resident_bytes) / ring_stage_bytes;
  stages = sw_or(sw_.stages, stages);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  a.stages = stages;
  a.ho = p.ho; a.wo = p.wo;
  a.stride_h = p.stride_h; a.stride_w = p.stride_w;
  a.pad_t = p.pad_t; a.pad_l = p.pad_l;
  a.dil_h = p.dil_h; a.dil_w = p.dil_w;
  a.out_mode = p.out_mode;
  a.ldy = p.ldy;
  a.y = p.y;
  a.scale = p.epi.scale; a.bias = p.epi.bias; a.act = p.epi.act; a.alpha = p.epi.alpha;
  a.acc_small = p.epi.acc_small && sw_.acc_small != 0;
  a.residual = p.residual; a.y_f32 = p.y_f32; a.y_i8 = p.y_i8;
  a.inv_next_scale = p.inv_next_scale;
  a.status = ctx->d_status;
#ifdef PLB_TC_FAULT_TEST
  a.test_skip_load = env_int("PLB_TC_TEST_SKIP_LOAD", 0);
#endif
  if (dual) {
    if (!staged) return fail(PLB_E_UNSUPPORTED, "dual mode needs the staged epilogue (16-byte aligned rows, power-of-two tile)");
    a.dual = 1;
    a.cchunks2 = p.cin_pad2 / a.kc;
    a.ksteps2 = a.cchunks2;
    a.im2col2 = p.im2col2;
    a.stride2_h = p.stride2_h;
    a.stride2_w = p.stride2_w;
    a.scale2 = p.scale2;
    a.bias2 = p.bias2;
    a.ho = p.ho; a.wo = p.wo;
  }

  const CUtensorMapSwizzle sw = swizzle_for(a.kc);
  {
    // filter: [cout, taps*cin_pad] bytes, box = kc x bn
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.taps) * p.cin_pad, static_cast<cuuint64_t>(p.cout)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.taps) * p.cin_pad};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(bn)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_tiled(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.b), dims,
                                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(filter) failed: %d", (int)r);
  }
  if (a.slab) {
    // plain tiled view of the NHWC input: a box is one channel chunk of a tile's input window
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.w),
                          static_cast<cuuint64_t>(p.h), static_cast<cuuint64_t>(p.batch)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(p.cin_pad),
                             static_cast<cuuint64_t>(p.cin_pad) * p.w,
                             static_cast<cuuint64_t>(p.cin_pad) * p.w * p.h};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(a.slab_w),
                         static_cast<cuuint32_t>(a.slab_rows / a.slab_w), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode_tiled(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(p.a), dims,
                                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(input window) failed: %d", (int)r);
  } else if (!p.im2col) {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.m_total)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.cin_pad)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(kTileM)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_tiled(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.a), dims,
                                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(activations) failed: %d", (int)r);
  } else {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.w),
                          static_cast<cuuint64_t>(p.h), static_cast<cuuint64_t>(p.batch)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(p.cin_pad),
                             static_cast<cuuint64_t>(p.cin_pad) * p.w,
                             static_cast<cuuint64_t>(p.cin_pad) * p.w * p.h};
    int lower[2] = {-p.pad_l, -p.pad_t};
    int upper[2] = {p.pad_r - (p.kw - 1) * p.dil_w, p.pad_b - (p.kh - 1) * p.dil_h};
    cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(p.stride_w), static_cast<cuuint32_t>(p.stride_h), 1};
    CUresult r = g_encode_im2col(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(p.a), dims,
                                 strides, lower, upper, static_cast<cuuint32_t>(a.kc),
                                 static_cast<cuuint32_t>(kTileM), estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeIm2col failed: %d", (int)r);
  }

  CUtensorMap& tmA2 = plan->tmA2;
  CUtensorMap& tmB2 = plan->tmB2;
  tmA2 = tmB;
  tmB2 = tmB;
  if (dual) {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cin_pad2), static_cast<cuuint64_t>(p.cout)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.cin_pad2)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(bn)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_tiled(&tmB2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.b2), dims, strides, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(shortcut filter) failed: %d", (int)r);
    if (!p.im2col2) {
      cuuint64_t adims[2] = {static_cast<cuuint64_t>(p.cin_pad2), static_cast<cuuint64_t>(p.m_total)};
      cuuint32_t abox[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(kTileM)};
      r = g_encode_tiled(&tmA2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.a2), adims, strides, abox, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(shortcut input) failed: %d", (int)r);
    } else {
      // 1x1 filter read with a stride: the im2col traversal with no halo
      cuuint64_t adims[4] = {static_cast<cuuint64_t>(p.cin_pad2), static_cast<cuuint64_t>(p.w2),
                             static_cast<cuuint64_t>(p.h2), static_cast<cuuint64_t>(p.batch)};
      cuuint64_t astr[3] = {static_cast<cuuint64_t>(p.cin_pad2), static_cast<cuuint64_t>(p.cin_pad2) * p.w2,
                            static_cast<cuuint64_t>(p.cin_pad2) * p.w2 * p.h2};
      // no halo: the bounding box is the whole image, base pixels advance by the stride
      int lower[2] = {0, 0};
      int upper[2] = {0, 0};
      cuuint32_t aestr[4] = {1, static_cast<cuuint32_t>(p.stride2_w), static_cast<cuuint32_t>(p.stride2_h), 1};
      r = g_encode_im2col(&tmA2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(p.a2), adims, astr, lower, upper,
                          static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(kTileM), aestr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeIm2col(shortcut input) failed: %d", (int)r);
    }
  }
  // output-side tensor maps: [m_total, ldy] matrices, 32-row boxes
  CUtensorMap& tmRes = plan->tmRes;
  CUtensorMap& tmOutW = plan->tmOutW;
  CUtensorMap& tmOutB = plan->tmOutB;
  tmRes = tmOutW = tmOutB = tmB;  // unused ones stay valid copies
  if (staged) {
    auto encode_out = [&](CUtensorMap* tm, const void* base, int elem_bytes, int box_cols,
                          CUtensorMapSwizzle swz) -> CUresult {
      if (a.slab) {
        // [batch, ho, wo, ldy]: a warp's 32 rows are 4 tile rows of 8 pixels
        const cuuint64_t row = static_cast<cuuint64_t>(p.ldy) * elem_bytes;
        cuuint64_t dims4[4] = {static_cast<cuuint64_t>(p.cout), static_cast<cuuint64_t>(p.wo),
                               static_cast<cuuint64_t>(p.ho), static_cast<cuuint64_t>(p.batch)};
        cuuint64_t strides4[3] = {row, row * p.wo, row * p.wo * p.ho};
        cuuint32_t box4[4] = {static_cast<cuuint32_t>(box_cols), 8, 4, 1};
        cuuint32_t estr4[4] = {1, 1, 1, 1};
        return g_encode_tiled(tm, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32,
                              4, const_cast<void*>(base), dims4, strides4, box4, estr4,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      }
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cout), static_cast<cuuint64_t>(p.m_total)};
      cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldy) * elem_bytes};
      cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), 32};
      cuuint32_t estr[2] = {1, 1};
      return g_encode_tiled(tm, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32,
                            2, const_cast<void*>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    CUresult r = CUDA_SUCCESS;
    const int wq = bn / (a.acc_bufs >= kEpilogueGroups ? 1 : kEpilogueGroups / a.acc_bufs);  // int8 bytes per staged row
    if (p.out_mode == OUT_ADD_RELU) {
      if (p.residual) r = encode_out(&tmRes, p.residual, 4, 32, CU_TENSOR_MAP_SWIZZLE_128B);
      if (r == CUDA_SUCCESS && p.y_f32) r = encode_out(&tmOutW, p.y_f32, 4, 32, CU_TENSOR_MAP_SWIZZLE_128B);
      if (r == CUDA_SUCCESS && p.y_i8) {
        if (a.res_prefetch) r = encode_out(&tmOutB, p.y_i8, 1, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
        else r = encode_out(&tmOutB, p.y_i8, 1, wq, swizzle_for_bytes(wq));
      }
    } else if (p.out_mode == OUT_I8) {
      r = encode_out(&tmOutB, p.y, 1, wq, swizzle_for_bytes(wq));
    } else {
      r = encode_out(&tmOutW, p.y, 4, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(output) failed: %d", (int)r);
  }

  auto smem_needed = [&]() {
    return static_cast<size_t>(a.staging_bytes) + a.resident_bytes + static_cast<size_t>(stages) * ring_stage_bytes +
           kCtrlBytes + 1024;
  };
  if (smem_needed() > 227 * 1024 && a.sb_cols > 0) {
    // a pipeline sized to the last kilobyte (minimum ring next to a large resident filter): the
    // scale / bias tables stay in global memory
    a.sb_cols = 0;
    a.staging_bytes = (a.sb_off + 1023) / 1024 * 1024;
  }
  const size_t smem = smem_needed();
  if (smem > 227 * 1024) return fail(PLB_E_UNSUPPORTED, "pipeline needs %zu bytes of shared memory", smem);
  {
    // tensor memory: acc_bufs buffers of the tile's columns rounded up to a power of two (twice that in dual mode)
    int acc_cols = 32;
    while (acc_cols < bn) acc_cols <<= 1;
    if (acc_cols * (dual ? 2 : 1) * a.acc_bufs > 512)
      return fail(PLB_E_INVALID, "tile of %d columns with %d accumulator buffers does not fit the 512 columns of tensor memory",
                  bn, a.acc_bufs);
  }
  IgemmKernel kernel = pick_kernel(p.out_mode, p.epi.act, staged);
  {
    // the attribute belongs to (function, device): remember which pairs have been configured
    std::lock_guard<std::mutex> lock(g_configure_mutex);
    static std::vector<std::pair<const void*, int>> configured;
    const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), ctx->device);
    if (std::find(configured.begin(), configured.end(), key) == configured.end()) {
      PLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      configured.push_back(key);
    }
  }
  const long tiles = static_cast<long>(tiles_m_eff) * a.tiles_n;
  if (tiles > 0x7fffffffL) return fail(PLB_E_UNSUPPORTED, "too many tiles");
  a.num_tiles = static_cast<int>(tiles);
  plan->kernel = kernel;
  plan->smem = smem;
  plan->grid = static_cast<unsigned>(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  return PLB_OK;
}

}  // namespace

int igemm_tc_launch(plb_ctx* ctx, const IgemmProblem& p, IgemmPlanCache* cache) {
  if (igemm_pair_wanted(ctx, p)) return igemm_pair_launch(ctx, p);
  static const TcSwitches kDefaults;
  const TcSwitches& sw = p.sw ? *p.sw : kDefaults;
  const IgemmPlan* plan = nullptr;
  IgemmPlan local;
  if (cache) {
    for (auto& e : cache->entries) {
      if (e.device == ctx->device && memcmp(&e.key, &p, sizeof(p)) == 0 && memcmp(&e.sw, &sw, sizeof(sw)) == 0) {
        plan = &e.plan;
        ++cache->hits;
        break;
      }
    }
    if (!plan) {
      constexpr size_t kMaxEntries = 8;
      IgemmPlanCache::Entry e;
      memcpy(&e.key, &p, sizeof(p));
      e.sw = sw;
      e.device = ctx->device;
      int rc = igemm_tc_plan(ctx, p, sw, &e.plan);
      if (rc) return rc;
      e.plan.a.status = nullptr;  // filled per launch: the status word belongs to the ctx
      if (cache->entries.size() < kMaxEntries) {
        cache->entries.push_back(e);
        plan = &cache->entries.back().plan;
      } else {
        cache->entries[cache->next] = e;
        plan = &cache->entries[cache->next].plan;
        cache->next = (cache->next + 1) % kMaxEntries;
      }
    }
  } else {
    int rc = igemm_tc_plan(ctx, p, sw, &local);
    if (rc) return rc;
    plan = &local;
  }
  IgemmArgs a = plan->a;
  a.status = ctx->d_status;
  PLB_CUDA(launch_kernel(plan->kernel, dim3(plan->grid), dim3(kThreads), plan->smem, ctx->stream, plan->tmA, plan->tmB,
                         plan->tmRes, plan->tmOutW, plan->tmOutB, plan->tmA2, plan->tmB2, a));
  ctx->launches++;
  if (a.slab) ctx->window_launches++;
  return PLB_OK;
}

}  // namespace plb
