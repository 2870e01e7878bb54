// Depthwise 3x3 convolution and the 1x1 convolution that follows it in ONE launch: the int8 output of the
// depthwise layer is produced by CUDA warps straight into the swizzled K-major operand tiles that tcgen05.mma
// consumes, so it never reaches memory (a MobileNet block reads its input and writes its output, nothing else).
// The reference runs the two layers as two kernels (lite/kernels/x86/conv_compute.cc:216-341 with groups = C, then
// the same file's 1x1 path); the arithmetic here is that of the two-kernel sequence, bit for bit: int32 depthwise
// sums -> fma(scale, bias) -> activation -> clamp -> round to nearest even -> int8, then the int8 GEMM and its
// requantiser.
//
// Geometry.  An output tile of the 1x1 stage is 128 pixels = TH rows x TW columns of one image (TW = 4, 8 or 16).
// A depthwise thread owns 4 channels x 4 columns and slides DOWN a strip of TW columns (dw_device.cuh), writing every
// finished output row into the operand tile that row belongs to; C * TW / 16 threads (a "group" of 1, 2, 4 or 8 warps)
// cover a strip, and the 8 depthwise warps of a CTA form 8 / that many groups working on different strips at once.
// A work item is a strip segment of seg_rows output rows (T = seg_rows / TH tiles); the items of a CTA are dealt to
// its groups round after round, and the tiles enter the operand ring in the fixed order (round, tile of the item,
// group), which every role can enumerate for itself:
//   depthwise groups  wait empty[stage], write the rows of a tile, arrive on full[stage]   (one arrival per warp)
//   MMA warp          waits full[stage] and an empty accumulator, issues the K steps against the resident filter,
//                     commits to empty[stage] and acc_full[buffer]
//   epilogue warps    (4, one per TMEM lane quadrant) requantise the accumulators, stage 32 pixels x 128 channels in
//                     shared memory and write them with one 4-D TMA store, which clips at the image border
// Every wait is bounded (tc::mbar_wait); a role that gives up raises the abort flag, the others follow, the CTA frees
// its tensor memory and returns, and the ctx status word carries the fault.
#include "fused_dwpw.cuh"

#include <algorithm>
#include <mutex>

#include "dw_device.cuh"
#include "tc_device.cuh"

namespace plb {
namespace {

using namespace tc;
using namespace dw;

constexpr int kDwWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kEpiWarp0 = kDwWarps;            // a multiple of 4: epilogue warp e reads TMEM lane quadrant e
constexpr int kMmaWarp = kDwWarps + kEpiWarps;
// Registers are handed out to warps four at a time, so the CTA is four whole warpgroups: two of depthwise warps, the
// epilogue warps, and the MMA warp with three idle companions.  The kernel starts with 128 registers per thread; the
// depthwise warpgroups then grow to 152 with what the other two give back (setmaxnreg).
constexpr int kThreads = 512;
constexpr int kDwRegs = 152, kEpiRegs = 112, kMmaRegs = 40;
constexpr int kMaxStages = 16;
constexpr int kMaxAccBufs = 8;
constexpr int kCtrlBytes = 1024;
constexpr int kStagingBytes = kEpiWarps * 2 * 4096;  // two buffers of 32 pixels x 128 bytes per epilogue warp

struct DwpwArgs {
  const int8_t* x;
  const int8_t* wdw;
  int cg_pad;
  const float* dw_scale;
  const float* dw_bias;
  float dw_lo, dw_ub;       // clamp of the depthwise requantiser: [-127, 127], [0, 127] or [0, alpha]
  int h, w, c, ho, wo, pad_t, pad_l;
  int tw, th, col_blocks, seg_rows, segs, tiles_per_item, total_items;
  int groups, warps_per_group;
  int kc, kchunks, stages, stage_bytes;
  int cout, acc_cols, acc_bufs, b_bytes;
  const float* scale;
  const float* bias;
  float alpha;
  int acc_small;
  int* status;
};

__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void bulk_wait_read_1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------ depthwise role
// State of the tile a group is filling.
struct TileCursor {
  uint32_t dst_row;   // shared-memory address of the current tile row (row 0 of the stage + ty * row pitch)
  int ty;             // row inside the tile
  int q;              // position of the tile in the CTA's tile order
  int tiles_done;
  bool ok;
};

template <int S, int CS>
__device__ __forceinline__ void depthwise_role(const DwpwArgs& a, const uint32_t ring, uint64_t* full_bar,
                                               uint64_t* empty_bar, volatile int* abort_flag, const int warp,
                                               const int lane, const int nb) {
  constexpr int IW = 3 * S + 3;
  const int wpg = a.warps_per_group;
  const int G = a.groups;
  const int g = warp / wpg;
  const int u = (warp - g * wpg) * 32 + lane;
  const int cquads = a.c >> 2;
  const int cg = u / cquads, cq = u - cg * cquads;
  const int c0 = cq * 4;
  const int cs = CS ? CS : a.c;
  const int T = a.tiles_per_item;

  uint32_t wr[3][4];
#pragma unroll
  for (int r = 0; r < 3; ++r)
    transpose4x4(__ldg(reinterpret_cast<const uint32_t*>(a.wdw + static_cast<long>(r * 3 + 0) * a.cg_pad + c0)),
                 __ldg(reinterpret_cast<const uint32_t*>(a.wdw + static_cast<long>(r * 3 + 1) * a.cg_pad + c0)),
                 __ldg(reinterpret_cast<const uint32_t*>(a.wdw + static_cast<long>(r * 3 + 2) * a.cg_pad + c0)), 0u, wr[r]);
  const float4 sc = *reinterpret_cast<const float4*>(a.dw_scale + c0);
  const float4 bi = *reinterpret_cast<const float4*>(a.dw_bias + c0);
  const float lo = a.dw_lo, ub = a.dw_ub;

  // Where this thread's four pixels of tile row 0 lie inside a stage: [K chunk][128 pixels][kc bytes], the 16-byte
  // chunks of a pixel XOR-swizzled with the pixel index as the matrix descriptor's swizzle mode expects.
  const int kc = a.kc;
  const int kch = c0 / kc, within = c0 - kch * kc, chunk = within >> 4;
  uint32_t offs[4];
#pragma unroll
  for (int ox = 0; ox < 4; ++ox) {
    const int r = cg * 4 + ox;
    const int swz = kc == 128 ? (r & 7) : (kc == 64 ? ((r >> 1) & 3) : ((r >> 2) & 1));
    offs[ox] = static_cast<uint32_t>(kch * (128 * kc) + r * kc + ((chunk ^ swz) << 4) + (within & 15));
  }
  const uint32_t row_pitch = static_cast<uint32_t>(a.tw * kc);
  // TW = 4 (kc = 128 only): the swizzle phase of a pixel row alternates from one tile row to the next
  const uint32_t row_toggle = a.tw == 4 ? 64u : 0u;
  const float2 magic = make_float2(12582912.f, 12582912.f), neg_magic = make_float2(-12582912.f, -12582912.f);

  for (int k = g; k < nb; k += G) {
    const int rd = k / G;
    const int Gk = min(G, nb - rd * G);
    const int item = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
    const int seg = item % a.segs;
    const int t = item / a.segs;
    const int cb = t % a.col_blocks;
    const long n = t / a.col_blocks;
    const int oh0 = seg * a.seg_rows;
    const int rows = min(a.seg_rows, a.ho - oh0);
    const int ow0 = cb * a.tw + cg * 4;
    const int ncols = a.wo - ow0;
    const int ih0 = oh0 * S - a.pad_t, iw0 = ow0 * S - a.pad_l;
    uint32_t colmask = 0;
    if (ncols > 0) {
#pragma unroll
      for (int ix = 0; ix < IW; ++ix)
        if (iw0 + ix >= 0 && iw0 + ix < a.w) colmask |= 1u << ix;
    }
    const long row_step = static_cast<long>(a.w) * cs;
    const int8_t* xrow = a.x + (((n * a.h + ih0) * a.w + iw0) * static_cast<long>(cs) + c0);
    const int in_rows = (rows - 1) * S + 3;

    TileCursor tc_;
    tc_.q = rd * T * G + g;
    tc_.ty = 0;
    tc_.tiles_done = 0;
    {
      const int stage = tc_.q % a.stages, use = tc_.q / a.stages;
      tc_.ok = mbar_wait(smem_u32(&empty_bar[stage]), (use & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_EMPTY);
      tc_.dst_row = ring + static_cast<uint32_t>(stage * a.stage_bytes);
    }
    // the tile is complete (or the item has no more rows for it): hand it to the MMA warp, move to the next one
    auto finish_tile = [&]() {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&full_bar[tc_.q % a.stages]));
      ++tc_.tiles_done;
      tc_.q += Gk;
      tc_.ty = 0;
      if (tc_.tiles_done < T) {
        const int stage = tc_.q % a.stages, use = tc_.q / a.stages;
        tc_.ok = mbar_wait(smem_u32(&empty_bar[stage]), (use & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_EMPTY);
        tc_.dst_row = ring + static_cast<uint32_t>(stage * a.stage_bytes);
      }
    };
    // one finished output row: requantise (same instruction sequence as the stand-alone kernel) and store
    auto emit_row = [&](int (&acc)[4][4]) {
#pragma unroll
      for (int ox = 0; ox < 4; ++ox) {
        const float2 v01 =
            __ffma2_rn(__fadd2_rn(make_float2(__int_as_float(acc[ox][0]), __int_as_float(acc[ox][1])), neg_magic),
                       make_float2(sc.x, sc.y), make_float2(bi.x, bi.y));
        const float2 v23 =
            __ffma2_rn(__fadd2_rn(make_float2(__int_as_float(acc[ox][2]), __int_as_float(acc[ox][3])), neg_magic),
                       make_float2(sc.z, sc.w), make_float2(bi.z, bi.w));
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[ox][c] = kDwMagic;
        const float2 q01 = __fadd2_rn(make_float2(fminf(fmaxf(v01.x, lo), ub), fminf(fmaxf(v01.y, lo), ub)), magic);
        const float2 q23 = __fadd2_rn(make_float2(fminf(fmaxf(v23.x, lo), ub), fminf(fmaxf(v23.y, lo), ub)), magic);
        if (ox < ncols)
          sts32(tc_.dst_row + offs[ox],
                __byte_perm(__byte_perm(__float_as_uint(q01.x), __float_as_uint(q01.y), 0x0040),
                            __byte_perm(__float_as_uint(q23.x), __float_as_uint(q23.y), 0x0040), 0x5410));
        offs[ox] ^= row_toggle;
      }
      tc_.dst_row += row_pitch;
      if (++tc_.ty == a.th) finish_tile();
    };

    uint32_t win[4][4];
    if (S == 1) {
      int acc[3][4][4];
#pragma unroll
      for (int p = 0; p < 3; ++p)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[p][i][c] = kDwMagic;
      uint32_t cur[3][6], nxt[3][6];
#pragma unroll
      for (int P = 0; P < 3; ++P) {
        dw_load_raw<1>(xrow, cs, P < in_rows && static_cast<unsigned>(ih0 + P) < static_cast<unsigned>(a.h), colmask, cur[P]);
        xrow += row_step;
      }
      for (int iy = 0; iy < in_rows && tc_.ok; iy += 3) {
#pragma unroll
        for (int P = 0; P < 3; ++P) {
          const int ir = iy + 3 + P;
          dw_load_raw<1>(xrow, cs, ir < in_rows && static_cast<unsigned>(ih0 + ir) < static_cast<unsigned>(a.h), colmask, nxt[P]);
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
          if (oy >= 0 && oy < rows && tc_.ok) {
            emit_row(acc[(P + 1) % 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[(P + 1) % 3][i][c] = kDwMagic;
          }
        }
#pragma unroll
        for (int P = 0; P < 3; ++P)
#pragma unroll
          for (int ix = 0; ix < 6; ++ix) cur[P][ix] = nxt[P][ix];
      }
    } else {
      int acc[2][4][4];
#pragma unroll
      for (int p = 0; p < 2; ++p)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[p][i][c] = kDwMagic;
      uint32_t cur[2][9], nxt[2][9];
#pragma unroll
      for (int P = 0; P < 2; ++P) {
        dw_load_raw<2>(xrow, cs, P < in_rows && static_cast<unsigned>(ih0 + P) < static_cast<unsigned>(a.h), colmask, cur[P]);
        xrow += row_step;
      }
      for (int iy = 0; iy < in_rows && tc_.ok; iy += 4) {
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          const int ir = iy + 2 * P;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int in = ir + 2 + q;
            dw_load_raw<2>(xrow, cs, in < in_rows && static_cast<unsigned>(ih0 + in) < static_cast<unsigned>(a.h), colmask, nxt[q]);
            xrow += row_step;
          }
          dw_make_win<2>(cur[0], win);
          dw_mac(acc[P], win, wr[0]);
          dw_mac(acc[P ^ 1], win, wr[2]);
          const int oy = (ir >> 1) - 1;
          if (oy >= 0 && oy < rows && tc_.ok) {
            emit_row(acc[P ^ 1]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[P ^ 1][i][c] = kDwMagic;
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
    // a last tile with fewer than TH rows, and tiles of the item past the image's last row
    while (tc_.ok && tc_.tiles_done < T) finish_tile();
    if (!tc_.ok) return;
    // (TW = 4) T * TH rows are an even count, so the swizzle phase of offs[] is back where it started
    if (row_toggle && ((rows & 1) != 0)) {
#pragma unroll
      for (int ox = 0; ox < 4; ++ox) offs[ox] ^= row_toggle;
    }
  }
}

// ------------------------------------------------------------------------------------------------ the kernel
template <int S, int CS, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
    dwpw_fused_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmOut, const DwpwArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem_al = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  // [epilogue staging][resident 1x1 filter][operand ring][barriers]
  uint8_t* b_smem = smem_al + kStagingBytes;
  uint8_t* ring_smem = b_smem + a.b_bytes;
  uint8_t* ctrl = ring_smem + a.stages * a.stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;
  uint64_t* acc_empty = acc_full + kMaxAccBufs;
  uint64_t* b_bar = acc_empty + kMaxAccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_cols = static_cast<uint32_t>(a.acc_cols * a.acc_bufs);
  // items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const int nb = (a.total_items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int total_tiles = nb * a.tiles_per_item;

  if (warp == kMmaWarp) {
    for (int i = lane; i < 2 * kMaxStages + 2 * kMaxAccBufs + 1; i += 32) {
      uint32_t count = 1;
      if (i < kMaxStages) count = static_cast<uint32_t>(a.warps_per_group);                           // full: one arrival per depthwise warp
      else if (i >= 2 * kMaxStages + kMaxAccBufs && i < 2 * kMaxStages + 2 * kMaxAccBufs) count = kEpiWarps;  // accumulator drained
      mbar_init(smem_u32(&full_bar[i]), count);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 0) *abort_flag = 0;
    if (lane < 2)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(lane == 0 ? &tmB : &tmOut)) : "memory");
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync_with_previous_kernel();

  if (warp < kDwWarps) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kDwRegs));
    depthwise_role<S, CS>(a, smem_u32(ring_smem), full_bar, empty_bar, abort_flag, warp, lane, nb);
  } else if (warp >= kMmaWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kMmaRegs));
    if (warp == kMmaWarp) {
    // ---------------------------------------------------------------------------------------------- MMA issue
    const bool leader = elect_one();
    // the 1x1 filter, once: [K chunk][cout rows][kc bytes], swizzled by the copy
    mbar_expect_tx_if(smem_u32(b_bar), static_cast<uint32_t>(a.b_bytes), leader);
    for (int kch = 0; kch < a.kchunks; ++kch)
      for (int n0 = 0; n0 < a.cout; n0 += 256)
        tma_load_2d_if(smem_u32(b_smem) + static_cast<uint32_t>((kch * a.cout + n0) * a.kc), &tmB, smem_u32(b_bar), kch * a.kc,
                       n0, leader);
    bool ok = mbar_wait(smem_u32(b_bar), 0, abort_flag, a.status, FAULT_WAIT_FULL);
    const uint32_t hi = static_cast<uint32_t>(make_smem_desc(0, a.kc) >> 32);
    const uint32_t ring_lo = ((smem_u32(ring_smem) >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t b_lo0 = ((smem_u32(b_smem) >> 4) & 0x3FFFu) | (1u << 16);
    const int mma_per_chunk = a.kc / 32;
    const int nchunk = a.cout < 256 ? a.cout : 256;
    // D = s32, A = B = s8, both K-major, M = 128, N = nchunk
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(nchunk >> 3) << 17) |
                           (static_cast<uint32_t>(128 >> 4) << 24);
    int stage = 0, buf = 0;
    uint32_t full_parity = 0, acc_parity = 1;
    for (int q = 0; q < total_tiles && ok; ++q) {
      ok = mbar_wait(smem_u32(&acc_empty[buf]), acc_parity, abort_flag, a.status, FAULT_WAIT_ACCUM);
      if (!ok) break;
      ok = mbar_wait(smem_u32(&full_bar[stage]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_lo = ring_lo + static_cast<uint32_t>((stage * a.stage_bytes) >> 4);
      for (int n0 = 0; n0 < a.cout; n0 += 256) {
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * a.acc_cols + n0);
        for (int kch = 0; kch < a.kchunks; ++kch) {
          const uint32_t a_k = a_lo + static_cast<uint32_t>((kch * 128 * a.kc) >> 4);
          const uint32_t b_k = b_lo0 + static_cast<uint32_t>(((kch * a.cout + n0) * a.kc) >> 4);
          for (int j = 0; j < mma_per_chunk; ++j)
            tc_mma_i8_halves(d_tmem, a_k + 2u * j, hi, b_k + 2u * j, hi, idesc, (kch | j) ? 1u : 0u, leader);
        }
      }
      tc_commit_if(smem_u32(&empty_bar[stage]), leader);
      tc_commit_if(smem_u32(&acc_full[buf]), leader);
      if (++stage == a.stages) {
        stage = 0;
        full_parity ^= 1;
      }
      if (++buf == a.acc_bufs) {
        buf = 0;
        acc_parity ^= 1;
      }
    }
    if (!ok || *abort_flag) mbar_wait_drain(smem_u32(b_bar), 0);
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kEpiRegs));
    // ---------------------------------------------------------------------------------------------- epilogue
    const int quad = warp - kEpiWarp0;
    const int wq = a.cout < 128 ? a.cout : 128;  // bytes of a staged pixel row
    const uint32_t st0 = smem_u32(smem_al) + static_cast<uint32_t>(quad * 8192);
    const int b_swz = wq == 128 ? (lane & 7) : (wq == 64 ? ((lane >> 1) & 3) : ((lane >> 2) & 1));
    const float ub = quant_upper_bound<ACT>(a.alpha);
    const int rows_per_warp = 32 / a.tw;  // tile rows of this warp's 32 pixels
    const int G = a.groups, T = a.tiles_per_item;
    int rd = 0, ti = 0, g = 0, Gk = min(G, nb);
    int buf = 0, sbuf = 0;
    uint32_t acc_parity = 0;
    bool ok = true;
    for (int q = 0; q < total_tiles && ok; ++q) {
      const int item = static_cast<int>(blockIdx.x) + (rd * G + g) * static_cast<int>(gridDim.x);
      const int seg = item % a.segs;
      const int t = item / a.segs;
      const int cb = t % a.col_blocks;
      const int n = t / a.col_blocks;
      const int x0 = cb * a.tw;
      const int y0 = seg * a.seg_rows + ti * a.th + quad * rows_per_warp;
      const bool active = y0 < a.ho;  // warp-uniform; rows and columns past the image are clipped by the store
      ok = mbar_wait(smem_u32(&acc_full[buf]), acc_parity, abort_flag, a.status, FAULT_WAIT_ACCUM);
      if (!ok) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + static_cast<uint32_t>(buf * a.acc_cols) + (static_cast<uint32_t>(quad * 32) << 16);
      for (int cgrp = 0; active && cgrp < a.cout; cgrp += 128) {
        const uint32_t st = st0 + static_cast<uint32_t>(sbuf * 4096);
        // the store issued two groups ago read this buffer: it must have finished reading
        if (lane == 0) bulk_wait_read_1();
        __syncwarp();
        const uint32_t row = st + static_cast<uint32_t>(lane * wq);
        for (int c = cgrp; c < cgrp + wq; c += 32) {
          uint32_t r[32];
          tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
          tc_wait_ld();
          const float4* sc4 = reinterpret_cast<const float4*>(a.scale + c);
          const float4* bi4 = reinterpret_cast<const float4*>(a.bias + c);
          const int chunk0 = (c - cgrp) >> 4;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t v[4];
            if (a.acc_small) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                v[j] = quant4<ACT, true>(&r[16 * h + 4 * j], __ldg(sc4 + 4 * h + j), __ldg(bi4 + 4 * h + j), a.alpha, ub);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                v[j] = quant4<ACT, false>(&r[16 * h + 4 * j], __ldg(sc4 + 4 * h + j), __ldg(bi4 + 4 * h + j), a.alpha, ub);
            }
            sts128(row + (((chunk0 + h) ^ b_swz) << 4), v[0], v[1], v[2], v[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(&tmOut, st, cgrp, x0, y0, n);
          bulk_commit();
        }
        sbuf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
      if (++buf == a.acc_bufs) {
        buf = 0;
        acc_parity ^= 1;
      }
      if (++g == Gk) {
        g = 0;
        if (++ti == T) {
          ti = 0;
          ++rd;
          Gk = min(G, nb - rd * G);
        }
      }
    }
    if (lane == 0) bulk_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

typedef void (*DwpwKernel)(const CUtensorMap, const CUtensorMap, const DwpwArgs);

template <int S, int CS>
DwpwKernel pick_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return dwpw_fused_kernel<S, CS, PLB_ACT_RELU>;
    case PLB_ACT_RELU6: return dwpw_fused_kernel<S, CS, PLB_ACT_RELU6>;
    case PLB_ACT_LEAKY: return dwpw_fused_kernel<S, CS, PLB_ACT_LEAKY>;
    default: return dwpw_fused_kernel<S, CS, PLB_ACT_NONE>;
  }
}
template <int S>
DwpwKernel pick_pitch(int c, int act) {
  switch (c) {
    case 32: return pick_act<S, 32>(act);
    case 64: return pick_act<S, 64>(act);
    case 128: return pick_act<S, 128>(act);
    default: return pick_act<S, 256>(act);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_tiled = nullptr;
std::mutex g_mutex;

int load_encoder() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_tiled) return PLB_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled unavailable");
  g_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  return PLB_OK;
}

CUtensorMapSwizzle swizzle_for(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

struct Tiling {
  int tw, th, seg_rows, segs, col_blocks, groups, warps_per_group, total_items, grid, stages;
};

// Estimated cost of a tiling, in warp instructions on the busiest SM (both roles share the SM's issue slots).
double tiling_cost(const DwpwProblem& p, const Tiling& t) {
  const int nb_max = (t.total_items + t.grid - 1) / t.grid;
  const int rounds = (nb_max + t.groups - 1) / t.groups;
  const int T = t.seg_rows / t.th;
  const double in_rows = (std::min(t.seg_rows, p.ho) - 1) * p.stride + 3;
  // a depthwise thread: ~ 40 instructions per input row (load, transpose, shift) + ~ 170 per output row (dp4a, requantiser, store)
  const double per_item_thread = in_rows * (p.stride == 1 ? 40.0 : 60.0) + std::min(t.seg_rows, p.ho) * 170.0;
  const double dw_total = nb_max * per_item_thread * t.warps_per_group;
  const double epi_total = static_cast<double>(nb_max) * T * 128.0 * p.cout * 4.5 / 32.0;
  // a round cannot finish before its slowest group: a lone warp issues at most about every other cycle
  const double critical = rounds * per_item_thread * 2.0;
  return std::max((dw_total + epi_total) / 4.0 / 0.8, critical);
}

size_t fixed_smem(const DwpwProblem& p) {
  return kStagingBytes + static_cast<size_t>(p.cout) * p.c + kCtrlBytes + 1024;  // 1024: alignment slack
}

int plan_tiling(const plb_ctx* ctx, const DwpwProblem& p, Tiling* out) {
  const int tws[3] = {16, 8, 4};
  const int max_stages = std::min<int>(kMaxStages, static_cast<int>((227 * 1024 - fixed_smem(p)) / (128 * p.c)));
  double best = 0;
  bool have = false;
  for (int tw : tws) {
    if (p.tw > 0 && p.tw != tw) continue;
    const int units = p.c * tw / 16;  // threads per strip
    if (units < 32 || units % 32 || units > 32 * kDwWarps) continue;
    if (tw == 4 && p.c < 128) continue;
    Tiling t;
    t.tw = tw;
    t.th = 128 / tw;
    t.warps_per_group = units / 32;
    t.groups = kDwWarps / t.warps_per_group;
    if (t.groups > max_stages) continue;  // every group fills a stage of its own
    t.stages = std::min(max_stages, 3 * t.groups);
    t.col_blocks = (p.wo + tw - 1) / tw;
    const int max_t = (p.ho + t.th - 1) / t.th;
    for (int tiles = 1; tiles <= max_t; ++tiles) {
      t.seg_rows = tiles * t.th;
      if (p.seg_rows > 0 && t.seg_rows != std::min((p.seg_rows + t.th - 1) / t.th, max_t) * t.th) continue;
      t.segs = (p.ho + t.seg_rows - 1) / t.seg_rows;
      // skip segmentations whose last segment wastes a whole tile or more
      if (p.seg_rows <= 0 && t.segs * t.seg_rows - p.ho >= t.th && tiles > 1) continue;
      const long items = static_cast<long>(p.batch) * t.col_blocks * t.segs;
      if (items > 0x3fffffff) continue;
      t.total_items = static_cast<int>(items);
      t.grid = static_cast<int>(std::min<long>(items, ctx->sm_count));
      const double cost = tiling_cost(p, t);
      if (!have || cost < best) {
        best = cost;
        *out = t;
        have = true;
      }
    }
  }
  if (!have) return fail(PLB_E_UNSUPPORTED, "no tiling for %d channels", p.c);
  return PLB_OK;
}

}  // namespace

bool dwpw_fused_supported(const plb_ctx* ctx, const DwpwProblem& p, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  (void)ctx;
  if (p.c != 32 && p.c != 64 && p.c != 128 && p.c != 256) return no("channels must be 32, 64, 128 or 256");
  if (p.stride != 1 && p.stride != 2) return no("stride must be 1 or 2");
  if (p.cout != 32 && p.cout != 64 && p.cout != 128 && p.cout != 256 && p.cout != 512) return no("output channels must be 32 .. 512, a power of two");
  if (p.dw_epi.act != PLB_ACT_NONE && p.dw_epi.act != PLB_ACT_RELU && p.dw_epi.act != PLB_ACT_RELU6)
    return no("depthwise activation must be none, relu or relu6");
  if (p.ldy % 16 != 0 || (reinterpret_cast<uintptr_t>(p.y) & 15)) return no("output rows must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(p.x) & 3) || (reinterpret_cast<uintptr_t>(p.wpw) & 15)) return no("input alignment");
  if (p.pad_t < 0 || p.pad_l < 0 || p.ho < 1 || p.wo < 1) return no("geometry");
  if (fixed_smem(p) + 2 * 128 * static_cast<size_t>(p.c) > 227 * 1024) return no("1x1 filter too large to stay in shared memory");
  return true;
}

int dwpw_fused_launch(plb_ctx* ctx, const DwpwProblem& p) {
  std::string why;
  if (!dwpw_fused_supported(ctx, p, &why)) return fail(PLB_E_UNSUPPORTED, "fused depthwise + 1x1: %s", why.c_str());
  int rc = load_encoder();
  if (rc) return rc;
  Tiling t;
  if ((rc = plan_tiling(ctx, p, &t))) return rc;

  DwpwArgs a;
  memset(&a, 0, sizeof(a));
  a.x = p.x; a.wdw = p.wdw; a.cg_pad = p.cg_pad;
  a.dw_scale = p.dw_epi.scale; a.dw_bias = p.dw_epi.bias;
  a.dw_lo = p.dw_epi.act == PLB_ACT_NONE ? -127.f : 0.f;
  a.dw_ub = p.dw_epi.act == PLB_ACT_RELU6 ? std::max(std::min(p.dw_epi.alpha, 127.f), -127.f) : 127.f;
  a.h = p.h; a.w = p.w; a.c = p.c; a.ho = p.ho; a.wo = p.wo; a.pad_t = p.pad_t; a.pad_l = p.pad_l;
  a.tw = t.tw; a.th = t.th; a.col_blocks = t.col_blocks; a.seg_rows = t.seg_rows; a.segs = t.segs;
  a.tiles_per_item = t.seg_rows / t.th; a.total_items = t.total_items;
  a.groups = t.groups; a.warps_per_group = t.warps_per_group;
  a.kc = p.c < 128 ? p.c : 128;
  a.kchunks = p.c / a.kc;
  a.stage_bytes = 128 * p.c;
  a.cout = p.cout;
  a.acc_cols = std::max(32, p.cout);
  a.acc_bufs = std::min(4, 512 / a.acc_cols);
  a.b_bytes = p.cout * p.c;
  a.scale = p.pw_epi.scale; a.bias = p.pw_epi.bias; a.alpha = p.pw_epi.alpha; a.acc_small = p.pw_epi.acc_small;
  a.status = ctx->d_status;
  a.stages = t.stages;
  const size_t smem = fixed_smem(p) + static_cast<size_t>(t.stages) * a.stage_bytes;

  CUtensorMap tmB, tmOut;
  {
    // 1x1 filter [cout][c]: boxes of kc bytes x up to 256 rows
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.c), static_cast<cuuint64_t>(p.cout)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.c)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(std::min(p.cout, 256))};
    const cuuint32_t es[2] = {1, 1};
    CUresult r = g_tiled(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.wpw), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(a.kc), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "tensor map of the 1x1 filter: error %d", static_cast<int>(r));
  }
  {
    // output [batch][ho][wo][cout] with pixel pitch ldy: boxes of 128 channels x TW columns x (32 / TW) rows
    const int wq = std::min(p.cout, 128);
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(p.cout), static_cast<cuuint64_t>(p.wo), static_cast<cuuint64_t>(p.ho),
                                static_cast<cuuint64_t>(p.batch)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(p.ldy), static_cast<cuuint64_t>(p.ldy) * p.wo,
                                   static_cast<cuuint64_t>(p.ldy) * p.wo * p.ho};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(wq), static_cast<cuuint32_t>(t.tw), static_cast<cuuint32_t>(32 / t.tw), 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = g_tiled(&tmOut, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, p.y, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle_for(wq), CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "tensor map of the output: error %d", static_cast<int>(r));
  }
  DwpwKernel kernel = p.stride == 1 ? pick_pitch<1>(p.c, p.pw_epi.act) : pick_pitch<2>(p.c, p.pw_epi.act);
  {
    // once per (kernel, device)
    static std::mutex attr_mutex;
    static std::vector<std::pair<const void*, int>> configured;
    std::lock_guard<std::mutex> lock(attr_mutex);
    const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), ctx->device);
    bool found = false;
    for (auto& k : configured) found = found || k == key;
    if (!found) {
      PLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      configured.push_back(key);
    }
  }
  PLB_CUDA(launch_kernel(kernel, dim3(t.grid), dim3(kThreads), smem, ctx->stream, tmB, tmOut, a));
  ++ctx->launches;
  ++ctx->dwpw_launches;
  return PLB_OK;
}

}  // namespace plb
