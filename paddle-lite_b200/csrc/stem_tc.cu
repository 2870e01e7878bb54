// First layer of a network (RGB stem: 7x7 or 3x3, stride 2, 3 input channels) in ONE launch, from the fp32 NCHW image
// to the int8 channels-last output.  The reference runs calib (fp32 -> int8, lite/backends/x86/math/calib.cc:25-151)
// and then im2col + GEMM (lite/kernels/x86/conv_compute.cc:292-341); here the calib, the im2col and the GEMM operand
// never reach memory: producer warps quantise the image rows a work item needs into shared memory (pixels x channels
// interleaved, zero padding in place), copy for every output pixel the 32-byte windows of the row-folded layout
// ([filter row pair j][row e of the pair][kw taps x 3 channels, padded to 32 bytes, or to 16 where a filter row has at
// most 16 bytes and a pixel 4 windows: 3x3 on RGB]) into the swizzled K-major operand
// tile, tcgen05.mma multiplies by the resident folded filter, and 12 epilogue warps requantise and store through TMA.
// Same arithmetic as the staged path (fold_rows + implicit GEMM), bit for bit: exact int32 sums of the same products.
//
// A work item is R output rows of one image with R * wo a multiple of 128 (8 rows of 112 pixels = 7 tiles), so tiles are
// runs of 128 consecutive output pixels; a CTA takes items blockIdx.x, blockIdx.x + gridDim.x, ...
// Roles: warps 0-7 calib team (image rows -> one of two quantised row buffers, one item ahead), warps 8-15 tile team
// (row buffer -> operand tiles), warps 16-27 epilogue (3 groups x 4 TMEM lane quadrants, group g takes every 3rd tile),
// warp 28 MMA issue (with three idle companions: registers are handed out to warps four at a time).  The teams hand
// row buffers to each other through mbarriers; all waits are bounded (tc::mbar_wait).
#include "stem_tc.cuh"

#include <algorithm>
#include <mutex>

#include "igemm_tc.cuh"
#include "tc_device.cuh"

namespace plb {
namespace {

using namespace tc;

constexpr int kCalibWarps = 8;                  // fp32 image rows -> quantised row buffers
constexpr int kTileWarps = 8;                   // row buffers -> operand tiles
constexpr int kTileThreads = 32 * kTileWarps;
constexpr int kProdWarps = kCalibWarps + kTileWarps;
constexpr int kEpiGroups = 3;
constexpr int kEpiWarps = 4 * kEpiGroups;
constexpr int kMmaWarp = kProdWarps + kEpiWarps;
constexpr int kThreads = 32 * (kMmaWarp + 4);
// Registers per thread and role, of the 64 the CTA starts with (setmaxnreg: a role's warpgroups give registers back or
// take more).  The MMA warp's loop is the pace maker of every tile: with 24 registers it spilled four of them.
constexpr int kCalibRegs = 56, kTileRegs = 72, kEpiRegs = 64, kMmaRegs = 56;
static_assert(32 * (kCalibWarps * kCalibRegs + kTileWarps * kTileRegs + kEpiWarps * kEpiRegs + 4 * kMmaRegs) <= 64 * kThreads,
              "the roles together may not ask for more registers than the CTA was launched with: an increase would wait forever");
constexpr int kMaxStages = 8;
constexpr int kMaxAccBufs = 8;
constexpr int kCtrlBytes = 1024;
constexpr int kStagingPerWarp = 2 * 2048;  // two buffers of 32 pixels x up to 64 channels

struct StemArgs {
  const float* x;
  int cin, h, w, ho, wo;
  int stride_h, stride_w, pad_t;
  int rows_in;        // image rows a work item needs
  int row_words;      // words per quantised row buffer
  int px0_word;       // word of pixel 0 in a row buffer (the left padding lies in front of it)
  int base_off;       // byte of output column 0's window in a row buffer
  int nwin;           // 32-byte windows per output pixel = fold_kh * fold_h
  int fold_h;
  int rows_item;      // output rows per work item (R)
  int tiles_item;     // R * wo / 128
  int items_per_image, total_items;
  int kchunks;        // K / row_bytes
  int row_bytes;      // bytes of K per operand-tile row: 128 (32-byte windows) or 64 (16-byte windows, 4 per pixel)
  int stages, stage_bytes;
  int cout, acc_cols, acc_bufs, b_bytes;
  float inv_scale;
  float scale[64], bias[64];  // requantiser tables: kernel arguments, read as constant-bank operands (compile-time columns)
  float alpha;
  int acc_small;
  int* status;
};

__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// All warps of a role's warpgroups: change the registers per thread from the launch value (64) to R.
template <int R>
__device__ __forceinline__ void role_registers() {
  if (R > 64) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
  if (R < 64) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// calib of the reference: sat(rne(max(x / scale, -127))); rounding by adding 1.5 * 2^23, result in the low byte.
// Two values per multiply and per add (f32x2 forms, IEEE per lane: the same bits as the scalar sequence).
__device__ __forceinline__ float clamp127(float v) { return fminf(fmaxf(v, -127.f), 127.f); }
__device__ __forceinline__ void calib_bits2(float x, float y, float2 inv2, uint32_t& bx, uint32_t& by) {
  const float2 p = __fmul2_rn(make_float2(x, y), inv2);
  const float2 r = __fadd2_rn(make_float2(clamp127(p.x), clamp127(p.y)), make_float2(12582912.f, 12582912.f));
  bx = __float_as_uint(r.x);
  by = __float_as_uint(r.y);
}

template <int ACT, int NWIN, int WB>
__global__ void __launch_bounds__(kThreads, 1)
    stem_tc_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmOut, const StemArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem_al = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  // [epilogue staging][resident filter][operand ring][quantised image rows][barriers]
  uint8_t* b_smem = smem_al + kEpiWarps * kStagingPerWarp;
  uint8_t* ring_smem = b_smem + a.b_bytes;
  uint32_t* rowbuf = reinterpret_cast<uint32_t*>(ring_smem + a.stages * a.stage_bytes);
  const int rowbuf_words = (a.rows_in * a.row_words + 255) & ~255;  // per buffer; there are two
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(rowbuf + 2 * rowbuf_words);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;
  uint64_t* acc_empty = acc_full + kMaxAccBufs;
  uint64_t* b_bar = acc_empty + kMaxAccBufs;
  uint64_t* rows_full = b_bar + 1;   // [2] a row buffer holds the quantised rows of an item
  uint64_t* rows_empty = rows_full + 2;  // [2] its tiles are built
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(rows_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_cols = static_cast<uint32_t>(a.acc_cols * a.acc_bufs);
  const int nb = (a.total_items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int total_tiles = nb * a.tiles_item;

  if (warp == kMmaWarp) {
    for (int i = lane; i < 2 * kMaxStages + 2 * kMaxAccBufs + 5; i += 32) {
      uint32_t count = 1;
      if (i < kMaxStages) count = kTileWarps;                                                           // full: one arrival per tile warp
      else if (i > 2 * kMaxStages + 2 * kMaxAccBufs) count = i <= 2 * kMaxStages + 2 * kMaxAccBufs + 2 ? kCalibWarps : kTileWarps;
      else if (i >= 2 * kMaxStages + kMaxAccBufs && i < 2 * kMaxStages + 2 * kMaxAccBufs) count = 4;  // drained by one epilogue group
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
  if (warp < kProdWarps) {
    // the padding bytes of the row buffers stay zero for the whole kernel; image bytes are rewritten per item
    for (int i = threadIdx.x; i < 2 * rowbuf_words; i += 32 * kProdWarps) rowbuf[i] = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync_with_previous_kernel();

  if (warp < kCalibWarps) {
    // ---------------------------------------------------------------------------------------------- calib team
    // fp32 image rows of item k -> [pixel][channel] bytes in row buffer k & 1, one item ahead of the tile team.
    role_registers<kCalibRegs>();
    const int tid = threadIdx.x;
    const int w4 = a.w >> 2;
    const long plane = static_cast<long>(a.h) * a.w;
    const int total_units = a.rows_in * w4;
    const int unit_r0 = tid / w4, unit_t0 = tid - unit_r0 * w4;
    const int unit_dr = (32 * kCalibWarps) / w4, unit_dt = 32 * kCalibWarps - unit_dr * w4;
    const float2 inv2 = make_float2(a.inv_scale, a.inv_scale);
    for (int k = 0; k < nb; ++k) {
      const int item = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
      const int n = item / a.items_per_image;
      const int ih0 = (item - n * a.items_per_image) * a.rows_item * a.stride_h - a.pad_t;
      const float* img = a.x + static_cast<long>(n) * a.cin * plane;
      const int b = k & 1;
      if (!mbar_wait(smem_u32(&rows_empty[b]), ((k >> 1) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_EMPTY)) break;
      const uint32_t rb0 = smem_u32(rowbuf + b * rowbuf_words);
      // a unit is 4 pixels of the three channels = 3 words; a thread takes units tid, tid + 256, ...
      // (row r and position t of a unit advance by the quotient and remainder of the step: no division per unit)
      int r = unit_r0, t = unit_t0;
      for (int u = tid; u < total_units; u += 32 * kCalibWarps) {
        const int ih = ih0 + r;
        uint32_t w0 = 0, w1 = 0, w2 = 0;
        if (ih >= 0 && ih < a.h) {
          const float4* src = reinterpret_cast<const float4*>(img + static_cast<long>(ih) * a.w) + t;
          const float4 c0 = __ldg(src), c1 = __ldg(src + (plane >> 2)), c2 = __ldg(src + 2 * (plane >> 2));
          uint32_t b[12];  // pixel-major: (c0, c1, c2) of pixel 0, then pixel 1, ...
          calib_bits2(c0.x, c1.x, inv2, b[0], b[1]);
          calib_bits2(c2.x, c0.y, inv2, b[2], b[3]);
          calib_bits2(c1.y, c2.y, inv2, b[4], b[5]);
          calib_bits2(c0.z, c1.z, inv2, b[6], b[7]);
          calib_bits2(c2.z, c0.w, inv2, b[8], b[9]);
          calib_bits2(c1.w, c2.w, inv2, b[10], b[11]);
          w0 = pack_low_bytes(b[0], b[1], b[2], b[3]);
          w1 = pack_low_bytes(b[4], b[5], b[6], b[7]);
          w2 = pack_low_bytes(b[8], b[9], b[10], b[11]);
        }
        const uint32_t d = rb0 + static_cast<uint32_t>((r * a.row_words + a.px0_word) * 4 + t * 12);
        sts32(d, w0);
        sts32(d + 4, w1);
        sts32(d + 8, w2);
        r += unit_dr;
        t += unit_dt;
        if (t >= w4) {
          t -= w4;
          ++r;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&rows_full[b]));
      // the rows of the item after the next one: into L2 while this team waits for a free buffer
      if (k + 2 < nb) {
        const int item2 = item + 2 * static_cast<int>(gridDim.x);
        const int n2 = item2 / a.items_per_image;
        const int ih02 = (item2 - n2 * a.items_per_image) * a.rows_item * a.stride_h - a.pad_t;
        const float* img2 = a.x + static_cast<long>(n2) * a.cin * plane;
        const int lpr = (a.w + 31) >> 5;  // 128-byte lines per image row
        for (int l = tid; l < a.rows_in * 3 * lpr; l += 32 * kCalibWarps) {
          const int rc = l / lpr, off = l - rc * lpr;
          const int r = rc / 3, ch = rc - r * 3;
          const int ih = ih02 + r;
          if (ih >= 0 && ih < a.h)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(img2 + ch * plane + static_cast<long>(ih) * a.w + off * 32));
        }
      }
    }
  } else if (warp < kProdWarps) {
    // ---------------------------------------------------------------------------------------------- tile team
    // For every output pixel the NWIN windows of WB (32 or 16) bytes, word-unaligned in the row buffers, into the
    // operand tile.  16-byte windows (a filter row of at most 16 bytes, 4 windows per pixel) make rows of 64 bytes with
    // the 64-byte swizzle: half the stores, loads and MMAs of the 32-byte form.
    role_registers<kTileRegs>();
    const int tid = threadIdx.x - 32 * kCalibWarps;
    const uint32_t ring = smem_u32(ring_smem);
    constexpr int kUpt = 128 * NWIN / kTileThreads;  // windows per thread and tile (2 or 4)
    constexpr int kPstep = kTileThreads / NWIN;      // pixels between a thread's consecutive windows
    // Lane -> (pixel, window).  With 8 windows per pixel a quarter warp takes windows 0-3 (or 4-7) of an even and an
    // odd pixel: its eight 16-byte stores then fall on eight different chunks of the swizzled 128-byte rows (the two
    // K chunks of one pixel, 16 KB apart, would meet in the same banks).
    const int pix0 = NWIN == 8 ? (tid >> 5) * 4 + ((lane >> 4) << 1) + ((lane >> 2) & 1) : tid / NWIN;
    const int wv = NWIN == 8 ? ((lane >> 3) & 1) * 4 + (lane & 3) : tid % NWIN;  // filter row pair j, row e of the pair
    const int wj = wv / a.fold_h, we = wv - wj * a.fold_h;
    const int kch = wv >> 2, sub = wv & 3;
    bool ok = true;
    int stage = 0;
    uint32_t empty_parity = 1;
    for (int k = 0; k < nb && ok; ++k) {
      const int b = k & 1;
      ok = mbar_wait(smem_u32(&rows_full[b]), (k >> 1) & 1, abort_flag, a.status, FAULT_WAIT_FULL);
      if (!ok) break;
      const uint32_t rb0 = smem_u32(rowbuf + b * rowbuf_words);
      int py = 0, q = pix0;  // output row (inside the item) and column of this thread's next window
      while (q >= a.wo) {
        q -= a.wo;
        ++py;
      }
      for (int t = 0; t < a.tiles_item && ok; ++t) {
        ok = mbar_wait(smem_u32(&empty_bar[stage]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
        if (!ok) break;
        const uint32_t tile = ring + static_cast<uint32_t>(stage * a.stage_bytes + kch * (128 * 128));
        constexpr int kWords = WB / 4;
        uint32_t v[kUpt][kWords + 1], shift[kUpt];
#pragma unroll
        for (int i = 0; i < kUpt; ++i) {
          const int rb = (py + wj) * a.fold_h + we;
          const int src = a.base_off + q * a.stride_w * 3;
          const uint32_t sa = rb0 + static_cast<uint32_t>((rb * a.row_words + (src >> 2)) * 4);
          shift[i] = static_cast<uint32_t>(src & 3) * 8;
#pragma unroll
          for (int j = 0; j <= kWords; ++j) v[i][j] = lds32(sa + 4 * j);
          q += kPstep;
          while (q >= a.wo) {
            q -= a.wo;
            ++py;
          }
        }
#pragma unroll
        for (int i = 0; i < kUpt; ++i) {
          const int m = pix0 + i * kPstep;
          uint32_t o[kWords];
#pragma unroll
          for (int j = 0; j < kWords; ++j) o[j] = __funnelshift_r(v[i][j], v[i][j + 1], shift[i]);
          if (WB == 32) {
            const uint32_t row = tile + static_cast<uint32_t>(m * 128);
            const int sw = m & 7;
            sts128(row + (((sub * 2) ^ sw) << 4), o[0], o[1], o[2], o[3]);
            sts128(row + (((sub * 2 + 1) ^ sw) << 4), o[kWords - 4], o[kWords - 3], o[kWords - 2], o[kWords - 1]);
          } else {
            // rows of 64 bytes, 64-byte swizzle: chunk j of row m lives at j ^ ((m >> 1) & 3); a quarter warp (an even
            // and an odd pixel x 4 windows) covers one 128-byte line
            const uint32_t row = tile + static_cast<uint32_t>(m * 64);
            sts128(row + ((wv ^ ((m >> 1) & 3)) << 4), o[0], o[1], o[2], o[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&full_bar[stage]));
        if (++stage == a.stages) {
          stage = 0;
          empty_parity ^= 1;
        }
      }
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(smem_u32(&rows_empty[b]));  // the calib team may overwrite this buffer
    }
  } else if (warp >= kMmaWarp) {
    role_registers<kMmaRegs>();
    if (warp == kMmaWarp) {
      // -------------------------------------------------------------------------------------------- MMA issue
      const bool leader = elect_one();
      mbar_expect_tx_if(smem_u32(b_bar), static_cast<uint32_t>(a.b_bytes), leader);
      for (int kc = 0; kc < a.kchunks; ++kc)
        tma_load_2d_if(smem_u32(b_smem) + static_cast<uint32_t>(kc * a.cout * a.row_bytes), &tmB, smem_u32(b_bar),
                       kc * a.row_bytes, 0, leader);
      bool ok = mbar_wait(smem_u32(b_bar), 0, abort_flag, a.status, FAULT_WAIT_FULL);
      const uint32_t hi = static_cast<uint32_t>(make_smem_desc(0, WB == 32 ? 128 : 64) >> 32);
      const uint32_t ring_lo = ((smem_u32(ring_smem) >> 4) & 0x3FFFu) | (1u << 16);
      const uint32_t b_lo0 = ((smem_u32(b_smem) >> 4) & 0x3FFFu) | (1u << 16);
      // D = s32, A = B = s8, both K-major, M = 128, N = cout
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a.cout >> 3) << 17) |
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
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * a.acc_cols);
        for (int kc = 0; kc < a.kchunks; ++kc) {
          const uint32_t a_k = a_lo + static_cast<uint32_t>((kc * 128 * a.row_bytes) >> 4);
          const uint32_t b_k = b_lo0 + static_cast<uint32_t>((kc * a.cout * a.row_bytes) >> 4);
#pragma unroll
          for (int j = 0; j < (WB == 32 ? 4 : 2); ++j) tc_mma_i8_halves(d_tmem, a_k + 2u * j, hi, b_k + 2u * j, hi, idesc, (kc | j) ? 1u : 0u, leader);
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
    // ---------------------------------------------------------------------------------------------- epilogue
    role_registers<kEpiRegs>();
    const int e = warp - kProdWarps;
    const int quad = e & 3, group = e >> 2;
    const int wq = a.cout;  // bytes of a staged pixel row (32 or 64)
    const uint32_t st0 = smem_u32(smem_al) + static_cast<uint32_t>(e * kStagingPerWarp);
    const int b_swz = wq == 64 ? ((lane >> 1) & 3) : ((lane >> 2) & 1);
    const float ub = quant_upper_bound<ACT>(a.alpha);
    int sbuf = 0;
    bool ok = true;
    // tile q of this CTA = tile t of its k-th item; the counters advance by one epilogue round (no divisions)
    int buf = group % a.acc_bufs, t = group, item = static_cast<int>(blockIdx.x);
    uint32_t parity = static_cast<uint32_t>(group / a.acc_bufs) & 1u;
    for (int q = group; q < total_tiles && ok; q += kEpiGroups, buf += kEpiGroups, t += kEpiGroups) {
      while (buf >= a.acc_bufs) {
        buf -= a.acc_bufs;
        parity ^= 1u;
      }
      while (t >= a.tiles_item) {
        t -= a.tiles_item;
        item += static_cast<int>(gridDim.x);
      }
      // an item is rows_item whole output rows of one image = tiles_item runs of 128 consecutive output pixels
      const int row0 = (item * a.tiles_item + t) * 128 + quad * 32;
      ok = mbar_wait(smem_u32(&acc_full[buf]), parity, abort_flag, a.status, FAULT_WAIT_ACCUM);
      if (!ok) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + static_cast<uint32_t>(buf * a.acc_cols) + (static_cast<uint32_t>(quad * 32) << 16);
      const uint32_t st = st0 + static_cast<uint32_t>(sbuf * 2048);
      if (lane == 0) bulk_wait_read_1();  // the store issued two tiles ago has finished reading this buffer
      __syncwarp();
      const uint32_t row = st + static_cast<uint32_t>(lane * wq);
      // scale / bias of a compile-time column are constant-bank operands: no loads in this loop
#define PLB_STEM_CHUNK(COL)                                                                                        \
  if (COL < a.cout) {                                                                                              \
    uint32_t r[32];                                                                                                \
    tc_ld32(lane_addr + COL, r);                                                                                   \
    tc_wait_ld();                                                                                                  \
    _Pragma("unroll") for (int h = 0; h < 2; ++h) {                                                                \
      uint32_t v[4];                                                                                               \
      _Pragma("unroll") for (int j = 0; j < 4; ++j) {                                                              \
        const int c0 = COL + 16 * h + 4 * j;                                                                       \
        const float4 sc = make_float4(a.scale[c0], a.scale[c0 + 1], a.scale[c0 + 2], a.scale[c0 + 3]);             \
        const float4 bi = make_float4(a.bias[c0], a.bias[c0 + 1], a.bias[c0 + 2], a.bias[c0 + 3]);                 \
        v[j] = a.acc_small ? quant4<ACT, true>(&r[16 * h + 4 * j], sc, bi, a.alpha, ub)                            \
                           : quant4<ACT, false>(&r[16 * h + 4 * j], sc, bi, a.alpha, ub);                          \
      }                                                                                                            \
      sts128(row + (((COL / 16 + h) ^ b_swz) << 4), v[0], v[1], v[2], v[3]);                                       \
    }                                                                                                              \
  }
      PLB_STEM_CHUNK(0)
      PLB_STEM_CHUNK(32)
#undef PLB_STEM_CHUNK
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));  // the accumulator is free before the store is issued
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmOut, st, 0, row0);
        bulk_commit();
      }
      sbuf ^= 1;
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

typedef void (*StemKernel)(const CUtensorMap, const CUtensorMap, const StemArgs);
template <int NWIN, int WB>
StemKernel pick_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return stem_tc_kernel<PLB_ACT_RELU, NWIN, WB>;
    case PLB_ACT_RELU6: return stem_tc_kernel<PLB_ACT_RELU6, NWIN, WB>;
    case PLB_ACT_LEAKY: return stem_tc_kernel<PLB_ACT_LEAKY, NWIN, WB>;
    default: return stem_tc_kernel<PLB_ACT_NONE, NWIN, WB>;
  }
}
StemKernel pick_kernel(int act, int nwin, int wb) {
  if (nwin == 8) return pick_act<8, 32>(act);
  return wb == 16 ? pick_act<4, 16>(act) : pick_act<4, 32>(act);
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

struct StemPlan {
  int rows_item, tiles_item, rows_in, row_words, px0_word, base_off, nwin, win_bytes, k_bytes, stages;
  size_t smem;
};

bool plan(const StemProblem& p, StemPlan* s, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (p.cin != 3) return no("3 input channels only");
  if (p.w % 4 != 0 || (reinterpret_cast<uintptr_t>(p.x) & 15)) return no("image rows must be 16-byte aligned");
  if (p.cout != 32 && p.cout != 64) return no("32 or 64 output channels only");
  if (p.epi.h_scale == nullptr || p.epi.h_bias == nullptr) return no("requantiser tables not available on the host");
  if (p.kw * p.cin > 32 || p.fold_h != p.stride_h || p.fold_h < 1) return no("filter row does not fit a 32-byte window");
  s->nwin = p.fold_kh * p.fold_h;
  if (s->nwin != 4 && s->nwin != 8) return no("4 or 8 windows per pixel only");
  // a filter row of at most 16 bytes (3x3 on RGB: 9) in 4 windows: 16-byte windows, K = 64, where the layer has that filter form
  s->win_bytes = (s->nwin == 4 && p.kw * p.cin <= 16 && p.wfold16 != nullptr && (reinterpret_cast<uintptr_t>(p.wfold16) & 15) == 0) ? 16 : 32;
  s->k_bytes = s->nwin * s->win_bytes;
  // output rows per item: the fewest whose pixels fill whole 128-pixel tiles
  int g = 128, b = p.wo;
  while (b) {
    const int t = g % b;
    g = b;
    b = t;
  }
  s->rows_item = 128 / g;
  if (s->rows_item > 16 || p.ho % s->rows_item != 0) return no("output rows do not group into whole 128-pixel tiles");
  s->tiles_item = s->rows_item * p.wo / 128;
  if (p.wo < 8) return no("image too narrow");
  s->rows_in = (s->rows_item - 1) * p.stride_h + s->nwin;
  const int pad_bytes = p.pad_l * p.cin;
  s->px0_word = (pad_bytes + 3) / 4;
  s->base_off = s->px0_word * 4 - pad_bytes;
  // bytes a row buffer must hold: the last window read (9 words from its first word) and the image itself
  const int last_src = s->base_off + (p.wo - 1) * p.stride_w * p.cin;
  const int need_words = std::max((last_src >> 2) + 9, s->px0_word + (p.w * p.cin + 3) / 4);
  s->row_words = need_words | 1;  // odd pitch: rows of one column fall into different banks
  if ((reinterpret_cast<uintptr_t>(p.wfold) & 15) || (reinterpret_cast<uintptr_t>(p.y) & 15)) return no("filter / output alignment");
  const size_t rowbuf_bytes = 2 * static_cast<size_t>((s->rows_in * s->row_words + 255) & ~255) * 4;
  const size_t fixed = static_cast<size_t>(kEpiWarps) * kStagingPerWarp + static_cast<size_t>(p.cout) * s->k_bytes + rowbuf_bytes + kCtrlBytes + 1024;
  const size_t stage_bytes = 128 * static_cast<size_t>(s->k_bytes);
  if (fixed + 2 * stage_bytes > 227 * 1024) return no("does not fit shared memory");
  s->stages = static_cast<int>(std::min<size_t>(kMaxStages, (227 * 1024 - fixed) / stage_bytes));
  s->smem = fixed + s->stages * stage_bytes;
  return true;
}

}  // namespace

bool stem_tc_supported(const plb_ctx* ctx, const StemProblem& p, std::string* why) {
  (void)ctx;
  StemPlan s;
  return plan(p, &s, why);
}

int stem_tc_launch(plb_ctx* ctx, const StemProblem& p) {
  StemPlan s;
  std::string why;
  if (!plan(p, &s, &why)) return fail(PLB_E_UNSUPPORTED, "one-launch stem: %s", why.c_str());
  int rc = load_encoder();
  if (rc) return rc;
  StemArgs a;
  memset(&a, 0, sizeof(a));
  a.x = p.x; a.cin = p.cin; a.h = p.h; a.w = p.w; a.ho = p.ho; a.wo = p.wo;
  a.stride_h = p.stride_h; a.stride_w = p.stride_w; a.pad_t = p.pad_t;
  a.rows_in = s.rows_in; a.row_words = s.row_words; a.px0_word = s.px0_word; a.base_off = s.base_off;
  a.nwin = s.nwin; a.fold_h = p.fold_h;
  a.rows_item = s.rows_item; a.tiles_item = s.tiles_item;
  a.items_per_image = p.ho / s.rows_item;
  const long items = static_cast<long>(p.batch) * a.items_per_image;
  if (items > 0x3fffffff || static_cast<long>(p.batch) * p.ho * p.wo > 0x7fffffffL) return fail(PLB_E_UNSUPPORTED, "batch too large");
  a.total_items = static_cast<int>(items);
  a.row_bytes = std::min(128, s.k_bytes);
  a.kchunks = s.k_bytes / a.row_bytes;
  a.stages = s.stages;
  a.stage_bytes = 128 * s.k_bytes;
  a.cout = p.cout;
  a.acc_cols = p.cout;
  a.acc_bufs = std::min(kMaxAccBufs, 512 / a.acc_cols);
  a.b_bytes = p.cout * s.k_bytes;
  a.inv_scale = 1.f / p.in_scale;
  memcpy(a.scale, p.epi.h_scale, sizeof(float) * p.cout);
  memcpy(a.bias, p.epi.h_bias, sizeof(float) * p.cout);
  a.alpha = p.epi.alpha; a.acc_small = p.epi.acc_small;
  a.status = ctx->d_status;

  CUtensorMap tmB, tmOut;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(s.k_bytes), static_cast<cuuint64_t>(p.cout)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(s.k_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(a.row_bytes), static_cast<cuuint32_t>(p.cout)};
    const cuuint32_t es[2] = {1, 1};
    const int8_t* wf = s.win_bytes == 16 ? p.wfold16 : p.wfold;
    CUresult r = g_tiled(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(wf), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, a.row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "tensor map of the folded filter: error %d", static_cast<int>(r));
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cout), static_cast<cuuint64_t>(p.batch) * p.ho * p.wo};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.cout)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(p.cout), 32};
    const cuuint32_t es[2] = {1, 1};
    CUresult r = g_tiled(&tmOut, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p.y, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         p.cout == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "tensor map of the output: error %d", static_cast<int>(r));
  }
  StemKernel kernel = pick_kernel(p.epi.act, s.nwin, s.win_bytes);
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
  const int grid = static_cast<int>(std::min<long>(items, ctx->sm_count));
  PLB_CUDA(launch_kernel(kernel, dim3(grid), dim3(kThreads), s.smem, ctx->stream, tmB, tmOut, a));
  ++ctx->launches;
  ++ctx->stem_launches;
  return PLB_OK;
}

}  // namespace plb
