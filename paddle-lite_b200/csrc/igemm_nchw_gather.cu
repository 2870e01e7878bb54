// 1x1 convolution on NCHW tensors whose images TMA cannot address (pixel counts that are not a multiple of 16: 14 x 14,
// 7 x 7, 10 x 10, ...), without any re-pitching pass.  Same orientation and arithmetic as igemm_nchw.cu (M = output channels,
// N = pixels, B = X[n] = [cin][hw] as an MN-major operand, exact int32 accumulators, the same requantiser); what differs
// is how the pixels get in and out:
//   * 8 gather warps copy X rows into the 128-byte-swizzled MN-major operand tile that TMA would have written: with
//     4-byte asynchronous copies (cp.async, several stages in flight) where the rows are a multiple of 4 bytes long,
//     otherwise with aligned 4-byte loads that are funnel-shifted into place in registers; a tile's columns are the pixels of G whole images, each padded
//     to P = hw rounded up to 16 columns (G = 256 / P), or 256-pixel runs of one larger image;
//   * the epilogue warps requantise 32 columns at a time into a small staging tile and write it out row by row, so that
//     the lanes of a warp store consecutive pixels of ONE output row.
// The filter still arrives through TMA (it is padded to whole 32-byte rows at prepare time).
// Replaces the same reference code as igemm_nchw.cu (lite/kernels/x86/conv_compute.cc:335-337 per image;
// lite/kernels/arm/sparse_conv_compute.cc:155-267 for the densified sparse_conv2d).
// Roles: warps 0-15 epilogue (4 groups x 4 TMEM lane quadrants), warps 16-23 gather, warp 24 filter TMA, warp 25 MMA issue
// (warps 26-27 idle: registers are handed out four warps at a time and re-balanced with setmaxnreg).  All waits bounded.
#include <algorithm>
#include <mutex>

#include "igemm_nchw.cuh"
#include "tc_device.cuh"

namespace plb {
namespace {

using namespace tc;

constexpr int kTileCout = 128;
constexpr int kEpilogueWarps = 16;
constexpr int kGatherWarps = 8;
constexpr int kGatherWarp0 = kEpilogueWarps;
constexpr int kProducerWarp = kEpilogueWarps + kGatherWarps;
constexpr int kMmaWarp = kProducerWarp + 1;
constexpr int kThreads = 32 * (kEpilogueWarps + kGatherWarps + 4);
constexpr int kEpiRegs = 80, kGatherRegs = 64, kCtrlRegs = 56;  // of the 72 per thread the CTA starts with
constexpr int kMaxStages = 8;
constexpr int kCtrlBytes = 1024;
constexpr int kStagePitch = 80;                                  // bytes between rows of an epilogue staging tile (64 + 16)
constexpr int kStagingBytes = kEpilogueWarps * 32 * kStagePitch;
constexpr int kMaxResidentW = 64 * 1024;
constexpr int kInFlight = 4;                                     // stages of copies a gather lane keeps pending
constexpr int kMaxIter = 2;                                      // 4-byte words of a 256-pixel row per gather lane: 64 / 32

struct GatherArgs {
  const int8_t* x;
  void* y;
  int batch, cin, cout, hw;
  int group_images;       // G: images per tile (1 when an image has more than 256 pixels)
  int image_cols;         // P: columns an image occupies in a tile (hw rounded up to 16), or the tile width when G == 1 and hw > 256
  int bn;                 // columns of a tile (multiple of 16, <= 256)
  int acc_stride;         // tensor-memory columns between the two accumulator buffers (power of two >= bn)
  int kc, ksteps, stages;
  int tiles_m, tiles_p, num_tiles;
  int resident_w, resident_bytes;
  int bres;               // pixel tiles stay in shared memory for ALL channel tiles: a CTA gathers a pixel tile once, then
                          // runs the channel tiles over it with the filter streamed through its own ring (wstages)
  int wstages, num_ptiles;
  int dup;
  int bytewise;           // hw % 4 != 0: image rows start at any byte; they are fetched as aligned words and funnel-shifted
  const float* scale;
  const float* bias;
  float alpha;
  int acc_small;
  int* status;
};

// 4-byte asynchronous copy global -> shared; `take` false: the word is written as zero and nothing is read
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool take) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(take ? 4 : 0) : "memory");
}
// waits until at most n (0 .. 4) of this thread's committed copy groups are pending
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Tile t: channel tile fastest, so CTAs running side by side gather the same pixels from L2.
// img = first image of the tile, p0 = first pixel (0 when a tile holds whole images).
__device__ __forceinline__ void decode_tile(const GatherArgs& a, int t, int& m0, int& p0, int& img) {
  const int m = t % a.tiles_m;
  const int r = t / a.tiles_m;
  const int pt = r % a.tiles_p;
  img = (r / a.tiles_p) * a.group_images;
  m0 = m * kTileCout;
  p0 = pt * a.bn;
}

// The j-th (channel tile, pixel tile) of this CTA; false past the end.  Streaming order: tiles blockIdx.x, + gridDim.x, ...
// with the channel tile fastest across CTAs.  Pixel-resident order (bres): pixel tiles blockIdx.x, + gridDim.x, ..., and
// for each of them every channel tile in turn.
__device__ __forceinline__ bool cta_tile(const GatherArgs& a, int j, int& m0, int& p0, int& img) {
  if (!a.bres) {
    const long t = static_cast<long>(blockIdx.x) + static_cast<long>(j) * gridDim.x;
    if (t >= a.num_tiles) return false;
    decode_tile(a, static_cast<int>(t), m0, p0, img);
    return true;
  }
  const int ptl = j / a.tiles_m;
  const long pt = static_cast<long>(blockIdx.x) + static_cast<long>(ptl) * gridDim.x;
  if (pt >= a.num_ptiles) return false;
  m0 = (j - ptl * a.tiles_m) * kTileCout;
  p0 = static_cast<int>(pt % a.tiles_p) * a.bn;
  img = static_cast<int>(pt / a.tiles_p) * a.group_images;
  return true;
}

template <int MODE, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
    igemm_nchw_gather_kernel(const __grid_constant__ CUtensorMap tmW, const GatherArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem_al = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  // [epilogue staging][resident filter][operand ring: per stage filter tile (unless resident) + pixel tile][barriers]
  const int halves = (a.bn + 127) >> 7;
  const int stage_a = (a.resident_w || a.bres) ? 0 : kTileCout * a.kc;
  const int stage_b = a.kc * 128 * halves;
  const int stage_bytes = stage_a + stage_b;
  uint8_t* smem_wres = smem_al + ((kStagingBytes + 1023) & ~1023);
  uint8_t* smem = smem_wres + a.resident_bytes;
  uint8_t* wring = smem + a.stages * stage_bytes;  // bres: ring of filter tiles
  uint8_t* ctrl = wring + a.wstages * kTileCout * a.kc;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint64_t* wres_bar = acc_empty + 2;
  uint64_t* wfull = wres_bar + 1;        // [kMaxStages] bres: filter ring
  uint64_t* wempty = wfull + kMaxStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wempty + kMaxStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_cols = 2u * static_cast<uint32_t>(a.acc_stride);

  if (warp == kProducerWarp) {
    constexpr int kBarriers = 4 * kMaxStages + 4 + 1;
    for (int i = lane; i < kBarriers; i += 32) {
      uint32_t count = 1;
      if (i < kMaxStages) count = kGatherWarps + ((a.resident_w || a.bres) ? 0 : 1);  // gather warps (+ the filter copy's arrival)
      else if (i >= 2 * kMaxStages + 2 && i < 2 * kMaxStages + 4) count = 8;  // two epilogue groups of four warps drain a buffer
      mbar_init(smem_u32(&full_bar[i]), count);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 0) {
      *abort_flag = 0;
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmW)) : "memory");
    }
    __syncwarp();
    if (a.resident_w && lane == 0) {
      // the filter is a layer constant: its copy does not wait for the preceding kernel
      const uint32_t bar = smem_u32(wres_bar);
      mbar_expect_tx(bar, static_cast<uint32_t>(a.ksteps * kTileCout * a.kc));
      const int m0 = (static_cast<int>(blockIdx.x) % a.tiles_m) * kTileCout;
      for (int ks = 0; ks < a.ksteps; ++ks) {
        tma_load_2d(smem_u32(smem_wres) + ks * kTileCout * a.kc, &tmW, bar, ks * a.kc, m0);
        if (a.dup) tma_load_2d(smem_u32(smem_wres) + ks * kTileCout * a.kc + 64 * a.kc, &tmW, bar, ks * a.kc, m0);
      }
    }
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync_with_previous_kernel();

  if (warp >= kProducerWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kCtrlRegs));
    if (warp == kProducerWarp && a.bres) {
      // ------------------------------------------------------------ filter tiles through TMA, a ring of their own
      const bool leader = elect_one();
      int ws = 0;
      uint32_t wparity = 1;
      bool ok = true;
      const uint32_t wbase = smem_u32(wring);
      const uint32_t wbytes = static_cast<uint32_t>(kTileCout * a.kc);
      int m0, p0, img;
      for (int j = 0; ok && cta_tile(a, j, m0, p0, img); ++j) {
        for (int ks = 0; ks < a.ksteps; ++ks) {
          ok = mbar_wait(smem_u32(&wempty[ws]), wparity, abort_flag, a.status, FAULT_WAIT_EMPTY);
          if (!ok) break;
          const uint32_t bar = smem_u32(&wfull[ws]);
          const uint32_t dst = wbase + ws * wbytes;
          mbar_expect_tx_if(bar, wbytes, leader);
          tma_load_2d_if(dst, &tmW, bar, ks * a.kc, m0, leader);
          if (a.dup) tma_load_2d_if(dst + 64 * a.kc, &tmW, bar, ks * a.kc, m0, leader);
          if (++ws == a.wstages) {
            ws = 0;
            wparity ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        for (int jj = 0; jj < a.wstages; ++jj) mbar_wait_drain(smem_u32(&wfull[jj]), jj < ws ? (wparity ^ 1u) : wparity);
      }
    } else if (warp == kProducerWarp && !a.resident_w) {
      // ------------------------------------------------------------ filter tiles through TMA
      const bool leader = elect_one();
      int s = 0;
      uint32_t empty_parity = 1;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      int m0, p0, img;
      for (int j = 0; ok && cta_tile(a, j, m0, p0, img); ++j) {
        for (int ks = 0; ks < a.ksteps; ++ks) {
          ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_base + s * stage_bytes;
          mbar_expect_tx_if(bar, static_cast<uint32_t>(stage_a), leader);
          tma_load_2d_if(dst, &tmW, bar, ks * a.kc, m0, leader);
          if (a.dup) tma_load_2d_if(dst + 64 * a.kc, &tmW, bar, ks * a.kc, m0, leader);
          if (++s == a.stages) {
            s = 0;
            empty_parity ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        // bounded wait for this warp's copies in flight
        for (int j = 0; j < a.stages; ++j) mbar_wait_drain(smem_u32(&full_bar[j]), j < s ? (empty_parity ^ 1u) : empty_parity);
      }
    } else if (warp == kProducerWarp) {
      if (*abort_flag) mbar_wait_drain(smem_u32(wres_bar), 0);
    } else if (warp == kMmaWarp) {
      // ------------------------------------------------------------ MMA issuer
      const bool leader = elect_one();
      // D = s32, A = B = s8, A K-major, B MN-major (bit 16), N = bn, M = 128
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(a.bn >> 3) << 17) |
                             (static_cast<uint32_t>(kTileCout >> 4) << 24);
      const int mma_per_stage = a.kc / 32;
      const uint32_t hi_a = static_cast<uint32_t>(make_smem_desc(0, a.kc) >> 32);
      // MN-major, 128-byte swizzle: groups of 8 K-rows are 1024 bytes apart; the next 128 columns kc * 128 bytes further
      const uint32_t hi_b = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t lbo_b = ((static_cast<uint32_t>(a.kc * 128) >> 4) & 0x3FFFu) << 16;
      const uint32_t ring_lo = (smem_u32(smem) >> 4) & 0x3FFFu;
      const uint32_t wres_lo = (smem_u32(smem_wres) >> 4) & 0x3FFFu;
      const uint32_t stage_lo = static_cast<uint32_t>(stage_bytes) >> 4;
      const uint32_t stage_a_lo = static_cast<uint32_t>(stage_a) >> 4;
      const uint32_t wstep_lo = static_cast<uint32_t>(kTileCout * a.kc) >> 4;
      int s = 0, it = 0;
      uint32_t full_parity = 0;
      bool ok = true;
      if (a.resident_w) {
        ok = mbar_wait(smem_u32(wres_bar), 0, abort_flag, a.status, FAULT_WAIT_FULL);
        tc_fence_after();
      }
      const uint32_t wring_lo = (smem_u32(wring) >> 4) & 0x3FFFu;
      int ws = 0;
      uint32_t wparity = 0;
      int m0, p0, img;
      for (; ok && cta_tile(a, it, m0, p0, img); ++it) {
        const int buf = it & 1;
        ok = mbar_wait(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * a.acc_stride;
        // pixel-resident order: the chunks of a pixel tile are waited for in its first channel-tile pass and given back
        // in its last one (stages == ksteps there, so s == ks and the parity follows the pixel tile)
        const int mt = a.bres ? it % a.tiles_m : 0;
        const bool first_pass = !a.bres || mt == 0, last_pass = !a.bres || mt == a.tiles_m - 1;
        for (int ks = 0; ks < a.ksteps; ++ks) {
          if (first_pass) {
            ok = mbar_wait(smem_u32(&full_bar[s]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
            if (!ok) break;
          }
          if (a.bres) {
            ok = mbar_wait(smem_u32(&wfull[ws]), wparity, abort_flag, a.status, FAULT_WAIT_FULL);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t st_lo = ring_lo + s * stage_lo;
          const uint32_t a_lo = (a.bres ? wring_lo + ws * wstep_lo : (a.resident_w ? wres_lo + ks * wstep_lo : st_lo)) | (1u << 16);
          const uint32_t b_lo = (st_lo + stage_a_lo) | lbo_b;
          for (int j = 0; j < mma_per_stage; ++j)  // 32 bytes of K: +32 B inside A's swizzle span, +32 rows (4 KiB) of B
            tc_mma_i8_halves(d_tmem, a_lo + 2u * j, hi_a, b_lo + 256u * j, hi_b, idesc, (ks | j) ? 1u : 0u, leader);
          if (a.bres) {
            tc_commit_if(smem_u32(&wempty[ws]), leader);
            if (++ws == a.wstages) {
              ws = 0;
              wparity ^= 1;
            }
          }
          if (last_pass) tc_commit_if(smem_u32(&empty_bar[s]), leader);
          if (++s == a.stages) {
            s = 0;
            if (last_pass) full_parity ^= 1;
          }
        }
        if (!ok) break;
        tc_commit_if(smem_u32(&acc_full[buf]), leader);
      }
    }
  } else if (warp >= kGatherWarp0) {
    // -------------------------------------------------------------- gather: X rows -> MN-major operand tile
    // Asynchronous 4-byte copies (cp.async, zero-filled where a word lies outside the image or the channels): a lane
    // issues the 32 words of its rows of a stage without holding them in registers and goes on to the next stage, so
    // several stages of loads are in flight per SM; a stage is handed to the MMA warp when the copies of the stage
    // issued kInFlight stages later have been committed and this one's have landed.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kGatherRegs));
    const int gw = warp - kGatherWarp0;  // rows gw, gw + 8, ...: (row & 7) == gw, the swizzle phase of all of them
    const int words = a.bn >> 2;         // 4-byte words of a tile row
    const long plane = static_cast<long>(a.cin) * a.hw;
    const int in_flight = a.stages - 1 < kInFlight ? a.stages - 1 : kInFlight;  // stages a lane keeps pending
    int s = 0, s_done = 0, pending = 0;
    uint32_t empty_parity = 1;
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    // hand over the oldest pending stage: its copies (and all older ones) have landed
    auto retire = [&]() {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&full_bar[s_done]));
      if (++s_done == a.stages) s_done = 0;
      --pending;
    };
    int m0, p0, img;
    for (int j = 0; ok && cta_tile(a, j, m0, p0, img); j += a.bres ? a.tiles_m : 1) {
      // this lane's words of a row: where they come from (image, pixel) and where they go (block of 128 columns, swizzled chunk)
      long goff[kMaxIter];
      uint32_t soff[kMaxIter];
      bool valid[kMaxIter], used[kMaxIter];
      int nbytes[kMaxIter];     // bytewise: bytes of the word that lie inside the image (0 .. 4)
      bool next_has[kMaxIter];  // bytewise: the next lane holds the following word of the same image row
#pragma unroll
      for (int it = 0; it < kMaxIter; ++it) {
        const int w = lane + 32 * it;
        const int col = 4 * w;
        int g = 0, p = p0 + col;
        if (a.group_images > 1 || a.tiles_p == 1) {
          g = col / a.image_cols;
          p = col - g * a.image_cols;
        }
        used[it] = w < words;
        valid[it] = used[it] && p < a.hw && img + g < a.batch;  // hw % 4 == 0: a word is inside the image or outside
        nbytes[it] = valid[it] ? (a.hw - p < 4 ? a.hw - p : 4) : 0;
        next_has[it] = lane < 31 && p + 4 < a.hw && (p + 4 < a.image_cols || !(a.group_images > 1 || a.tiles_p == 1));
        goff[it] = valid[it] ? static_cast<long>(img + g) * plane + p : 0;
        const int colb = col & 127;
        soff[it] = static_cast<uint32_t>((col >> 7) * (a.kc * 128) + (((colb >> 4) ^ gw) << 4) + (colb & 15));
      }
      for (int ks = 0; ks < a.ksteps; ++ks) {
        if (!mbar_try_wait(smem_u32(&empty_bar[s]), empty_parity)) {
          // About to block on the MMA warp: everything issued so far has to be handed over first.  In the pixel-resident
          // order a chunk is given back only after the LAST channel-tile pass over ALL chunks of its pixel tile, which
          // cannot start before the chunks still pending here have arrived.
          asm volatile("cp.async.wait_all;" ::: "memory");
          while (pending > 0) retire();
          ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
          if (!ok) break;
        }
        const uint32_t dst = smem_base + s * stage_bytes + stage_a;
        if (a.bytewise) {
          // Rows at any byte alignment: a lane loads the aligned word that holds the first byte of its word, takes the
          // following aligned word from the next lane (or loads it itself where the next lane holds something else), and
          // funnel-shifts.  No aligned word is read that does not contain a byte of the image.  Four rows per batch.
          for (int c0 = gw; c0 < a.kc; c0 += 32) {
            uint32_t lo[4][kMaxIter], hi[4][kMaxIter];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int cc = c0 + 8 * r;
              const int ch = ks * a.kc + cc;
              const bool row_ok = ch < a.cin;
              const int8_t* src = a.x + static_cast<long>(row_ok ? ch : 0) * a.hw;
#pragma unroll
              for (int it = 0; it < kMaxIter; ++it) {
                const uintptr_t addr = reinterpret_cast<uintptr_t>(src + goff[it]);
                const uint32_t shift = static_cast<uint32_t>(addr & 3u);
                const uint32_t* wp = reinterpret_cast<const uint32_t*>(addr & ~static_cast<uintptr_t>(3));
                const bool take = row_ok && nbytes[it] > 0;
                lo[r][it] = take ? __ldg(wp) : 0u;
                const bool need_hi = take && shift + static_cast<uint32_t>(nbytes[it]) > 4u;
                hi[r][it] = (need_hi && !next_has[it]) ? __ldg(wp + 1) : 0u;
              }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int cc = c0 + 8 * r;
              const int ch = ks * a.kc + cc;
              const int8_t* src = a.x + static_cast<long>(ch < a.cin ? ch : 0) * a.hw;
#pragma unroll
              for (int it = 0; it < kMaxIter; ++it) {
                const uint32_t from_next = __shfl_down_sync(0xffffffffu, lo[r][it], 1);
                const uint32_t shift = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src + goff[it]) & 3u);
                const uint32_t h = next_has[it] ? from_next : hi[r][it];
                const uint32_t val = __funnelshift_r(lo[r][it], h, shift * 8u);
                if (cc < a.kc && used[it]) sts32(dst + static_cast<uint32_t>(cc * 128) + soff[it], val);
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&full_bar[s]));
          if (++s_done == a.stages) s_done = 0;
          if (++s == a.stages) {
            s = 0;
            empty_parity ^= 1;
          }
          continue;
        }
        for (int cc = gw; cc < a.kc; cc += 8) {
          const int ch = ks * a.kc + cc;
          const bool row_ok = ch < a.cin;
          const int8_t* src = a.x + static_cast<long>(row_ok ? ch : 0) * a.hw;
#pragma unroll
          for (int it = 0; it < kMaxIter; ++it)
            if (used[it]) cp_async4(dst + static_cast<uint32_t>(cc * 128) + soff[it], src + goff[it], row_ok && valid[it]);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        ++pending;
        if (++s == a.stages) {
          s = 0;
          empty_parity ^= 1;
        }
        if (pending > in_flight) {
          cp_async_wait_pending(in_flight);
          retire();
        }
      }
    }
    // the copies still in flight land (bounded by the memory system, not by another role), then their stages are handed over
    asm volatile("cp.async.wait_all;" ::: "memory");
    while (pending > 0) retire();
  } else {
    // -------------------------------------------------------------- epilogue: 4 groups x 4 warps
    // Groups 0/1 take the CTA's even tiles (buffer 0), groups 2/3 the odd ones; the two groups of a tile take alternate
    // chunks of 32 columns.  Warp w reads tensor-memory lanes 32*(w%4) .. +31 = 32 output channels; with duplicated
    // accumulator rows (cout <= 64) quadrants 2 and 3 repeat the channels of 0 and 1 and take every other chunk of theirs.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpiRegs));
    const int group = warp >> 2, quad = warp & 3;
    const int buf = group >> 1, col_par = group & 1;
    const int row_quad = a.dup ? (quad & 1) : quad;
    const int chunk0 = col_par + (a.dup ? 2 * (quad >> 1) : 0);
    const int chunk_step = a.dup ? 4 : 2;
    const uint32_t st = smem_u32(smem_al) + static_cast<uint32_t>(warp * 32 * kStagePitch);
    const float ub = quant_upper_bound<ACT>(a.alpha);
    const bool grouped = a.group_images > 1 || a.tiles_p == 1;
    bool ok = true;
    for (int it = buf; ok; it += 2) {
      int m0, p0, img;
      if (!cta_tile(a, it, m0, p0, img)) break;
      const int row0 = m0 + row_quad * 32;
      const bool active = row0 < a.cout;  // warp-uniform
      const int ch = row0 + lane;
      float sc = 0.f, bi = 0.f;
      if (MODE != OUT_ACC && ch < a.cout) {
        sc = __ldg(a.scale + ch);
        bi = __ldg(a.bias + ch);
      }
      const float4 sc4 = make_float4(sc, sc, sc, sc), bi4 = make_float4(bi, bi, bi, bi);
      ok = mbar_wait(smem_u32(&acc_full[buf]), (it >> 1) & 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
      tc_fence_after();
      if (!ok) break;
      const uint32_t lane_addr = tmem_base + buf * a.acc_stride + (static_cast<uint32_t>(quad * 32) << 16);
      for (int c = chunk0 * 32; active && c < a.bn; c += chunk_step * 32) {
        if (!grouped && p0 + c >= a.hw) break;  // warp-uniform: pixels past the image
        uint32_t r[32];
        tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
        tc_wait_ld();
        const uint32_t row = st + static_cast<uint32_t>(lane * kStagePitch);
        if (MODE == OUT_I8) {
          uint32_t q[8];
          if (a.acc_small) {
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = quant4<ACT, true>(&r[4 * j], sc4, bi4, a.alpha, ub);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = quant4<ACT, false>(&r[4 * j], sc4, bi4, a.alpha, ub);
          }
          __syncwarp();  // the previous chunk has been read out of the staging tile
          sts128(row, q[0], q[1], q[2], q[3]);
          sts128(row + 16, q[4], q[5], q[6], q[7]);
          __syncwarp();
          // 8 passes of 4 rows x 8 words: the lanes of a quarter warp store 32 consecutive pixels of one output row
          const int j = lane & 7;
          const int col = c + 4 * j;
          int g = 0, p = p0 + col;
          if (grouped) {
            g = col / a.image_cols;
            p = col - g * a.image_cols;
          }
          int nv = a.hw - p;
          nv = nv < 0 ? 0 : (nv > 4 ? 4 : nv);
          if (col >= a.bn || img + g >= a.batch) nv = 0;
          int8_t* ybase = static_cast<int8_t*>(a.y) + (static_cast<long>(img + g) * a.cout) * a.hw + p;
#pragma unroll
          for (int pass = 0; pass < 8; ++pass) {
            const int rr = pass * 4 + (lane >> 3);
            const uint32_t word = lds32(st + static_cast<uint32_t>(rr * kStagePitch + 4 * j));
            const int co = row0 + rr;
            if (co < a.cout && nv > 0) {
              int8_t* dstp = ybase + static_cast<long>(co) * a.hw;
              if (!a.bytewise) {
                *reinterpret_cast<uint32_t*>(dstp) = word;  // hw % 4 == 0: whole words, 4-byte aligned
              } else {
#pragma unroll
                for (int b = 0; b < 4; ++b)
                  if (b < nv) dstp[b] = static_cast<int8_t>(word >> (8 * b));
              }
            }
          }
        } else {
          // fp32 / int32: 16 columns (64 bytes per row) at a time through the staging tile
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t v[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int acc = static_cast<int>(r[16 * hh + e]);
              v[e] = MODE == OUT_ACC ? static_cast<uint32_t>(acc)
                                     : __float_as_uint(act_f32<ACT>(fmaf(__int2float_rn(acc), sc, bi), a.alpha));
            }
            __syncwarp();
#pragma unroll
            for (int e = 0; e < 4; ++e) sts128(row + 16 * e, v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
            __syncwarp();
            const int j = lane & 15;
            const int col = c + 16 * hh + j;
            int g = 0, p = p0 + col;
            if (grouped) {
              g = col / a.image_cols;
              p = col - g * a.image_cols;
            }
            const bool col_ok = col < a.bn && p < a.hw && img + g < a.batch;
            uint32_t* ybase = static_cast<uint32_t*>(a.y) + (static_cast<long>(img + g) * a.cout) * a.hw + p;
#pragma unroll
            for (int pass = 0; pass < 16; ++pass) {
              const int rr = pass * 2 + (lane >> 4);
              const uint32_t word = lds32(st + static_cast<uint32_t>(rr * kStagePitch + 4 * j));
              const int co = row0 + rr;
              if (co < a.cout && col_ok) ybase[static_cast<long>(co) * a.hw] = word;
            }
          }
        }
      }
      // this warp no longer reads the buffer: let the MMA warp overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

typedef void (*GatherKernel)(const CUtensorMap, const GatherArgs);

template <int MODE>
GatherKernel pick_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return igemm_nchw_gather_kernel<MODE, PLB_ACT_RELU>;
    case PLB_ACT_RELU6: return igemm_nchw_gather_kernel<MODE, PLB_ACT_RELU6>;
    case PLB_ACT_LEAKY: return igemm_nchw_gather_kernel<MODE, PLB_ACT_LEAKY>;
    default: return igemm_nchw_gather_kernel<MODE, PLB_ACT_NONE>;
  }
}
GatherKernel pick_kernel(int mode, int act) {
  if (mode == OUT_I8) return pick_act<OUT_I8>(act);
  if (mode == OUT_F32) return pick_act<OUT_F32>(act);
  return igemm_nchw_gather_kernel<OUT_ACC, PLB_ACT_NONE>;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mutex;

int load_encoder() {
  if (g_encode) return PLB_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr)
    return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return PLB_OK;
}

}  // namespace

namespace {

struct GatherPlan {
  GatherArgs a;
  long grid;
  size_t smem;
};

// Tile shapes, tile order and shared-memory layout of a problem; false (with the reason) when the kernel cannot take it.
bool plan_gather(const plb_ctx* ctx, const NchwProblem& p, GatherPlan* plan, std::string* why) {
  auto no = [&](const char* msg) {
    if (why) *why = msg;
    return false;
  };
  if (p.out_mode != OUT_I8 && p.out_mode != OUT_F32 && p.out_mode != OUT_ACC) return no("output mode");
  if (p.x_pitch || p.y_pitch) return no("dense NCHW tensors only");
  if (p.cin_pad % 32 != 0 || p.cin > p.cin_pad) return no("filter rows must be padded to a multiple of 32 bytes");
  if (p.batch <= 0 || p.cout <= 0 || p.cin <= 0 || p.hw <= 0) return no("empty problem");
  if (reinterpret_cast<uintptr_t>(p.w) & 15) return no("the filter must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(p.x) & 3) || (reinterpret_cast<uintptr_t>(p.y) & 3)) return no("tensors must be 4-byte aligned");
  if (static_cast<long>(p.batch) * p.cin * p.hw > 0x7fffffffL * 16) return no("tensor too large");
  GatherArgs& a = plan->a;
  memset(&a, 0, sizeof(a));
  a.x = p.x; a.y = p.y;
  a.batch = p.batch; a.cin = p.cin; a.cout = p.cout; a.hw = p.hw;
  a.kc = p.cin_pad % 128 == 0 ? 128 : (p.cin_pad % 64 == 0 ? 64 : 32);
  a.ksteps = p.cin_pad / a.kc;
  a.tiles_m = (p.cout + kTileCout - 1) / kTileCout;
  a.dup = p.cout <= 64;
  a.bytewise = p.hw % 4 != 0;
  const int staging = (kStagingBytes + 1023) & ~1023;
  const int budget = 225 * 1024 - staging - kCtrlBytes;
  const int wtile = kTileCout * a.kc;
  // Pixel-resident order (a pixel tile is gathered once and all channel tiles run over it) needs every K chunk of the
  // pixel tile plus a ring of at least three filter tiles in shared memory; it pays as soon as there are two channel tiles.
  auto bres_fits = [&](int bn) { return a.ksteps <= kMaxStages && a.ksteps * a.kc * 128 * ((bn + 127) / 128) + 3 * wtile <= budget; };
  const bool want_bres = a.tiles_m >= 2 && p.bres_switch != 0;
  long groups;
  bool bres = false;
  if (p.hw <= 256) {
    // whole images per tile, each padded to a multiple of 16 columns
    a.image_cols = (p.hw + 15) / 16 * 16;
    a.group_images = 256 / a.image_cols;
    // prefer a tile that fits the pixel-resident order (long K: 128 columns instead of 256)
    if (want_bres && !bres_fits(a.group_images * a.image_cols) && a.image_cols <= 128 && bres_fits(128))
      a.group_images = 128 / a.image_cols;
    bres = want_bres && bres_fits(a.group_images * a.image_cols);
    // small grids: fewer images per tile so that every SM gets a tile (a pixel tile in the pixel-resident order), as
    // long as a tile keeps at least 128 columns
    auto work_items = [&](int g) {
      const long pt = (p.batch + g - 1) / g;
      return bres ? pt : pt * a.tiles_m;
    };
    while (a.group_images > 1 && work_items(a.group_images) < ctx->sm_count &&
           ((a.group_images / 2) * a.image_cols >= 128 || work_items(a.group_images) < ctx->sm_count / 2))
      a.group_images /= 2;
    a.bn = a.group_images * a.image_cols;
    a.tiles_p = 1;
    groups = (p.batch + a.group_images - 1) / a.group_images;
  } else {
    a.group_images = 1;
    a.bn = (want_bres && !bres_fits(256) && bres_fits(128)) ? 128 : 256;
    a.image_cols = a.bn;
    a.tiles_p = (p.hw + a.bn - 1) / a.bn;
    groups = p.batch;
    bres = want_bres && bres_fits(a.bn);
  }
  a.acc_stride = 32;
  while (a.acc_stride < a.bn) a.acc_stride <<= 1;
  const long ptiles = groups * a.tiles_p;
  const long tiles = ptiles * a.tiles_m;
  if (tiles > 0x7fffffffL) return no("too many tiles");
  a.num_tiles = static_cast<int>(tiles);
  a.num_ptiles = static_cast<int>(ptiles);
  const int halves = (a.bn + 127) / 128;
  const int stage_b = a.kc * 128 * halves;
  a.bres = bres && (p.bres_switch == 1 || ptiles >= ctx->sm_count / 2);
  // Where this kernel is the better choice (measured, batch 256): in the pixel-resident order (512 -> 512 on 14 x 14:
  // 40 us against 48 re-pitched; 1024 -> 1024 on 7 x 7: 49 against 58 staged); gathered per channel tile only with
  // 4-byte outputs and 4-byte-aligned rows (66 against 152).  An explicit switch (tests) overrides.
  if (p.bres_switch != 0 && p.bres_switch != 1 && !a.bres && (a.bytewise || p.out_mode == OUT_I8))
    return no("not the better path for this shape");
  int stage_bytes;
  if (a.bres) {
    plan->grid = ptiles < ctx->sm_count ? ptiles : ctx->sm_count;
    a.resident_w = 0;
    a.resident_bytes = 0;
    stage_bytes = stage_b;
    a.stages = a.ksteps;
    a.wstages = std::min(kMaxStages, (budget - a.ksteps * stage_b) / wtile);
  } else {
    const int resident_bytes = a.ksteps * wtile;
    plan->grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    a.resident_w = plan->grid % a.tiles_m == 0 && resident_bytes <= kMaxResidentW && tiles > plan->grid;
    a.resident_bytes = a.resident_w ? resident_bytes : 0;
    stage_bytes = (a.resident_w ? 0 : wtile) + stage_b;
    int stages = (budget - a.resident_bytes) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return no("the operand ring does not fit");
    a.stages = stages;
    a.wstages = 0;
  }
  plan->smem = static_cast<size_t>(staging) + a.resident_bytes + static_cast<size_t>(a.stages) * stage_bytes +
               static_cast<size_t>(a.wstages) * wtile + kCtrlBytes + 1024;
  return true;
}

}  // namespace

bool igemm_nchw_gather_supported(const plb_ctx* ctx, const NchwProblem& p, std::string* why) {
  GatherPlan plan;
  return plan_gather(ctx, p, &plan, why);
}

int igemm_nchw_gather_launch(plb_ctx* ctx, const NchwProblem& p) {
  std::string why;
  GatherPlan plan;
  if (!plan_gather(ctx, p, &plan, &why)) return fail(PLB_E_UNSUPPORTED, "NCHW gather path: %s", why.c_str());
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc = load_encoder();
    if (rc) return rc;
  }
  GatherArgs& a = plan.a;
  const long grid_l = plan.grid;
  const size_t smem = plan.smem;
  a.scale = p.epi.scale; a.bias = p.epi.bias; a.alpha = p.epi.alpha; a.acc_small = p.epi.acc_small;
  a.status = ctx->d_status;

  alignas(64) CUtensorMap tmW;
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.cout)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.cin_pad)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(a.dup ? 64 : kTileCout)};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = a.kc == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                              : (a.kc == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = g_encode(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.w), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(filter) failed: %d", (int)r);
  }
  GatherKernel kernel = pick_kernel(p.out_mode, p.epi.act);
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    static std::vector<std::pair<const void*, int>> configured;
    const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), ctx->device);
    bool found = false;
    for (auto& k : configured) found = found || k == key;
    if (!found) {
      PLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      configured.push_back(key);
    }
  }
  const unsigned grid = static_cast<unsigned>(grid_l);
  PLB_CUDA(launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, ctx->stream, tmW, a));
  ctx->launches++;
  ctx->nchw_launches++;
  ctx->nchw_gather_launches++;
  return PLB_OK;
}

}  // namespace plb
