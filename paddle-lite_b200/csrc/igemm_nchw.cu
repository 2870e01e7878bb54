// 1x1 convolution on NCHW tensors as the reference lays them out, on the sm_100a tensor cores,
// without any layout staging pass.
//
// The reference's 1x1 path feeds the NCHW input directly to its GEMM as the B matrix
// (lite/kernels/x86/conv_compute.cc:335-337: C[cout, hw] = W[cout, cin] * X[cin, hw] per image), and the
// ARM sparse_conv2d kernels walk the same [cin][hw] rows (lite/kernels/arm/sparse_conv_compute.cc:155-267,
// lite/backends/arm/math/sparse_conv_impl.cc:3688-3790).  This kernel keeps that orientation:
//   M (tensor-memory lanes)   = output channels, 128 per tile; A = filter rows [cout][cin], K-major
//   N (tensor-memory columns) = pixels of ONE image, 128 or 256 per tile; B = X[n] = [cin][hw] exactly as it
//                               lies in memory, i.e. an MN-major operand (pixels contiguous)
// so D[cout][pixel] rows are NCHW rows and leave through TMA stores.  TMA brings X tiles as boxes of
// {128 pixels, KC channels} with the 128-byte swizzle, which is the canonical MN-major layout of
// tcgen05.mma (8 K-rows x 128 bytes per swizzle atom, atoms along K 1024 bytes apart, the second 128 pixels
// of a 256-pixel tile KC*128 bytes further).  Per-channel scale and bias are per LANE here: one scalar pair
// per thread.  Accumulators are exact int32; the epilogue is the same fmaf / round-to-nearest-even / clamp
// sequence as in the channels-last kernel, hence bit-identical results.
//
// Used for: plb_conv_run (NCHW) of unpadded stride-1 1x1 layers, and through it the densified sparse_conv2d.
// Needs hw % 16 == 0 (TMA strides); other shapes keep the staged path.
#include "igemm_nchw.cuh"

#include <mutex>

#include "tc_device.cuh"

namespace plb {
namespace {

using namespace tc;

constexpr int kTileCout = 128;
constexpr int kEpilogueGroups = 4;
constexpr int kEpilogueWarps = 4 * kEpilogueGroups;
constexpr int kProducerWarp = kEpilogueWarps;
constexpr int kMmaWarp = kEpilogueWarps + 1;
constexpr int kThreads = 32 * (kEpilogueWarps + 2);
constexpr int kMaxStages = 8;
constexpr int kCtrlBytes = 1024;
constexpr int kStagingBytes = kEpilogueWarps * 4096;  // one 4 KiB staging tile per epilogue warp
constexpr int kMaxResidentW = 64 * 1024;

struct NchwArgs {
  int cout, hw;
  int bn;                 // pixels per tile: 128 or 256
  int kc, ksteps, stages;
  int tiles_m, tiles_p, num_tiles;  // channel tiles, pixel tiles per image, all tiles
  int resident_w;         // the filter rows of this CTA's channel tile stay in shared memory (every tile of a CTA has the
                          // same channel tile when the grid size is a multiple of the number of channel tiles)
  int resident_bytes;
  int dup;                // cout <= 64: filter rows 0..63 are loaded twice (accumulator lanes 64..127 repeat lanes 0..63)
                          // so that all four lane quadrants, i.e. all four schedulers of the SM, share the epilogue:
                          // quadrants 2 and 3 take the second half of a group's pixels
  const float* scale;
  const float* bias;
  float alpha;
  int acc_small;
  int* status;
};

// Tile t: channel tile fastest, so CTAs running side by side share the same pixels in L2.
__device__ __forceinline__ void decode_tile(const NchwArgs& a, int t, int& m0, int& p0, int& img) {
  const int m = t % a.tiles_m;
  const int r = t / a.tiles_m;
  const int pt = r % a.tiles_p;
  img = r / a.tiles_p;
  m0 = m * kTileCout;
  p0 = pt * a.bn;
}

template <int MODE, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
    igemm_nchw_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const __grid_constant__ CUtensorMap tmOut, const NchwArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem_al = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  // [epilogue staging][resident filter][operand ring: per stage filter tile (unless resident) + pixel tile][barriers]
  const int stage_a = a.resident_w ? 0 : kTileCout * a.kc;
  const int stage_b = a.kc * a.bn;
  const int stage_bytes = stage_a + stage_b;
  uint8_t* smem_wres = smem_al + kStagingBytes;
  uint8_t* smem = smem_wres + a.resident_bytes;
  uint8_t* ctrl = smem + a.stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint64_t* wres_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wres_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_cols = 2u * static_cast<uint32_t>(a.bn);  // two accumulator buffers

  if (warp == kProducerWarp) {
    constexpr int kBarriers = 2 * kMaxStages + 4 + 1;
    for (int i = lane; i < kBarriers; i += 32) {
      const bool drained = i >= 2 * kMaxStages + 2 && i < 2 * kMaxStages + 4;
      mbar_init(smem_u32(&full_bar[i]), drained ? 8 : 1);  // two epilogue groups of four warps drain a buffer
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 0) *abort_flag = 0;
    {
      const CUtensorMap* map = lane == 0 ? &tmW : lane == 1 ? &tmX : &tmOut;
      if (lane < 3) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
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
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync_with_previous_kernel();

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    const bool leader = elect_one();
    int s = 0;
    uint32_t empty_parity = 1;
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    const int halves = a.bn / 128;
    for (int tile = blockIdx.x; tile < a.num_tiles && ok; tile += gridDim.x) {
      int m0, p0, img;
      decode_tile(a, tile, m0, p0, img);
      for (int ks = 0; ks < a.ksteps; ++ks) {
        ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
        if (!ok) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t dst = smem_base + s * stage_bytes;
        mbar_expect_tx_if(bar, static_cast<uint32_t>(stage_bytes), leader);
        if (!a.resident_w) {
          tma_load_2d_if(dst, &tmW, bar, ks * a.kc, m0, leader);
          if (a.dup) tma_load_2d_if(dst + 64 * a.kc, &tmW, bar, ks * a.kc, m0, leader);
        }
        // X[img][ks*kc .. +kc)[p0 .. +bn): one box per 128 pixels; rows past cin and pixels past hw arrive as zeros
        for (int h = 0; h < halves; ++h)
          tma_load_3d_if(dst + stage_a + h * a.kc * 128, &tmX, bar, p0 + 128 * h, ks * a.kc, img, leader);
        if (++s == a.stages) {
          s = 0;
          empty_parity ^= 1;
        }
      }
    }
    if (!ok || *abort_flag) {
      // a role of this CTA gave up: bounded wait for this warp's copies in flight (see igemm_tc.cu)
      for (int j = 0; j < a.stages; ++j)
        mbar_wait_drain(smem_u32(&full_bar[j]), j < s ? (empty_parity ^ 1u) : empty_parity);
      if (a.resident_w) mbar_wait_drain(smem_u32(wres_bar), 0);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    const bool leader = elect_one();
    // D = s32, A = B = s8, A K-major, B MN-major (bit 16), N = bn, M = 128
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(a.bn >> 3) << 17) |
                           (static_cast<uint32_t>(kTileCout >> 4) << 24);
    const int mma_per_stage = a.kc / 32;
    const uint32_t hi_a = static_cast<uint32_t>(make_smem_desc(0, a.kc) >> 32);
    // MN-major, 128-byte swizzle: groups of 8 K-rows are 1024 bytes apart (stride byte offset); the next 128
    // pixels are kc * 128 bytes further (leading byte offset)
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
    for (int tile = blockIdx.x; tile < a.num_tiles && ok; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      ok = mbar_wait(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * a.bn;
      for (int ks = 0; ks < a.ksteps; ++ks) {
        ok = mbar_wait(smem_u32(&full_bar[s]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st_lo = ring_lo + s * stage_lo;
        const uint32_t a_lo = (a.resident_w ? wres_lo + ks * wstep_lo : st_lo) | (1u << 16);
        const uint32_t b_lo = (st_lo + stage_a_lo) | lbo_b;
        for (int j = 0; j < mma_per_stage; ++j)  // 32 bytes of K: +32 B inside A's swizzle span, +32 rows (4 KiB) of B
          tc_mma_i8_halves(d_tmem, a_lo + 2u * j, hi_a, b_lo + 256u * j, hi_b, idesc, (ks | j) ? 1u : 0u, leader);
        tc_commit_if(smem_u32(&empty_bar[s]), leader);
        if (++s == a.stages) {
          s = 0;
          full_parity ^= 1;
        }
      }
      if (!ok) break;
      tc_commit_if(smem_u32(&acc_full[buf]), leader);
    }
  } else {
    // ------------------------------------------------------------ epilogue: 4 groups x 4 warps
    // Groups 0/1 take the CTA's even tiles (buffer 0), groups 2/3 the odd ones; the two groups of a tile split
    // its pixels in halves.  Warp w reads tensor-memory lanes 32*(w%4) .. +31 = 32 output channels.
    const int group = warp >> 2, quad = warp & 3;
    const int buf = group >> 1, col_par = group & 1;
    // pixels (= int8 bytes per staged row) of this warp: half a tile per group, halved again between the
    // lane quadrants 0/1 and 2/3 when the accumulator rows are duplicated
    const int wq = a.dup ? a.bn / 4 : a.bn / 2;
    const int cbase = col_par * (a.bn / 2) + (a.dup ? (quad >> 1) * wq : 0);
    const int row_quad = a.dup ? (quad & 1) : quad;  // which 32 output channels of the tile this warp owns
    const uint32_t st = smem_u32(smem_al) + warp * 4096;
    // int8 staging rows are wq bytes long, swizzled with span wq as the store's tensor map is
    const int b_swz = wq == 128 ? (lane & 7) : (wq == 64 ? ((lane >> 1) & 3) : ((lane >> 2) & 1));
    const float ub = quant_upper_bound<ACT>(a.alpha);
    bool stores_pending = false;
    bool ok = true;
    for (int it = buf; ok; it += 2) {
      const long tile_l = static_cast<long>(blockIdx.x) + static_cast<long>(it) * gridDim.x;
      if (tile_l >= a.num_tiles) break;
      int m0, p0, img;
      decode_tile(a, static_cast<int>(tile_l), m0, p0, img);
      const int row0 = m0 + row_quad * 32;
      const bool active = row0 < a.cout;          // warp-uniform
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
      const uint32_t lane_addr = tmem_base + buf * a.bn + (static_cast<uint32_t>(quad * 32) << 16);
      bool wrote_b = false;
      for (int c = cbase; active && c < cbase + wq; c += 32) {
        if (p0 + c >= a.hw) break;                // warp-uniform: pixels past the image
        uint32_t r[32];
        tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
        tc_wait_ld();
        if (stores_pending && (MODE != OUT_I8 || c == cbase)) {
          // the staging tile is about to be overwritten: earlier stores must have read it
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
          stores_pending = false;
        }
        if (MODE == OUT_I8) {
          const uint32_t row = st + lane * wq;
          const int chunk0 = (c - cbase) >> 4;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t q[4];
            if (a.acc_small) {
#pragma unroll
              for (int j = 0; j < 4; ++j) q[j] = quant4<ACT, true>(&r[16 * h + 4 * j], sc4, bi4, a.alpha, ub);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) q[j] = quant4<ACT, false>(&r[16 * h + 4 * j], sc4, bi4, a.alpha, ub);
            }
            sts128(row + (((chunk0 + h) ^ b_swz) << 4), q[0], q[1], q[2], q[3]);
          }
          wrote_b = true;
        } else {
          const uint32_t row = st + lane * 128;
          const int sw = lane & 7;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int acc = static_cast<int>(r[4 * j + e]);
              v[e] = MODE == OUT_ACC ? static_cast<uint32_t>(acc)
                                     : __float_as_uint(act_f32<ACT>(fmaf(__int2float_rn(acc), sc, bi), a.alpha));
            }
            sts128(row + ((j ^ sw) << 4), v[0], v[1], v[2], v[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmOut, st, p0 + c, row0, img);  // clips channels past cout and pixels past hw
            bulk_commit();
          }
          stores_pending = true;
        }
      }
      if (wrote_b) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmOut, st, p0 + cbase, row0, img);
          bulk_commit();
        }
        stores_pending = true;
      }
      // this warp no longer reads the buffer: let the MMA warp overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
    }
    if (lane == 0) bulk_wait_all();  // staging memory must outlive the stores reading it
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

typedef void (*NchwKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const NchwArgs);

template <int MODE>
NchwKernel pick_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return igemm_nchw_kernel<MODE, PLB_ACT_RELU>;
    case PLB_ACT_RELU6: return igemm_nchw_kernel<MODE, PLB_ACT_RELU6>;
    case PLB_ACT_LEAKY: return igemm_nchw_kernel<MODE, PLB_ACT_LEAKY>;
    default: return igemm_nchw_kernel<MODE, PLB_ACT_NONE>;
  }
}

NchwKernel pick_kernel(int mode, int act) {
  if (mode == OUT_I8) return pick_act<OUT_I8>(act);
  if (mode == OUT_F32) return pick_act<OUT_F32>(act);
  return igemm_nchw_kernel<OUT_ACC, PLB_ACT_NONE>;
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

bool igemm_nchw_supported(const NchwProblem& p, std::string* why) {
  auto no = [&](const char* msg) {
    if (why) *why = msg;
    return false;
  };
  if (p.out_mode != OUT_I8 && p.out_mode != OUT_F32 && p.out_mode != OUT_ACC) return no("output mode");
  const int xp = p.x_pitch ? p.x_pitch : p.hw, yp = p.y_pitch ? p.y_pitch : p.hw;
  if (xp % 16 != 0 || xp < p.hw) return no("input rows must be a multiple of 16 bytes apart (TMA row strides)");
  if ((yp * (p.out_mode == OUT_I8 ? 1 : 4)) % 16 != 0 || yp < p.hw) return no("output rows must be a multiple of 16 bytes apart");
  if (p.cin_pad % 32 != 0 || p.cin > p.cin_pad) return no("filter rows must be padded to a multiple of 32 bytes");
  if (p.batch <= 0 || p.cout <= 0 || p.cin <= 0) return no("empty problem");
  if ((reinterpret_cast<uintptr_t>(p.x) & 15) || (reinterpret_cast<uintptr_t>(p.w) & 15) ||
      (reinterpret_cast<uintptr_t>(p.y) & 15))
    return no("tensor base addresses must be 16-byte aligned");
  return true;
}

int igemm_nchw_launch(plb_ctx* ctx, const NchwProblem& p) {
  std::string why;
  if (!igemm_nchw_supported(p, &why)) return fail(PLB_E_UNSUPPORTED, "NCHW tensor-core path: %s", why.c_str());
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc = load_encoder();
    if (rc) return rc;
  }
  NchwArgs a;
  memset(&a, 0, sizeof(a));
  a.cout = p.cout;
  a.hw = p.hw;
  a.kc = p.cin_pad % 128 == 0 ? 128 : (p.cin_pad % 64 == 0 ? 64 : 32);
  a.ksteps = p.cin_pad / a.kc;
  a.tiles_m = (p.cout + kTileCout - 1) / kTileCout;
  a.dup = p.cout <= 64;
  // 256-pixel tiles halve the filter traffic per pixel; small images and small grids take 128
  a.bn = 256;
  if (p.hw <= 128 || static_cast<long>(p.batch) * ((p.hw + 255) / 256) * a.tiles_m < 2L * ctx->sm_count) a.bn = 128;
  a.tiles_p = (p.hw + a.bn - 1) / a.bn;
  const long tiles = static_cast<long>(p.batch) * a.tiles_p * a.tiles_m;
  if (tiles > 0x7fffffffL) return fail(PLB_E_UNSUPPORTED, "too many tiles");
  a.num_tiles = static_cast<int>(tiles);
  const int resident_bytes = a.ksteps * kTileCout * a.kc;
  const long grid_l = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  a.resident_w = grid_l % a.tiles_m == 0 && resident_bytes <= kMaxResidentW && tiles > grid_l;
  a.resident_bytes = a.resident_w ? resident_bytes : 0;
  const int stage_bytes = (a.resident_w ? 0 : kTileCout * a.kc) + a.kc * a.bn;
  int stages = (225 * 1024 - kStagingBytes - a.resident_bytes - kCtrlBytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return fail(PLB_E_UNSUPPORTED, "NCHW tensor-core path: the operand ring does not fit");
  a.stages = stages;
  a.scale = p.epi.scale;
  a.bias = p.epi.bias;
  a.alpha = p.epi.alpha;
  a.acc_small = p.epi.acc_small;
  a.status = ctx->d_status;

  alignas(64) CUtensorMap tmW, tmX, tmOut;
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
  {
    // X as [batch][cin][hw] bytes: a box is 128 pixels of kc channels of one image
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(p.hw), static_cast<cuuint64_t>(p.cin), static_cast<cuuint64_t>(p.batch)};
    const cuuint64_t xp = p.x_pitch ? p.x_pitch : p.hw;
    cuuint64_t strides[2] = {xp, xp * p.cin};
    cuuint32_t box[3] = {128, static_cast<cuuint32_t>(a.kc), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(p.x), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(NCHW input) failed: %d", (int)r);
  }
  {
    // Y as [batch][cout][hw]: a warp stores 32 channels x (bn/2 int8 pixels | 32 fp32 / int32 pixels)
    const int eb = p.out_mode == OUT_I8 ? 1 : 4;
    const int wq = a.dup ? a.bn / 4 : a.bn / 2;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(p.hw), static_cast<cuuint64_t>(p.cout), static_cast<cuuint64_t>(p.batch)};
    const cuuint64_t yp = p.y_pitch ? p.y_pitch : p.hw;
    cuuint64_t strides[2] = {yp * eb, yp * p.cout * eb};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(eb == 1 ? wq : 32), 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle sw = (eb == 4 || wq == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : (wq == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = g_encode(&tmOut, eb == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.y, dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(NCHW output) failed: %d", (int)r);
  }
  const size_t smem = static_cast<size_t>(kStagingBytes) + a.resident_bytes + static_cast<size_t>(stages) * stage_bytes +
                      kCtrlBytes + 1024;
  NchwKernel kernel = pick_kernel(p.out_mode, p.epi.act);
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
  const unsigned grid = static_cast<unsigned>(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  PLB_CUDA(launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, ctx->stream, tmW, tmX, tmOut, a));
  ctx->launches++;
  ctx->nchw_launches++;
  return PLB_OK;
}

}  // namespace plb
