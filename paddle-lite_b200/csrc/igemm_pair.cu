// Two-SM tiles for the compute-bound int8 GEMMs (3x3 convolutions with many channels, large fc layers):
// tcgen05.mma.cta_group::2, one 256 x BN output tile per PAIR of CTAs (a cluster of two).
//
// Why: with one CTA per tile every 128 x BN x 32 MMA reads 4 KiB of A and BN * 32 bytes of B from shared memory
// and the copy engine writes the same amount into the operand ring; with BN = 128..256 that is the whole
// shared-memory bandwidth of an SM, and every CTA streams the whole filter.  In a pair each CTA holds its own 128
// rows of A and HALF of the filter tile, the tensor cores of both SMs read both halves, and each SM's accumulator
// (128 lanes x BN columns of tensor memory) is drained by its own epilogue warps exactly as in the one-SM kernel.
// Replaces the same reference code as igemm_tc.cu (im2col + gemm_s8u8, lite/backends/x86/math/gemm_s8u8_kernel.cc:353-891).
//
// Protocol between the two CTAs (rank 0 = leader, issues every MMA).  No multicast of any kind; every copy is a TMA
// load into the executing CTA's own shared memory:
//   full[s]       leader only.  The leader's producer arms it with the bytes of BOTH CTAs' copies of stage s; the copies
//                 of both CTAs complete on it (cp.async.bulk.tensor with .cta_group::2 may signal the partner's barrier).
//   empty[s]      each CTA its own.  The leader's MMA warp signals both with two tcgen05.commit (its own barrier and the
//                 follower's, addressed through the cluster window) once the MMAs reading stage s have retired.
//   acc_full[b]   each CTA its own, signalled the same way after a tile's last MMA.
//   acc_empty[b]  leader only: epilogue warps of BOTH CTAs arrive here (mbarrier.arrive on the cluster address) when they
//                 have drained buffer b.
// Every wait is bounded (tc::mbar_wait); a CTA that gives up makes its partner's waits run out too, both drain, meet at
// the closing cluster barrier, free their tensor memory and return.
#include "igemm_pair.cuh"

#include <algorithm>
#include <mutex>

#include "tc_device.cuh"

namespace plb {
namespace {

using namespace tc;

constexpr int kRowsPerCta = 128;
constexpr int kEpilogueGroups = 4;
constexpr int kEpilogueWarps = 4 * kEpilogueGroups;
constexpr int kProducerWarp = kEpilogueWarps;
constexpr int kMmaWarp = kEpilogueWarps + 1;
constexpr int kThreads = 32 * (kEpilogueWarps + 2);
constexpr int kMaxStages = 12;
constexpr int kCtrlBytes = 1024;
constexpr int kStagingBytes = kEpilogueWarps * 4096;

struct PairArgs {
  int im2col;
  int m_total, cout;
  int bn, kc, cchunks, ksteps, stages;
  int kh, kw;
  int ho, wo, stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int tiles_n, num_tiles;   // channel tiles, pair tiles (256 rows x bn)
  int ldy;
  const float* scale;
  const float* bias;
  float alpha;
  int acc_small;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc2_mma_i8(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "@q tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, p;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tc2_commit_if(uint32_t bar, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(bar),
      "r"(static_cast<uint32_t>(issue))
      : "memory");
}

// TMA loads whose completion may be counted on the partner CTA's barrier (cluster address)
__device__ __forceinline__ void tma2_load_2d_if(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];\n\t"
      "}" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tma2_load_im2col_4d_if(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w,
                                                       int h, int n, uint16_t off_w, uint16_t off_h, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %9, 0;\n\t"
      "@q cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};\n\t"
      "}" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h),
      "r"(static_cast<uint32_t>(issue))
      : "memory");
}

template <int MODE, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
    igemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmOut, const PairArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem_al = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  // [epilogue staging][operand ring: per stage 128 rows of A + bn/2 rows of B][barriers]
  const int stage_a = kRowsPerCta * a.kc;
  const int stage_b = (a.bn / 2) * a.kc;
  const int stage_bytes = stage_a + stage_b;
  uint8_t* smem = smem_al + kStagingBytes;
  uint8_t* ctrl = smem + a.stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool is_leader = rank == 0;
  const int pair = static_cast<int>(blockIdx.x >> 1), num_pairs = static_cast<int>(gridDim.x >> 1);
  uint32_t acc_cols = 32;
  while (acc_cols < static_cast<uint32_t>(a.bn)) acc_cols <<= 1;
  const uint32_t tmem_cols = 2 * acc_cols;  // two accumulator buffers

  if (warp == kProducerWarp) {
    constexpr int kBarriers = 2 * kMaxStages + 4;
    for (int i = lane; i < kBarriers; i += 32) {
      // "buffer drained": four warps of each of the two groups sharing a buffer, in both CTAs
      const bool drained = i >= 2 * kMaxStages + 2;
      mbar_init(smem_u32(&full_bar[i]), drained ? 16 : 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 0) *abort_flag = 0;
    {
      const CUtensorMap* map = lane == 0 ? &tmA : lane == 1 ? &tmB : &tmOut;
      if (lane < 3) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
    }
  }
  if (warp == kMmaWarp) {
    // both CTAs of the pair allocate the same columns, from the warp of the same index
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync_with_previous_kernel();

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    const bool leader_lane = elect_one();
    int s = 0;
    uint32_t empty_parity = 1;
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t leader_full0 = map_to_cta(smem_u32(&full_bar[0]), 0);  // both CTAs' copies complete on the leader's barriers
    for (int tile = pair; tile < a.num_tiles && ok; tile += num_pairs) {
      const int tm = tile / a.tiles_n;
      const int m0 = tm * 2 * kRowsPerCta + static_cast<int>(rank) * kRowsPerCta;
      const int n0 = (tile - tm * a.tiles_n) * a.bn + static_cast<int>(rank) * (a.bn / 2);
      int q0 = 0, p0 = 0, cn = 0;
      if (a.im2col) {
        q0 = m0 % a.wo;
        const int t = m0 / a.wo;
        p0 = t % a.ho;
        cn = t / a.ho;
      }
      const int cw = q0 * a.stride_w - a.pad_l, ch = p0 * a.stride_h - a.pad_t;
      int r = 0, sx = 0, cc = 0, kb = 0;
      for (int ks = 0; ks < a.ksteps; ++ks) {
        ok = mbar_wait(smem_u32(&empty_bar[s]), empty_parity, abort_flag, a.status, FAULT_WAIT_EMPTY);
        if (!ok) break;
        const uint32_t bar = leader_full0 + 8u * s;
        const uint32_t dst = smem_base + s * stage_bytes;
        // the leader arms the barrier with the bytes of both CTAs (the follower's bytes may land first: the count
        // goes negative for a moment, the phase cannot complete before this arrival)
        if (is_leader) mbar_expect_tx_if(smem_u32(&full_bar[s]), 2u * static_cast<uint32_t>(stage_bytes), leader_lane);
        if (a.im2col)
          tma2_load_im2col_4d_if(dst, &tmA, bar, cc * a.kc, cw, ch, cn, static_cast<uint16_t>(sx * a.dil_w),
                                 static_cast<uint16_t>(r * a.dil_h), leader_lane);
        else
          tma2_load_2d_if(dst, &tmA, bar, kb, m0, leader_lane);
        tma2_load_2d_if(dst + stage_a, &tmB, bar, kb, n0, leader_lane);
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
    }
    if ((!ok || *abort_flag) && is_leader) {
      // gave up: bounded wait for the copies in flight (both CTAs' copies are counted on the leader's barriers)
      for (int j = 0; j < a.stages; ++j)
        mbar_wait_drain(smem_u32(&full_bar[j]), j < s ? (empty_parity ^ 1u) : empty_parity);
    }
  } else if (warp == kMmaWarp) {
    const bool leader_lane = elect_one();
    int s = 0, it = 0;
    uint32_t full_parity = 0;
    bool ok = true;
    if (is_leader) {
      // ---------------------------------------------------------- leader: MMA issue for both SMs (the follower's warp idles)
      // D = s32, A = B = s8, K-major, N = bn, M = 256 (128 rows per CTA)
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a.bn >> 3) << 17) |
                             (static_cast<uint32_t>(256 >> 4) << 24);
      const int mma_per_stage = a.kc / 32;
      const uint32_t hi = static_cast<uint32_t>(make_smem_desc(0, a.kc) >> 32);
      const uint32_t ring_lo = ((smem_u32(smem) >> 4) & 0x3FFFu) | (1u << 16);
      const uint32_t stage_lo = static_cast<uint32_t>(stage_bytes) >> 4;
      const uint32_t stage_a_lo = static_cast<uint32_t>(stage_a) >> 4;
      const uint32_t peer_empty0 = map_to_cta(smem_u32(&empty_bar[0]), 1);
      const uint32_t peer_acc_full0 = map_to_cta(smem_u32(&acc_full[0]), 1);
      for (int tile = pair; tile < a.num_tiles && ok; tile += num_pairs, ++it) {
        const int buf = it & 1;
        ok = mbar_wait(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * acc_cols;
        for (int ks = 0; ks < a.ksteps; ++ks) {
          ok = mbar_wait(smem_u32(&full_bar[s]), full_parity, abort_flag, a.status, FAULT_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = ring_lo + s * stage_lo;
          const uint32_t b_lo = a_lo + stage_a_lo;
          for (int j = 0; j < mma_per_stage; ++j)
            tc2_mma_i8(d_tmem, a_lo + 2u * j, hi, b_lo + 2u * j, hi, idesc, (ks | j) ? 1u : 0u, leader_lane);
          tc2_commit_if(smem_u32(&empty_bar[s]), leader_lane);   // stage s is free: in this CTA ...
          tc2_commit_if(peer_empty0 + 8u * s, leader_lane);       // ... and in the partner
          if (++s == a.stages) {
            s = 0;
            full_parity ^= 1;
          }
        }
        if (!ok) break;
        tc2_commit_if(smem_u32(&acc_full[buf]), leader_lane);
        tc2_commit_if(peer_acc_full0 + 8u * buf, leader_lane);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: 4 groups x 4 warps per CTA, own 128 rows
    // Groups 0/1 take the pair's even tiles (buffer 0), groups 2/3 the odd ones; the two groups of a tile split its
    // channels in halves.  One lane owns one output row (pixel) and 32 channels per chunk.
    const int group = warp >> 2, quad = warp & 3;
    const int buf = group >> 1, col_par = group & 1;
    const int wq = a.bn / 2;  // channels (= int8 bytes per staged row) of this group
    const int cbase = col_par * wq;
    const uint32_t st = smem_u32(smem_al) + warp * 4096;
    const int b_swz = wq == 128 ? (lane & 7) : (wq == 64 ? ((lane >> 1) & 3) : (wq == 32 ? ((lane >> 2) & 1) : 0));
    const float ub = quant_upper_bound<ACT>(a.alpha);
    const uint32_t leader_acc_empty = map_to_cta(smem_u32(&acc_empty[buf]), 0);
    bool stores_pending = false;
    bool ok = true;
    for (int it = buf; ok; it += 2) {
      const long tile_l = static_cast<long>(pair) + static_cast<long>(it) * num_pairs;
      if (tile_l >= a.num_tiles) break;
      const int tile = static_cast<int>(tile_l);
      const int tm = tile / a.tiles_n;
      const int m0 = tm * 2 * kRowsPerCta + static_cast<int>(rank) * kRowsPerCta;
      const int n0 = (tile - tm * a.tiles_n) * a.bn;
      const int row0 = m0 + quad * 32;
      const bool active = row0 < a.m_total;  // warp-uniform
      ok = mbar_wait(smem_u32(&acc_full[buf]), (it >> 1) & 1, abort_flag, a.status, FAULT_WAIT_ACCUM);
      if (!ok) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * acc_cols + (static_cast<uint32_t>(quad * 32) << 16);
      bool wrote_b = false;
      for (int c = cbase; active && c < cbase + wq; c += 32) {
        if (n0 + c >= a.cout) break;  // warp-uniform
        uint32_t r[32];
        tc_ld32(lane_addr + static_cast<uint32_t>(c), r);
        tc_wait_ld();
        if (stores_pending && (MODE != OUT_I8 || c == cbase)) {
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
          stores_pending = false;
        }
        const float4* sc4 = reinterpret_cast<const float4*>(a.scale + n0 + c);  // tables are padded past cout
        const float4* bi4 = reinterpret_cast<const float4*>(a.bias + n0 + c);
        if (MODE == OUT_I8) {
          const uint32_t row = st + lane * wq;
          const int chunk0 = (c - cbase) >> 4;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t q[4];
            if (a.acc_small) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                q[j] = quant4<ACT, true>(&r[16 * h + 4 * j], __ldg(sc4 + 4 * h + j), __ldg(bi4 + 4 * h + j), a.alpha, ub);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                q[j] = quant4<ACT, false>(&r[16 * h + 4 * j], __ldg(sc4 + 4 * h + j), __ldg(bi4 + 4 * h + j), a.alpha, ub);
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
            if (MODE == OUT_ACC) {
#pragma unroll
              for (int e = 0; e < 4; ++e) v[e] = r[4 * j + e];
            } else {
              const float4 sc = __ldg(sc4 + j), bi = __ldg(bi4 + j);
              v[0] = __float_as_uint(act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j]), sc.x, bi.x), a.alpha));
              v[1] = __float_as_uint(act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j + 1]), sc.y, bi.y), a.alpha));
              v[2] = __float_as_uint(act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j + 2]), sc.z, bi.z), a.alpha));
              v[3] = __float_as_uint(act_f32<ACT>(fmaf(__int2float_rn((int)r[4 * j + 3]), sc.w, bi.w), a.alpha));
            }
            sts128(row + ((j ^ sw) << 4), v[0], v[1], v[2], v[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmOut, st, n0 + c, row0);  // clips rows past m_total and channels past cout
            bulk_commit();
          }
          stores_pending = true;
        }
      }
      if (wrote_b) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmOut, st, n0 + cbase, row0);
          bulk_commit();
        }
        stores_pending = true;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(leader_acc_empty);  // the leader's barrier, also from the leader itself
    }
    if (lane == 0) bulk_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory its partner's MMAs or epilogue may still touch
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

typedef void (*PairKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const PairArgs);

template <int MODE>
PairKernel pick_act(int act) {
  switch (act) {
    case PLB_ACT_RELU: return igemm_pair_kernel<MODE, PLB_ACT_RELU>;
    case PLB_ACT_RELU6: return igemm_pair_kernel<MODE, PLB_ACT_RELU6>;
    case PLB_ACT_LEAKY: return igemm_pair_kernel<MODE, PLB_ACT_LEAKY>;
    default: return igemm_pair_kernel<MODE, PLB_ACT_NONE>;
  }
}
PairKernel pick_kernel(int mode, int act) {
  if (mode == OUT_I8) return pick_act<OUT_I8>(act);
  if (mode == OUT_F32) return pick_act<OUT_F32>(act);
  return igemm_pair_kernel<OUT_ACC, PLB_ACT_NONE>;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeTiledFn g_tiled = nullptr;
EncodeIm2colFn g_im2col = nullptr;
std::mutex g_mutex;

int load_encoders() {
  if (g_tiled && g_im2col) return PLB_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled unavailable");
  g_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  fn = nullptr;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return fail(PLB_E_CUDA, "cuTensorMapEncodeIm2col unavailable");
  g_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  return PLB_OK;
}

}  // namespace

bool igemm_pair_wanted(const plb_ctx* ctx, const IgemmProblem& p) {
  const int sw = p.sw ? p.sw->pair : -1;
  if (sw == 0) return false;
  if (p.out_mode != OUT_I8 && p.out_mode != OUT_F32 && p.out_mode != OUT_ACC) return false;
  if (p.a2 != nullptr || p.cin_pad % 32 != 0 || ctx->sm_count < 2) return false;
  const int cout16 = (p.cout + 15) / 16 * 16;
  const int bn = cout16 < 256 ? cout16 : 256;
  if (bn != 64 && bn != 128 && bn != 256) return false;   // staged epilogue: power-of-two channel tiles
  if (p.out_mode == OUT_I8 ? p.ldy % 16 != 0 : p.ldy % 4 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15) ||
      (reinterpret_cast<uintptr_t>(p.y) & 15))
    return false;
  if (sw == 1) return true;
  // Default: large flat GEMMs (fc) with 256-wide channel tiles and enough tiles to keep every pair busy, where the
  // one-SM kernel is bound by shared-memory bandwidth (4096^3: 51 us against 56 us, 2.69 POP/s).  Convolutions
  // fetched tap by tap stay with the one-SM kernel: they are bound by the number of TMA instructions per K step,
  // which pairing does not change (3x3 128 -> 128 on 28 x 28: 20 us against 18 us).
  // Large launches of convolutions with 256-wide channel tiles gain too once every pair has several tiles (3x3 256 -> 256
  // on 14 x 14: 25.9 us against 26.2 at 256 images, 46 against 49 at 512, 86 against 97 at 1024 = 0.61 of the datasheet peak).
  const long tiles = static_cast<long>((p.m_total + 255) / 256) * ((p.cout + bn - 1) / bn);
  if (p.im2col) return bn == 256 && tiles >= ctx->sm_count;
  return p.cin_pad >= 2048 && bn == 256 && tiles >= ctx->sm_count / 2;
}

int igemm_pair_launch(plb_ctx* ctx, const IgemmProblem& p) {
  std::string why;
  if (!igemm_tc_supported(p, &why)) return fail(PLB_E_UNSUPPORTED, "two-SM tensor-core path: %s", why.c_str());
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc = load_encoders();
    if (rc) return rc;
  }
  PairArgs a;
  memset(&a, 0, sizeof(a));
  a.im2col = p.im2col;
  a.m_total = p.m_total;
  a.cout = p.cout;
  a.kc = p.cin_pad % 128 == 0 ? 128 : (p.cin_pad % 64 == 0 ? 64 : 32);
  a.cchunks = p.cin_pad / a.kc;
  a.kh = p.im2col ? p.kh : 1;
  a.kw = p.im2col ? p.kw : 1;
  a.ksteps = a.kh * a.kw * a.cchunks;
  const int cout16 = (p.cout + 15) / 16 * 16;
  a.bn = cout16 < 256 ? cout16 : 256;
  a.tiles_n = (p.cout + a.bn - 1) / a.bn;
  const long tiles = static_cast<long>((p.m_total + 255) / 256) * a.tiles_n;
  if (tiles > 0x7fffffffL) return fail(PLB_E_UNSUPPORTED, "too many tiles");
  a.num_tiles = static_cast<int>(tiles);
  const int stage_bytes = (kRowsPerCta + a.bn / 2) * a.kc;
  int stages = (225 * 1024 - kStagingBytes - kCtrlBytes) / stage_bytes;
  if (p.sw && p.sw->stages > 0) stages = p.sw->stages;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return fail(PLB_E_UNSUPPORTED, "two-SM tensor-core path: the operand ring does not fit");
  a.stages = stages;
  a.ho = p.ho; a.wo = p.wo;
  a.stride_h = p.stride_h; a.stride_w = p.stride_w;
  a.pad_t = p.pad_t; a.pad_l = p.pad_l;
  a.dil_h = p.dil_h; a.dil_w = p.dil_w;
  a.ldy = p.ldy;
  a.scale = p.epi.scale; a.bias = p.epi.bias; a.alpha = p.epi.alpha;
  a.acc_small = p.epi.acc_small && (!p.sw || p.sw->acc_small != 0);
  a.status = ctx->d_status;

  alignas(64) CUtensorMap tmA, tmB, tmOut;
  const CUtensorMapSwizzle sw = a.kc == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                            : (a.kc == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  {
    // filter [cout, taps*cin_pad]: each CTA of a pair fetches bn/2 rows
    const cuuint64_t kbytes = static_cast<cuuint64_t>(a.kh * a.kw) * p.cin_pad;
    cuuint64_t dims[2] = {kbytes, static_cast<cuuint64_t>(p.cout)};
    cuuint64_t strides[1] = {kbytes};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(a.bn / 2)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_tiled(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.b), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(filter halves) failed: %d", (int)r);
  }
  if (!p.im2col) {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.m_total)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.cin_pad)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(kRowsPerCta)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_tiled(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.a), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(activations) failed: %d", (int)r);
  } else {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.w), static_cast<cuuint64_t>(p.h),
                          static_cast<cuuint64_t>(p.batch)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(p.cin_pad), static_cast<cuuint64_t>(p.cin_pad) * p.w,
                             static_cast<cuuint64_t>(p.cin_pad) * p.w * p.h};
    int lower[2] = {-p.pad_l, -p.pad_t};
    int upper[2] = {p.pad_r - (p.kw - 1) * p.dil_w, p.pad_b - (p.kh - 1) * p.dil_h};
    cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(p.stride_w), static_cast<cuuint32_t>(p.stride_h), 1};
    CUresult r = g_im2col(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(p.a), dims, strides, lower, upper,
                          static_cast<cuuint32_t>(a.kc), static_cast<cuuint32_t>(kRowsPerCta), estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeIm2col failed: %d", (int)r);
  }
  {
    const int eb = p.out_mode == OUT_I8 ? 1 : 4;
    const int wq = a.bn / 2;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cout), static_cast<cuuint64_t>(p.m_total)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldy) * eb};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(eb == 1 ? wq : 32), 32};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle osw = (eb == 4 || wq == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                                   : (wq == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = g_tiled(&tmOut, eb == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, p.y, dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, osw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PLB_E_CUDA, "cuTensorMapEncodeTiled(output) failed: %d", (int)r);
  }
  const size_t smem = static_cast<size_t>(kStagingBytes) + static_cast<size_t>(stages) * stage_bytes + kCtrlBytes + 1024;
  PairKernel kernel = pick_kernel(p.out_mode, p.epi.act);
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    static std::vector<std::pair<const void*, int>> configured;
    const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), ctx->device);
    if (std::find(configured.begin(), configured.end(), key) == configured.end()) {
      PLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      configured.push_back(key);
    }
  }
  const long max_pairs = ctx->sm_count / 2;
  const unsigned pairs = static_cast<unsigned>(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  PLB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmOut, a));
  ctx->launches++;
  ctx->pair_launches++;
  return PLB_OK;
}

}  // namespace plb
