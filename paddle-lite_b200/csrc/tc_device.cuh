// Device-side building blocks shared by the tensor-core kernels: PTX wrappers (mbarrier, TMA,
// tcgen05), bounded waits, the requantiser and the shared-memory staging helpers.
#pragma once
#include "common.cuh"

namespace plb {
namespace tc {

#ifdef PLB_TC_TEST_WAIT_LIMIT
constexpr uint32_t kWaitLimit = PLB_TC_TEST_WAIT_LIMIT;  // test build: waits give up after a few microseconds
#else
constexpr uint32_t kWaitLimit = 1u << 22;      // polls before a wait is declared lost
#endif
#ifndef PLB_POLL_SPIN
#define PLB_POLL_SPIN 8
#endif
constexpr uint32_t kPollSpin = PLB_POLL_SPIN;  // polls in a row before a waiting warp starts to sleep between polls
constexpr uint32_t kDrainLimit = 1u << 12;     // polls per barrier while a CTA that gave up waits for its copies in flight

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false (and records `code`) when the limit is reached or another
// role of this CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > kPollSpin) {
      __nanosleep(32);
      if ((it & 255u) == 0 && *abort_flag) return false;
    }
  }
  *abort_flag = 1;
  if (atomicCAS(status, 0, code) == 0) status[1] = static_cast<int>(blockIdx.x);
  return false;
}
// After a lost wait: give a copy that may still be in flight a bounded time to land.  Records nothing.
__device__ __forceinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kDrainLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return;
    __nanosleep(64);
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Predicated forms for the producer warp (see tc_mma_i8_halves).
__device__ __forceinline__ void mbar_expect_tx_if(uint32_t bar, uint32_t bytes, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t"
      "}" ::"r"(bar),
      "r"(bytes), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_if(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                               bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];\n\t"
      "}" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_if(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                               int c2, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %6, 0;\n\t"
      "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];\n\t"
      "}" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_if(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                               int c2, int c3, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "@q cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];\n\t"
      "}" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_if(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c,
                                                      int w, int h, int n, uint16_t off_w, uint16_t off_h,
                                                      bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %9, 0;\n\t"
      "@q cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};\n\t"
      "}" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h),
      "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// tcgen05.mma with the two shared-memory descriptors given as 32-bit halves (the high halves are loop constants).
// Issued by the lane(s) whose `issue` flag is set: the role loops run warp-uniformly and only the
// instruction itself is predicated, which keeps its operands warp-uniform values.
__device__ __forceinline__ void tc_mma_i8_halves(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc, uint32_t accumulate, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tc_commit_if(uint32_t bar, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(bar),
      "r"(static_cast<uint32_t>(issue))
      : "memory");
}
// One lane of a converged warp (the same one on every call).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are `kc` bytes long and
// swizzled with span `kc` (32/64/128): groups of 8 rows are 8*kc bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, int kc) {
  const uint32_t layout = kc == 128 ? 2u : (kc == 64 ? 4u : 6u);
  const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = ((static_cast<uint32_t>(8 * kc) >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// ---------------------------------------------------------------- epilogue of 32 columns
// One thread owns one output row (pixel) and 32 consecutive output channels of it, i.e. one
// full 32-byte sector of an int8 row or one full 128-byte line of an fp32 row.
//
// Rounding to int8 avoids the slow float->int conversion pipe: after clamping to
// [-127, 127] the value is added to 1.5 * 2^23, whose ulp is 1, so the addition itself rounds
// to nearest-even and leaves the two's-complement result in the low mantissa byte.

constexpr float kRoundMagic = 12582912.f;  // 1.5 * 2^23

__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Four int32 accumulators -> four requantised bytes clamp(rne(act(fmaf(float(acc), scale, bias))), -127, 127),
// with fewer instructions than the straightforward sequence and bit-identical results:
// * fp32 work on two values per instruction (f32x2 forms of add and fma, IEEE per lane);
// * SMALL (the host has proven |acc| < 2^22 from the filter): int -> float through the mantissa of
//   1.5 * 2^23 (one integer add and one fp add, exact) instead of the quarter-rate conversion pipe;
// * rounding by adding 1.5 * 2^23 AFTER the clamp to [-127, 127] (rounding and clamping commute because
//   the bounds are integers; the add is exact only inside that range, and clamping the bit pattern
//   afterwards instead would need an integer subtraction that overflows for v in (-2^24.6, -2^23.6)).
constexpr int kMagicBits = 0x4B400000;  // bit pattern of kRoundMagic

template <int ACT>
__device__ __forceinline__ float clamp_act(float v, float alpha, float ub) {
  if (ACT == PLB_ACT_NONE) return fminf(fmaxf(v, -127.f), 127.f);
  if (ACT == PLB_ACT_RELU) return fminf(fmaxf(v, 0.f), 127.f);
  if (ACT == PLB_ACT_RELU6) return fminf(fmaxf(v, 0.f), ub);  // ub = alpha limited to [-127, 127]
  v = v <= 0.f ? alpha * v : v;
  return fminf(fmaxf(v, -127.f), 127.f);
}

template <int ACT, bool SMALL>
__device__ __forceinline__ uint32_t quant4(const uint32_t* r, const float4 sc, const float4 bi, const float alpha,
                                           const float ub) {
  float2 f01, f23;
  if (SMALL) {
    const float2 nm = make_float2(-kRoundMagic, -kRoundMagic);
    f01 = __fadd2_rn(make_float2(__int_as_float(static_cast<int>(r[0]) + kMagicBits),
                                 __int_as_float(static_cast<int>(r[1]) + kMagicBits)), nm);
    f23 = __fadd2_rn(make_float2(__int_as_float(static_cast<int>(r[2]) + kMagicBits),
                                 __int_as_float(static_cast<int>(r[3]) + kMagicBits)), nm);
  } else {
    f01 = make_float2(__int2float_rn(static_cast<int>(r[0])), __int2float_rn(static_cast<int>(r[1])));
    f23 = make_float2(__int2float_rn(static_cast<int>(r[2])), __int2float_rn(static_cast<int>(r[3])));
  }
  const float2 v01 = __ffma2_rn(f01, make_float2(sc.x, sc.y), make_float2(bi.x, bi.y));
  const float2 v23 = __ffma2_rn(f23, make_float2(sc.z, sc.w), make_float2(bi.z, bi.w));
  const float2 m2 = make_float2(kRoundMagic, kRoundMagic);
  const float2 t01 = __fadd2_rn(make_float2(clamp_act<ACT>(v01.x, alpha, ub), clamp_act<ACT>(v01.y, alpha, ub)), m2);
  const float2 t23 = __fadd2_rn(make_float2(clamp_act<ACT>(v23.x, alpha, ub), clamp_act<ACT>(v23.y, alpha, ub)), m2);
  return pack_low_bytes(__float_as_uint(t01.x), __float_as_uint(t01.y), __float_as_uint(t23.x), __float_as_uint(t23.y));
}

template <int ACT>
__device__ __forceinline__ float quant_upper_bound(float alpha) {
  return ACT == PLB_ACT_RELU6 ? fmaxf(fminf(alpha, 127.f), -127.f) : 127.f;  // a (senseless) negative bound still ends in [-127, 127]
}

// 256-bit global accesses: one full 32-byte sector per lane and instruction
__device__ __forceinline__ void st_global_v8(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                             uint32_t e, uint32_t f, uint32_t g, uint32_t h) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a), "r"(b),
               "r"(c), "r"(d), "r"(e), "r"(f), "r"(g), "r"(h)
               : "memory");
}
__device__ __forceinline__ void st_global_v8f(float* p, float4 lo, float4 hi) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(lo.x),
               "f"(lo.y), "f"(lo.z), "f"(lo.w), "f"(hi.x), "f"(hi.y), "f"(hi.z), "f"(hi.w)
               : "memory");
}
__device__ __forceinline__ void ld_global_v8f(const float* p, float* out) {
  asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3]), "=f"(out[4]), "=f"(out[5]),
                 "=f"(out[6]), "=f"(out[7])
               : "l"(p));
}

template <int ACT>
__device__ __forceinline__ float act_f32(float v, float alpha) {
  if (ACT == PLB_ACT_RELU) return fmaxf(v, 0.f);
  if (ACT == PLB_ACT_RELU6) return fminf(fmaxf(v, 0.f), alpha);
  if (ACT == PLB_ACT_LEAKY) return v <= 0.f ? alpha * v : v;
  return v;
}

// ---------------------------------------------------------------- staging through shared memory
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace tc
}  // namespace plb
