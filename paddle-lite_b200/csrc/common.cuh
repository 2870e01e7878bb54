// Shared host/device definitions for the plb200 kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/plb200.h"

// ---------------------------------------------------------------- error plumbing
namespace plb {

extern thread_local std::string g_last_error;
int fail(int code, const char* fmt, ...);

#define PLB_CUDA(expr)                                                                    \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return plb::fail(PLB_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                       __FILE__, __LINE__);                                               \
  } while (0)

#define PLB_REQUIRE(cond, ...)                                   \
  do {                                                           \
    if (!(cond)) return plb::fail(PLB_E_INVALID, __VA_ARGS__);   \
  } while (0)

// Device status word layout: status[0] = first fault code (0 = none), status[1] = detail.
enum DeviceFault : int {
  FAULT_NONE = 0,
  FAULT_WAIT_FULL = 1,   // MMA issuer gave up waiting for a TMA stage
  FAULT_WAIT_EMPTY = 2,  // TMA producer gave up waiting for a free stage
  FAULT_WAIT_ACCUM = 3,  // epilogue gave up waiting for the accumulator
};

}  // namespace plb

struct plb_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  int* d_status = nullptr;      // 2 ints on the device
  int* h_status = nullptr;      // pinned host copy, filled by an async copy in front of every host-side wait
  void* ws = nullptr;           // layout-staging scratch
  size_t ws_bytes = 0;
  bool ws_owned = false;
  long launches = 0;
  long window_launches = 0;     // tensor-core convolutions that ran in window (slab) mode
  long pair_launches = 0;       // GEMMs that ran as two-SM tiles (cta_group::2)
  long stem_launches = 0;       // first layers that ran from the fp32 image in one launch (no staging pass)
  long dwpw_launches = 0;       // depthwise + 1x1 pairs that ran as one launch
  long nchw_gather_launches = 0;  // ... of which on images TMA cannot address (operand tiles filled by gather warps)
  long nchw_launches = 0;       // 1x1 convolutions that ran on NCHW tensors directly (no layout staging)
  int reserve(size_t bytes);    // make ws at least `bytes`
};

// ---------------------------------------------------------------- epilogue description
struct EpiParams {
  const float* scale;   // [C] folded ws*in_s(/out_s)
  const float* bias;    // [C] folded bias(/out_s), zeros when absent
  int act;              // PLB_ACT_*
  float alpha;          // already divided by out_s where the reference does so
  int acc_small = 0;    // 1: 128 * (largest sum of |w| over one output channel) < 2^22, so every accumulator is
                        // below 2^22 in magnitude and converts to float exactly through the mantissa trick
  const float* h_scale = nullptr;  // host copies of scale / bias (or null): the one-launch first layer passes the
  const float* h_bias = nullptr;   // tables inside its kernel arguments
};

#ifdef __CUDACC__
namespace plb {

// Programmatic dependent launch: every kernel of the library is launched with the
// programmatic-stream-serialization attribute, so its blocks may start while the previous
// kernel on the stream is still draining.  A kernel therefore (1) lets its own dependents
// start early and (2) waits for the previous grid to finish and flush before it touches
// global memory.  Both instructions are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_sync_with_previous_kernel() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

bool pdl_enabled();  // PLB_PDL=0 in the environment turns the launch attribute off

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float act_apply(float v, int act, float alpha) {
  // gemm_fuse_relu_bias of the reference (gemm_s8u8_kernel.cc:31-55)
  if (act == PLB_ACT_RELU) return v > 0.f ? v : 0.f;
  if (act == PLB_ACT_RELU6) {
    v = v > 0.f ? v : 0.f;
    return v < alpha ? v : alpha;
  }
  if (act == PLB_ACT_LEAKY) return v <= 0.f ? alpha * v : v;
  return v;
}

// round-to-nearest-even, clamp to [-127, 127] (cvtps_epi32 + packs + max(-127))
__device__ __forceinline__ int requant_i8(float v) {
  int r = __float2int_rn(v);  // saturates on overflow, NaN -> 0
  r = r > 127 ? 127 : r;
  r = r < -127 ? -127 : r;
  return r;
}

// calib fp32 -> int8 of the reference: q = sat(rne(max(x * inv_scale, -127)))
__device__ __forceinline__ int calib_i8(float x, float inv_scale) {
  float v = x * inv_scale;
  v = v > -127.f ? v : -127.f;
  int r = __float2int_rn(v);
  return r > 127 ? 127 : r;
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
         ((uint32_t)(d & 0xff) << 24);
}

}  // namespace plb
#endif
