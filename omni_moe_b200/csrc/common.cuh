// Shared helpers for the sm_100a kernels of libomni_moe_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/omni_moe_b200.h"

namespace omni {

// Records the message returned by omni_last_error() and yields the error code.
int fail(int code, const char* fmt, ...);

#define OMNI_REQUIRE(cond, ...)                      \
  do {                                               \
    if (!(cond)) return ::omni::fail(-1, __VA_ARGS__); \
  } while (0)

// Checks the launch itself (configuration errors show up here; kernels report through status words).
int check_launch(const char* what);

// omni_router_gate whose launch does nothing when `enable` is given and *enable == 0 on the device at the time it
// runs (a value written by an earlier kernel on the stream); sqrt_n < 128.
int router_gate_if(const void* x, const void* gate_x, const void* gate_y, int64_t num_tokens, int hidden, int sqrt_n,
                   float* logits, const int* enable, int32_t* status, void* stream);

constexpr unsigned FULL_MASK = 0xffffffffu;

// Programmatic dependent launch.  A kernel launched with launch_after_predecessor() may start while the
// kernel before it on the stream is still running; pdl_wait() blocks until that kernel has completed
// and its memory is visible, so everything before pdl_wait() (shared-memory set-up, TMEM allocation,
// descriptor prefetch) overlaps the predecessor's tail.  pdl_launch_dependents() lets the next kernel
// start early.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launches `kernel` so that it may overlap the tail of the previous kernel on `st` (see pdl_wait).
// OMNI_MOE_B200_PDL=0 turns the overlap off (ordinary stream order).
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_predecessor(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                            Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Per-device "done once" flag for settings that belong to a (kernel, device) pair, such as
// cudaFuncSetAttribute: a process that drives several GPUs must repeat them on each.
struct OncePerDevice {
  bool done[64] = {};
  // true the first time it is called with a given current device
  bool first() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return true;
    const bool was = done[dev];
    done[dev] = true;
    return !was;
  }
};

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Maps a float to an unsigned key whose integer order is the float order; -0.0 is first
// folded into +0.0 so the two tie, as they do under a float comparison.
__device__ __forceinline__ uint32_t float_to_key(float f) {
  uint32_t u = __float_as_uint(__fadd_rn(f, 0.0f));
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }
// two special-function operations (ex2, rcp) instead of a full-precision division; ~2 ulp
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// L2 cache policies for 128-bit loads: rows that are streamed once should leave L2 first, rows that
// are gathered again and again should stay.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ldg128_hint(const void* ptr, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr), "l"(policy));
  return v;
}

// 128-bit read-only load of 8 bf16.
__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t v) {
  // a bf16 is the upper half of an fp32
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

__device__ __forceinline__ uint32_t float2_to_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL_MASK, v, o));
  return v;
}

}  // namespace omni
