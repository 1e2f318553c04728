// Self-test of the bounded device-side wait that every mbarrier poll of the GEMM kernels goes through.
//
// A wait that can never be satisfied must not hang the GPU: after a limited number of probes it raises the block's
// abort flag, reports OMNI_ST_WAIT_TIMEOUT through the status word and returns false, and every later wait of the
// block returns false at once.  The kernel below drives exactly that path on purpose-built state - a barrier of
// its own on which nobody ever arrives, with a small probe limit - so the path can be exercised on a GPU without
// starving a real kernel, without a trap, a bad address or an endless loop; the context stays usable.
#include "tcgen05.cuh"

namespace omni {
namespace {

__global__ void wait_timeout_selftest_kernel(int* out, uint32_t limit) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  int first = -1, second = -1;
  if (threadIdx.x == 0) first = tc::mbar_wait_slow(tc::smem_u32(&bar), 0, &abort_flag, out, limit) ? 1 : 0;
  __syncthreads();
  // the abort flag is up now: any other wait of the block gives up on its first look at it
  if (threadIdx.x == 32) second = tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_flag, out) ? 1 : 0;
  if (threadIdx.x == 0) out[1] = first, out[3] = abort_flag;
  if (threadIdx.x == 32) out[2] = second;
}

}  // namespace
}  // namespace omni

extern "C" int omni_selftest_wait_timeout(int32_t* out4, int probe_limit, void* stream) {
  OMNI_REQUIRE(out4 != nullptr, "out4 must not be NULL");
  OMNI_REQUIRE(probe_limit >= 1 && probe_limit <= (1 << 20), "probe_limit must be in [1, 2^20], got %d", probe_limit);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(out4, 0, 4 * sizeof(int32_t), st);
  omni::wait_timeout_selftest_kernel<<<1, 64, 0, st>>>(out4, static_cast<uint32_t>(probe_limit));
  return omni::check_launch("wait_timeout_selftest_kernel");
}
