// Product-key router selection as a kernel of its own: one warp per token (see router_select.cuh).
#include "router_select.cuh"

namespace omni {
namespace {

using namespace sel;
constexpr int kWarpsPerBlock = 4;

template <int VPL, int CPL, bool PRE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) router_topk_kernel(const TopkArgs a) {
  __shared__ WarpScratch<VPL, CPL> s_warp[kWarpsPerBlock];
  __shared__ RegionTable s_region;
  build_region_table(s_region, a.kk, a.k, kWarpsPerBlock);
  const int lane = lane_id();
  const int warp = threadIdx.x >> 5;
  const int k = a.k;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (t >= a.T) return;
  uint32_t rkey[kMaxK / 32], rflat[kMaxK / 32];
  select_token<VPL, CPL, PRE>(a, t, s_warp[warp], s_region.cell, rkey, rflat);

  // ---- results: lane (r % 32) holds rank r in slot r / 32 ----------------------------------
#pragma unroll
  for (int s = 0; s < kMaxK / 32; ++s) {
    const int r = s * 32 + lane;
    if (r < k) {
      const float sc = key_to_float(rkey[s]);
      const int64_t o = t * k + r;
      a.scores[o] = sc;
      if (a.idx_is_i64) reinterpret_cast<int64_t*>(a.indices)[o] = rflat[s];
      else reinterpret_cast<int32_t*>(a.indices)[o] = static_cast<int32_t>(rflat[s]);
      if (a.weights) a.weights[o] = expf(sc);
    }
  }
}

template <int VPL, bool PRE>
int launch_cpl(const TopkArgs& a, cudaStream_t st) {
  const unsigned grid = static_cast<unsigned>(ceil_div64(a.T, kWarpsPerBlock));
  const dim3 block(kWarpsPerBlock * 32);
  const int need = ceil_div(a.cells, 32);
  // An SM runs blocks of different kernels side by side only if they agree on its shared-memory /
  // L1 split.  The GEMMs of the layer need the largest shared-memory split; asking for the same one
  // here lets these small blocks run next to a GEMM block instead of waiting for the SM to drain.
#define OMNI_TOPK_LAUNCH(CPL_)                                                                                  \
  do {                                                                                                          \
    static OncePerDevice once;                                                                                  \
    if (once.first())                                                                                           \
      cudaFuncSetAttribute(router_topk_kernel<VPL, CPL_, PRE>, cudaFuncAttributePreferredSharedMemoryCarveout,  \
                           cudaSharedmemCarveoutMaxShared);                                                     \
    router_topk_kernel<VPL, CPL_, PRE><<<grid, block, 0, st>>>(a);                                              \
  } while (0)
  if (need <= 2) OMNI_TOPK_LAUNCH(2);
  else if (need <= 4) OMNI_TOPK_LAUNCH(4);
  else if (need <= 10) OMNI_TOPK_LAUNCH(10);
  else OMNI_TOPK_LAUNCH(22);
#undef OMNI_TOPK_LAUNCH
  return check_launch("router_topk_kernel");
}

template <bool PRE>
int launch(const TopkArgs& a, cudaStream_t st) {
  if (a.n <= 64) return launch_cpl<2, PRE>(a, st);
  if (a.n <= 128) return launch_cpl<4, PRE>(a, st);
  if (a.n <= 256) return launch_cpl<8, PRE>(a, st);
  if (a.n <= 512) return launch_cpl<16, PRE>(a, st);
  return launch_cpl<32, PRE>(a, st);
}

int check_common(int64_t T, int n, int k, const void* scores, const void* indices) {
  OMNI_REQUIRE(T >= 0, "num_tokens must be >= 0, got %lld", static_cast<long long>(T));
  OMNI_REQUIRE(n >= 1 && n <= 1024, "sqrt_n must be in [1, 1024], got %d", n);
  OMNI_REQUIRE(k >= 1 && k <= kMaxK, "k must be in [1, %d], got %d", kMaxK, k);
  OMNI_REQUIRE(static_cast<int64_t>(k) <= static_cast<int64_t>(n) * n, "k = %d exceeds the %d experts", k, n * n);
  OMNI_REQUIRE(T == 0 || (scores && indices), "scores and indices must not be NULL");
  return 0;
}

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" int omni_router_topk(const void* log_probs_x, const void* log_probs_y, int in_dtype,
                                int64_t num_tokens, int sqrt_n, int k, float* scores, void* indices,
                                int idx_is_i64, float* weights, void* stream) {
  if (int e = check_common(num_tokens, sqrt_n, k, scores, indices)) return e;
  OMNI_REQUIRE(in_dtype == OMNI_F32 || in_dtype == OMNI_BF16 || in_dtype == OMNI_F16, "unknown in_dtype %d", in_dtype);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(log_probs_x && log_probs_y, "log_probs_x / log_probs_y must not be NULL");
  TopkArgs a{};
  a.in_x = log_probs_x, a.in_y = log_probs_y, a.in_dtype = in_dtype, a.ld_in = sqrt_n;
  a.T = num_tokens, a.n = sqrt_n, a.k = k, a.kk = sqrt_n < k ? sqrt_n : k;
  a.cells = region_cells(a.kk, k);
  a.scores = scores, a.indices = indices, a.idx_is_i64 = idx_is_i64, a.weights = weights;
  return launch<false>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_router_logits_topk(const float* logits, int64_t ld_logits, const float* bn_scale,
                                       const float* bn_shift, int64_t num_tokens, int sqrt_n, int k,
                                       float* scores, void* indices, int idx_is_i64, float* weights,
                                       float* log_probs_out, void* stream) {
  if (int e = check_common(num_tokens, sqrt_n, k, scores, indices)) return e;
  OMNI_REQUIRE(ld_logits >= 2 * sqrt_n, "ld_logits %lld < 2*sqrt_n", static_cast<long long>(ld_logits));
  OMNI_REQUIRE((bn_scale == nullptr) == (bn_shift == nullptr), "bn_scale and bn_shift must be given together");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(logits, "logits must not be NULL");
  TopkArgs a{};
  a.in_x = logits, a.in_y = nullptr, a.in_dtype = OMNI_F32, a.ld_in = ld_logits;
  a.bn_scale = bn_scale, a.bn_shift = bn_shift, a.lp_out = log_probs_out;
  a.T = num_tokens, a.n = sqrt_n, a.k = k, a.kk = sqrt_n < k ? sqrt_n : k;
  a.cells = region_cells(a.kk, k);
  a.scores = scores, a.indices = indices, a.idx_is_i64 = idx_is_i64, a.weights = weights;
  return launch<true>(a, static_cast<cudaStream_t>(stream));
}

#ifdef OMNI_TUNING
// tuning builds only: reads (summed over the slots) and clears the section clocks of select_token
extern "C" OMNI_API int omni_debug_select_profile(unsigned long long* host_out8) {
  static unsigned long long buf[4096 * 8];
  if (cudaMemcpyFromSymbol(buf, omni::sel::g_sel_prof, sizeof(buf)) != cudaSuccess) return -3;
  for (int i = 0; i < 8; ++i) host_out8[i] = 0;
  for (int s = 0; s < 4096; ++s)
    for (int i = 0; i < 8; ++i) host_out8[i] += buf[s * 8 + i];
  for (auto& v : buf) v = 0;
  return cudaMemcpyToSymbol(omni::sel::g_sel_prof, buf, sizeof(buf)) == cudaSuccess ? 0 : -3;
}
#endif
