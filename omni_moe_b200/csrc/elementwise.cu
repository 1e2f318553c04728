// Memory-bound helpers of the MLP backward: a bf16 matrix transpose (the tensor-core GEMMs here take
// both operands with the contraction dimension contiguous, so weight gradients, which contract over
// tokens, are fed transposed copies) and the SwiGLU derivative.
#include "common.cuh"

namespace omni {
namespace {

constexpr int kTile = 64;

// out[c, r] = in[r, c] for r < rows, 0 for rows <= r < out_cols (the padding keeps the rows of `out`
// 16-byte aligned for TMA when `rows` is not a multiple of 8); ldo = row stride of out.
// cols, ld_in, out_cols, ldo even.
__global__ void __launch_bounds__(256) transpose_bf16_kernel(const uint16_t* __restrict__ in, int64_t rows, int64_t cols,
                                                             int64_t ld_in, uint16_t* __restrict__ out, int64_t out_cols, int64_t ldo) {
  __shared__ uint16_t tile[kTile][kTile + 2];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * kTile, c0 = static_cast<int64_t>(blockIdx.y) * kTile;
#pragma unroll
  for (int i = 0; i < kTile / 8; ++i) {
    const int r = ty + 8 * i;
    const int64_t gr = r0 + r, gc = c0 + 2 * tx;
    uint32_t v = 0;
    if (gr < rows && gc < cols) v = __ldg(reinterpret_cast<const uint32_t*>(in + gr * ld_in + gc));
    tile[r][2 * tx] = static_cast<uint16_t>(v & 0xffffu);
    tile[r][2 * tx + 1] = static_cast<uint16_t>(v >> 16);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kTile / 8; ++i) {
    const int c = ty + 8 * i;
    const int64_t gc = c0 + c, gr = r0 + 2 * tx;
    if (gc < cols && gr < out_cols) {
      const uint32_t v = static_cast<uint32_t>(tile[2 * tx][c]) | (static_cast<uint32_t>(tile[2 * tx + 1][c]) << 16);
      *reinterpret_cast<uint32_t*>(out + gc * ldo + gr) = v;
    }
  }
}

// gu [T, 2I] = (gate | up) pre-activations, dact [T, I]:
//   act = silu(gate) * up,  dgate = dact * up * silu'(gate),  dup = dact * silu(gate);  dgu = (dgate | dup)
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                                         int64_t T, int I, __nv_bfloat16* __restrict__ dgu,
                                                         __nv_bfloat16* __restrict__ act) {
  const int vec_per_row = I / 8;
  const int64_t total = T * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int c = static_cast<int>(i - t * vec_per_row) * 8;
    const uint4 gv = ldg128(gu + t * 2 * I + c), uv = ldg128(gu + t * 2 * I + I + c), dv = ldg128(dact + t * I + c);
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&uv);
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dv);
    uint32_t og[4], ou[4], oa[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 g = bf16x2_to_float2(pg[q]), u = bf16x2_to_float2(pu[q]), d = bf16x2_to_float2(pd[q]);
      float rg[2], ru[2], ra[2];
      const float gg[2] = {g.x, g.y}, uu[2] = {u.x, u.y}, dd[2] = {d.x, d.y};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float sig = 1.0f / (1.0f + __expf(-gg[e]));
        const float sl = gg[e] * sig;
        ra[e] = sl * uu[e];
        rg[e] = dd[e] * uu[e] * (sig * (1.0f + gg[e] * (1.0f - sig)));
        ru[e] = dd[e] * sl;
      }
      og[q] = float2_to_bf16x2(rg[0], rg[1]);
      ou[q] = float2_to_bf16x2(ru[0], ru[1]);
      oa[q] = float2_to_bf16x2(ra[0], ra[1]);
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * I + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + t * 2 * I + I + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    if (act) *reinterpret_cast<uint4*>(act + t * I + c) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" int omni_transpose_bf16(const void* in, int64_t rows, int64_t cols, int64_t ld_in, void* out, int64_t out_cols,
                                   int64_t ldo, void* stream) {
  OMNI_REQUIRE(rows >= 0 && cols >= 0, "bad sizes");
  OMNI_REQUIRE(cols % 2 == 0 && ld_in % 2 == 0 && out_cols % 2 == 0 && ldo % 2 == 0, "cols, ld_in, out_cols and ldo must be even");
  OMNI_REQUIRE(ld_in >= cols && out_cols >= rows && ldo >= out_cols, "leading dimensions too small");
  if (cols == 0 || out_cols == 0) return 0;
  OMNI_REQUIRE(in && out, "NULL argument");
  OMNI_REQUIRE((reinterpret_cast<uintptr_t>(in) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0, "pointers must be 4-byte aligned");
  const int64_t gx = ceil_div64(out_cols, kTile), gy = ceil_div64(cols, kTile);
  OMNI_REQUIRE(gy <= 65535, "too many columns for one launch: %lld", static_cast<long long>(cols));
  transpose_bf16_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(in), rows, cols, ld_in, static_cast<uint16_t*>(out), out_cols, ldo);
  return check_launch("transpose_bf16_kernel");
}

extern "C" int omni_swiglu_bwd(const void* gate_up, const void* dact, int64_t num_tokens, int intermediate, void* dgate_up,
                               void* act, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(gate_up && dact && dgate_up, "NULL argument");
  OMNI_REQUIRE(aligned16(gate_up) && aligned16(dact) && aligned16(dgate_up) && aligned16(act), "pointers must be 16-byte aligned");
  const int64_t total = num_tokens * (intermediate / 8);
  const int64_t blocks = ceil_div64(total, 256);
  const unsigned grid = static_cast<unsigned>(blocks < 148 * 16 ? blocks : 148 * 16);
  swiglu_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<const __nv_bfloat16*>(dact), num_tokens, intermediate,
      static_cast<__nv_bfloat16*>(dgate_up), static_cast<__nv_bfloat16*>(act));
  return check_launch("swiglu_bwd_kernel");
}
