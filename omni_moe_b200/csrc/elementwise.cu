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
//   act = silu(gate) * up,  dgate = dact * up * silu'(gate),  dup = dact * silu(gate)
// Outputs: dgu [T, 2I] = (dgate | dup) for the input-gradient GEMM and, for the weight-gradient GEMMs
// that contract over tokens, the transposed copies dgu_t [2I, ld_t] and act_t [I, ld_t] (columns
// T..ld_t-1 zero).  A block owns a 64-token x 64-column tile; the transposes go through shared memory.
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                                         int64_t T, int I, float limit, __nv_bfloat16* __restrict__ dgu,
                                                         uint16_t* __restrict__ dgu_t, uint16_t* __restrict__ act_t, int64_t ld_t,
                                                         __nv_bfloat16* __restrict__ act) {
  __shared__ uint16_t s_dg[kTile][kTile + 2], s_du[kTile][kTile + 2], s_ac[kTile][kTile + 2];
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * kTile;
  const int c0 = blockIdx.y * kTile;
  const int tr = threadIdx.x >> 3, tc = (threadIdx.x & 7) * 8;  // 32 rows x 8 column groups of 8
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = tr + 32 * half;
    const int64_t t = r0 + r;
    const int c = c0 + tc;
    uint32_t og[4] = {0, 0, 0, 0}, ou[4] = {0, 0, 0, 0}, oa[4] = {0, 0, 0, 0};
    if (t < T && c < I) {
      const uint4 gv = ldg128(gu + t * 2 * I + c), uv = ldg128(gu + t * 2 * I + I + c), dv = ldg128(dact + t * I + c);
      const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&uv);
      const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 g = bf16x2_to_float2(pg[q]), u = bf16x2_to_float2(pu[q]), d = bf16x2_to_float2(pd[q]);
        float rg[2], ru[2], ra[2];
        const float gg[2] = {g.x, g.y}, uu[2] = {u.x, u.y}, dd[2] = {d.x, d.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          // clamp of the forward (limit > 0): values are limited to [-limit, limit] and no gradient passes
          // where the pre-activation lies outside (the boundary itself passes, as torch.clamp does)
          const bool g_in = !(limit > 0.f) || fabsf(gg[e]) <= limit, u_in = !(limit > 0.f) || fabsf(uu[e]) <= limit;
          const float gc = g_in ? gg[e] : copysignf(limit, gg[e]), uc = u_in ? uu[e] : copysignf(limit, uu[e]);
          const float sig = 1.0f / (1.0f + __expf(-gc));
          const float sl = gc * sig;
          ra[e] = sl * uc;
          rg[e] = g_in ? dd[e] * uc * (sig * (1.0f + gc * (1.0f - sig))) : 0.f;
          ru[e] = u_in ? dd[e] * sl : 0.f;
        }
        og[q] = float2_to_bf16x2(rg[0], rg[1]);
        ou[q] = float2_to_bf16x2(ru[0], ru[1]);
        oa[q] = float2_to_bf16x2(ra[0], ra[1]);
      }
      *reinterpret_cast<uint4*>(dgu + t * 2 * I + c) = make_uint4(og[0], og[1], og[2], og[3]);
      *reinterpret_cast<uint4*>(dgu + t * 2 * I + I + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
      if (act) *reinterpret_cast<uint4*>(act + t * I + c) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
    }
    if (dgu_t) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        s_dg[r][tc + 2 * q] = static_cast<uint16_t>(og[q] & 0xffffu), s_dg[r][tc + 2 * q + 1] = static_cast<uint16_t>(og[q] >> 16);
        s_du[r][tc + 2 * q] = static_cast<uint16_t>(ou[q] & 0xffffu), s_du[r][tc + 2 * q + 1] = static_cast<uint16_t>(ou[q] >> 16);
        s_ac[r][tc + 2 * q] = static_cast<uint16_t>(oa[q] & 0xffffu), s_ac[r][tc + 2 * q + 1] = static_cast<uint16_t>(oa[q] >> 16);
      }
    }
  }
  if (!dgu_t) return;
  __syncthreads();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t gr = r0 + 2 * tx;  // token pair
  if (gr >= ld_t) return;
#pragma unroll
  for (int i = 0; i < kTile / 8; ++i) {
    const int c = ty + 8 * i;
    const int gc = c0 + c;
    if (gc >= I) continue;
    const uint32_t vg = static_cast<uint32_t>(s_dg[2 * tx][c]) | (static_cast<uint32_t>(s_dg[2 * tx + 1][c]) << 16);
    const uint32_t vu = static_cast<uint32_t>(s_du[2 * tx][c]) | (static_cast<uint32_t>(s_du[2 * tx + 1][c]) << 16);
    const uint32_t va = static_cast<uint32_t>(s_ac[2 * tx][c]) | (static_cast<uint32_t>(s_ac[2 * tx + 1][c]) << 16);
    *reinterpret_cast<uint32_t*>(dgu_t + static_cast<int64_t>(gc) * ld_t + gr) = vg;
    *reinterpret_cast<uint32_t*>(dgu_t + (static_cast<int64_t>(I) + gc) * ld_t + gr) = vu;
    *reinterpret_cast<uint32_t*>(act_t + static_cast<int64_t>(gc) * ld_t + gr) = va;
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

extern "C" int omni_swiglu_bwd_limit(const void* gate_up, const void* dact, int64_t num_tokens, int intermediate, float limit,
                                     void* dgate_up, void* dgate_up_t, void* act_t, int64_t ld_t, void* act, void* stream) {
  OMNI_REQUIRE(limit >= 0.f, "limit must be >= 0 (0 = no clamp)");
  OMNI_REQUIRE(num_tokens >= 0 && intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8");
  OMNI_REQUIRE((dgate_up_t == nullptr) == (act_t == nullptr), "dgate_up_t and act_t must be given together");
  OMNI_REQUIRE(dgate_up_t == nullptr || (ld_t >= num_tokens && ld_t % 2 == 0), "ld_t must be even and >= num_tokens");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(gate_up && dact && dgate_up, "NULL argument");
  OMNI_REQUIRE(aligned16(gate_up) && aligned16(dact) && aligned16(dgate_up) && aligned16(dgate_up_t) && aligned16(act_t) && aligned16(act),
               "pointers must be 16-byte aligned");
  // with transposed outputs the token tiles also cover the padding columns num_tokens..ld_t-1 (zeros)
  const int64_t gx = ceil_div64(dgate_up_t ? ld_t : num_tokens, kTile);
  const int64_t gy = ceil_div64(intermediate, kTile);
  OMNI_REQUIRE(gy <= 65535, "intermediate too large for one launch");
  swiglu_bwd_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<const __nv_bfloat16*>(dact), num_tokens, intermediate, limit,
      static_cast<__nv_bfloat16*>(dgate_up), static_cast<uint16_t*>(dgate_up_t), static_cast<uint16_t*>(act_t), ld_t,
      static_cast<__nv_bfloat16*>(act));
  return check_launch("swiglu_bwd_kernel");
}

extern "C" int omni_swiglu_bwd(const void* gate_up, const void* dact, int64_t num_tokens, int intermediate, void* dgate_up,
                               void* dgate_up_t, void* act_t, int64_t ld_t, void* stream) {
  return omni_swiglu_bwd_limit(gate_up, dact, num_tokens, intermediate, 0.f, dgate_up, dgate_up_t, act_t, ld_t, nullptr, stream);
}

// ------------------------------------------------------------------------------------------------
// Training-mode BatchNorm of the router logits (nn.BatchNorm1d(affine=False), batch statistics over
// all T tokens): column mean and biased variance of logits [T, C] (C = 2 * sqrt_n, both axes), folded
// into the per-column scale / shift the selection kernels take, plus the update of the running
// statistics.  Two launches, no atomics:
//   bn_partial_kernel   block b owns rows [b * kBnRows, ...): per column its mean and sum of squared
//                       deviations (two sweeps over the block's rows, so nothing cancels); it also
//                       counts the batch in num_batches_tracked
//   bn_finalize_kernel  one thread per column combines the block partials in block order (weighted mean of
//                       the means, squared deviations re-centred on it), writes scale = rsqrt(var + eps),
//                       shift = -mean * scale, and updates running_mean / running_var (momentum, unbiased
//                       variance) and num_batches_tracked exactly as nn.BatchNorm1d does in training.
namespace omni {
namespace {
constexpr int kBnRows = 32;

__global__ void __launch_bounds__(256) bn_partial_kernel(const float* __restrict__ z, int64_t T, int C, int64_t ld,
                                                         float* __restrict__ partial /*[blocks, 2, C]*/, long long* nbt_x,
                                                         long long* nbt_y) {
  // this batch counts: the finalize kernel, launched after this one, reads the incremented counters
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (nbt_x) *nbt_x += 1;
    if (nbt_y) *nbt_y += 1;
  }
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * kBnRows;
  const int rows = (T - r0 < kBnRows) ? static_cast<int>(T - r0) : kBnRows;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float sum = 0.f;
    for (int r = 0; r < rows; ++r) sum += z[(r0 + r) * ld + c];
    const float mean = sum / static_cast<float>(rows);
    float m2 = 0.f;
    for (int r = 0; r < rows; ++r) {
      const float d = z[(r0 + r) * ld + c] - mean;
      m2 = __fmaf_rn(d, d, m2);
    }
    partial[(static_cast<int64_t>(blockIdx.x) * 2 + 0) * C + c] = mean;
    partial[(static_cast<int64_t>(blockIdx.x) * 2 + 1) * C + c] = m2;
  }
}

__global__ void __launch_bounds__(256) bn_finalize_kernel(const float* __restrict__ partial, int blocks, int64_t T, int C,
                                                          int n_axis, float eps_x, float eps_y, float momentum_x, float momentum_y,
                                                          float* __restrict__ scale, float* __restrict__ shift,
                                                          void* run_mean_x, void* run_var_x, void* run_mean_y, void* run_var_y,
                                                          int run_dtype, long long* nbt_x, long long* nbt_y) {
  // 256 threads = 8 slices x 32 columns: slice s adds the block partials b = s, s + 8, ...; the eight slice sums are
  // added in slice order.  All blocks but the last hold kBnRows rows: the batch mean is the count-weighted mean of
  // the block means and the squared deviations add up as sum_b [M2_b + n_b (mean_b - mean)^2].
  __shared__ float s_part[8][32];
  const int col = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + col;
  const bool live = c < C;
  const float n = static_cast<float>(T);
  float wsum = 0.f;
  if (live)
    for (int b = slice; b < blocks; b += 8) {
      const int64_t left = T - static_cast<int64_t>(b) * kBnRows;
      const float nb = static_cast<float>(left < kBnRows ? left : kBnRows);
      wsum = __fmaf_rn(nb, partial[(static_cast<int64_t>(b) * 2 + 0) * C + c], wsum);
    }
  s_part[slice][col] = wsum;
  __syncthreads();
  float mean = 0.f;
#pragma unroll
  for (int s_ = 0; s_ < 8; ++s_) mean += s_part[s_][col];
  mean /= n;
  __syncthreads();
  float q = 0.f;
  if (live)
    for (int b = slice; b < blocks; b += 8) {
      const int64_t left = T - static_cast<int64_t>(b) * kBnRows;
      const float nb = static_cast<float>(left < kBnRows ? left : kBnRows);
      const float d = partial[(static_cast<int64_t>(b) * 2 + 0) * C + c] - mean;
      q += partial[(static_cast<int64_t>(b) * 2 + 1) * C + c] + nb * d * d;
    }
  s_part[slice][col] = q;
  __syncthreads();
  if (slice != 0 || !live) return;
  float m2 = 0.f;
#pragma unroll
  for (int s_ = 0; s_ < 8; ++s_) m2 += s_part[s_][col];
  const float var = m2 / n;  // biased: what normalises the batch
  const bool is_y = c >= n_axis;
  const float eps = is_y ? eps_y : eps_x;
  const float sc = rsqrtf(var + eps);
  scale[c] = sc;
  shift[c] = -mean * sc;
  void* rm = is_y ? run_mean_y : run_mean_x;
  void* rv = is_y ? run_var_y : run_var_x;
  long long* nbt = is_y ? nbt_y : nbt_x;
  if (rm != nullptr && rv != nullptr) {
    const int j = is_y ? c - n_axis : c;
    float mom = is_y ? momentum_y : momentum_x;
    // momentum < 0 stands for None: cumulative moving average over the batches seen so far
    if (mom < 0.f) mom = 1.0f / static_cast<float>(nbt ? *nbt : 1);  // already counts this batch
    const float unbiased = n > 1.f ? m2 / (n - 1.f) : var;
    if (run_dtype == OMNI_F32) {
      float* m = static_cast<float*>(rm);
      float* v = static_cast<float*>(rv);
      m[j] = (1.f - mom) * m[j] + mom * mean;
      v[j] = (1.f - mom) * v[j] + mom * unbiased;
    } else {
      __nv_bfloat16* m = static_cast<__nv_bfloat16*>(rm);
      __nv_bfloat16* v = static_cast<__nv_bfloat16*>(rv);
      m[j] = __float2bfloat16_rn((1.f - mom) * __bfloat162float(m[j]) + mom * mean);
      v[j] = __float2bfloat16_rn((1.f - mom) * __bfloat162float(v[j]) + mom * unbiased);
    }
  }
}

}  // namespace
}  // namespace omni

extern "C" size_t omni_router_bn_train_scratch_bytes(int64_t num_tokens, int sqrt_n) {
  if (num_tokens <= 0 || sqrt_n <= 0) return 0;
  return static_cast<size_t>(ceil_div64(num_tokens, kBnRows)) * 2 * (2 * static_cast<size_t>(sqrt_n)) * sizeof(float);
}

extern "C" int omni_router_bn_train(const float* logits, int64_t ld_logits, int64_t num_tokens, int sqrt_n, float eps_x,
                                    float eps_y, float momentum_x, float momentum_y, void* running_mean_x, void* running_var_x,
                                    void* running_mean_y, void* running_var_y, int running_dtype, int64_t* num_batches_tracked_x,
                                    int64_t* num_batches_tracked_y, float* bn_scale, float* bn_shift, void* scratch,
                                    size_t scratch_bytes, void* stream) {
  OMNI_REQUIRE(num_tokens >= 1 && sqrt_n >= 1, "num_tokens and sqrt_n must be >= 1");
  OMNI_REQUIRE(ld_logits >= 2 * sqrt_n, "ld_logits %lld < 2*sqrt_n", static_cast<long long>(ld_logits));
  OMNI_REQUIRE(running_dtype == OMNI_F32 || running_dtype == OMNI_BF16, "running statistics must be float32 or bfloat16");
  OMNI_REQUIRE(logits && bn_scale && bn_shift && scratch, "NULL argument");
  OMNI_REQUIRE((running_mean_x == nullptr) == (running_var_x == nullptr) && (running_mean_y == nullptr) == (running_var_y == nullptr),
               "running mean and variance must be given together");
  OMNI_REQUIRE(scratch_bytes >= omni_router_bn_train_scratch_bytes(num_tokens, sqrt_n), "scratch too small: need %zu bytes",
               omni_router_bn_train_scratch_bytes(num_tokens, sqrt_n));
  const int C = 2 * sqrt_n;
  const int64_t blocks = ceil_div64(num_tokens, kBnRows);
  OMNI_REQUIRE(blocks < (int64_t(1) << 31), "too many tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(scratch);
  bn_partial_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(logits, num_tokens, C, ld_logits, partial,
                                                                   reinterpret_cast<long long*>(num_batches_tracked_x),
                                                                   reinterpret_cast<long long*>(num_batches_tracked_y));
  if (int e = check_launch("bn_partial_kernel")) return e;
  bn_finalize_kernel<<<ceil_div(C, 32), 256, 0, st>>>(partial, static_cast<int>(blocks), num_tokens, C, sqrt_n, eps_x, eps_y,
                                                      momentum_x, momentum_y, bn_scale, bn_shift, running_mean_x, running_var_x,
                                                      running_mean_y, running_var_y, running_dtype,
                                                      reinterpret_cast<long long*>(num_batches_tracked_x),
                                                      reinterpret_cast<long long*>(num_batches_tracked_y));
  return check_launch("bn_finalize_kernel");
}
