// Backward passes of the router op and of the routed-expert op.
//
// Router (scores[t,j] = lpx[t, ix] + lpy[t, iy]):
//   dlpx[t, ix] += dscores[t,j],  dlpy[t, iy] += dscores[t,j]
//   router_bwd_kernel: one warp per token, the two gradient rows live in shared memory; the lane
//   (column mod 32) owns a column, so the adds of one column happen in program order of one lane:
//   no atomics, the same bits on every run.
//
// Routed experts, per pair p = (t, j), e = indices[t, j], g = weights[t, j]:
//   S  = x[t] . Up[e]            h = silu(S)          dA = dY[t] . Down[e]
//   dg = dA * h                  c = g * h            dS = dA * g * silu'(S)
//   dX[t]    += dS * Up[e]       (token-centric: in the dots kernel for rows up to 1024 columns, else the
//                                forward's combine kernel with Up and dS)
//   dUp[e]   += dS * x[t]        dDown[e] += c * dY[t]      (expert-centric, needs the schedule)
//   expert_bwd_dots_kernel  token-centric, one warp per token: both dot products of every pair, then
//                           dS, c and dg at the pair's place in the [T, k] tables.
//   expert_bwd_rows_kernel  one warp per expert segment of the schedule: walks the segment's pairs in
//                           sorted (= ascending pair id) order and accumulates both gradient rows in
//                           fp32 registers, 1024 columns at a time; each touched row is written once.
//                           Rows no pair touches are not written (the caller zero-fills a dense table
//                           or asks for compact rows, one per segment).
#include "common.cuh"

namespace omni {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;

// ------------------------------------------------------------------------------------------------
// router
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) router_bwd_kernel(const float* __restrict__ dscores, const void* __restrict__ indices,
                                                              int idx_is_i64, int64_t T, int n, int k, float* __restrict__ dlx,
                                                              float* __restrict__ dly, int* __restrict__ status) {
  extern __shared__ float s_rows[];  // per warp: n floats for the x axis, n for the y axis
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (t >= T) return;
  float* sx = s_rows + static_cast<size_t>(warp) * 2 * n;
  float* sy = sx + n;
  for (int c = lane; c < 2 * n; c += 32) sx[c] = 0.f;
  __syncwarp();
  bool bad = false;
  for (int j0 = 0; j0 < k; j0 += 32) {
    const int j = j0 + lane;
    int64_t e = -1;
    float d = 0.f;
    if (j < k) {
      e = idx_is_i64 ? reinterpret_cast<const int64_t*>(indices)[t * k + j] : reinterpret_cast<const int32_t*>(indices)[t * k + j];
      d = dscores[t * k + j];
      if (e < 0 || e >= static_cast<int64_t>(n) * n) bad = true, e = -1;
    }
    const int ix = e < 0 ? -1 : static_cast<int>(e / n);
    const int iy = e < 0 ? -1 : static_cast<int>(e - static_cast<int64_t>(ix) * n);
    const int cnt = min(32, k - j0);
    for (int i = 0; i < cnt; ++i) {
      const int bx = __shfl_sync(FULL_MASK, ix, i), by = __shfl_sync(FULL_MASK, iy, i);
      const float bd = __shfl_sync(FULL_MASK, d, i);
      if (bx >= 0) {
        if ((bx & 31) == lane) sx[bx] += bd;
        if ((by & 31) == lane) sy[by] += bd;
      }
    }
  }
  __syncwarp();
  for (int c = lane; c < n; c += 32) {
    dlx[t * n + c] = sx[c];
    dly[t * n + c] = sy[c];
  }
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

// ------------------------------------------------------------------------------------------------
// routed experts
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 dot8f(const uint4& a, const uint4& b, float2 acc) {
  const uint32_t* pa = reinterpret_cast<const uint32_t*>(&a);
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc = __ffma2_rn(bf16x2_to_float2(pa[i]), bf16x2_to_float2(pb[i]), acc);
  return acc;
}
__device__ __forceinline__ void axpy8f(float c, const uint4& d, float2 (&acc)[4]) {
  const uint32_t* pd = reinterpret_cast<const uint32_t*>(&d);
  const float2 c2 = make_float2(c, c);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = __ffma2_rn(c2, bf16x2_to_float2(pd[i]), acc[i]);
}

// One warp per token.  The token's x and dY rows are read through L1 (every pair of the token reads
// them again), the expert rows are streamed past it.
__global__ void __launch_bounds__(kThreads) expert_bwd_dots_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
    const __nv_bfloat16* __restrict__ dy, const float* __restrict__ weights, const int32_t* __restrict__ indices, int64_t T,
    int k, int H, int64_t N, float* __restrict__ ds, float* __restrict__ cdown, float* __restrict__ dg, int* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (t >= T) return;
  const __nv_bfloat16* xr = x + t * H;
  const __nv_bfloat16* dyr = dy + t * H;
  bool bad = false;
  for (int j0 = 0; j0 < k; j0 += 32) {
    const int j = j0 + lane;
    int my_e = -1;
    float my_g = 0.f;
    if (j < k) {
      my_e = indices[t * k + j];
      my_g = weights[t * k + j];
      if (my_e < 0 || my_e >= N) bad = true, my_e = -1;
    }
    const int cnt = min(32, k - j0);
    float my_ds = 0.f, my_c = 0.f, my_dg = 0.f;
    for (int i = 0; i < cnt; ++i) {
      const int e = __shfl_sync(FULL_MASK, my_e, i);
      if (e < 0) continue;  // warp-uniform
      const __nv_bfloat16* ur = up + static_cast<int64_t>(e) * H;
      const __nv_bfloat16* dr = down + static_cast<int64_t>(e) * H;
      float2 s2 = make_float2(0.f, 0.f), a2 = make_float2(0.f, 0.f);
      for (int c0 = lane * 8; c0 < H; c0 += 1024) {
        uint4 uv[4], dv[4], xv[4], gv[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int col = c0 + v * 256;
          const bool ld = col < H;
          uv[v] = ld ? ldg128(ur + col) : make_uint4(0, 0, 0, 0);
          dv[v] = ld ? ldg128(dr + col) : make_uint4(0, 0, 0, 0);
          xv[v] = ld ? *reinterpret_cast<const uint4*>(xr + col) : make_uint4(0, 0, 0, 0);
          gv[v] = ld ? *reinterpret_cast<const uint4*>(dyr + col) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          s2 = dot8f(xv[v], uv[v], s2);
          a2 = dot8f(gv[v], dv[v], a2);
        }
      }
      const float S = warp_sum(s2.x + s2.y);
      const float dA = warp_sum(a2.x + a2.y);
      if (lane == i) {
        const float sig = 1.0f / (1.0f + __expf(-S));
        const float h = S * sig;
        my_dg = dA * h;
        my_c = my_g * h;
        my_ds = dA * my_g * (sig * (1.0f + S * (1.0f - sig)));
      }
    }
    if (j < k) {
      ds[t * k + j] = my_ds;
      cdown[t * k + j] = my_c;
      dg[t * k + j] = my_dg;
    }
  }
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

template <bool OUT_F32>
__device__ __forceinline__ void store8(void* base, int64_t off, const float2 (&a)[4]) {
  if (OUT_F32) {
    float* o = reinterpret_cast<float*>(base) + off;
    *reinterpret_cast<float4*>(o) = make_float4(a[0].x, a[0].y, a[1].x, a[1].y);
    *reinterpret_cast<float4*>(o + 4) = make_float4(a[2].x, a[2].y, a[3].x, a[3].y);
  } else {
    uint4 p;
    p.x = float2_to_bf16x2(a[0].x, a[0].y), p.y = float2_to_bf16x2(a[1].x, a[1].y);
    p.z = float2_to_bf16x2(a[2].x, a[2].y), p.w = float2_to_bf16x2(a[3].x, a[3].y);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + off) = p;
  }
}

// The same for rows of at most 1024 columns: the token's x and dy rows stay in registers, unpacked to
// fp32 pairs, so a pair costs two row gathers and nothing else; two pairs are in flight.
__device__ __forceinline__ float2 dot8u(const float2 (&a)[4], const uint4& b, float2 acc) {
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc = __ffma2_rn(a[i], bf16x2_to_float2(pb[i]), acc);
  return acc;
}

template <int HV>
__global__ void __launch_bounds__(kThreads) expert_bwd_dots_reg_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
    const __nv_bfloat16* __restrict__ dy, const float* __restrict__ weights, const int32_t* __restrict__ indices, int64_t T,
    int k, int H, int64_t N, float* __restrict__ ds, float* __restrict__ cdown, float* __restrict__ dg, void* __restrict__ dx,
    int dx_f32, int* __restrict__ status) {
  constexpr bool kUnpacked = HV <= 4;
  constexpr int UNR = HV <= 4 ? 2 : 1;
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (t >= T) return;
  const int c0 = lane * 8;
  uint4 xv[HV], gv[HV];
  float2 xf[kUnpacked ? HV : 1][4], gf[kUnpacked ? HV : 1][4];
#pragma unroll
  for (int v = 0; v < HV; ++v) {
    const int col = c0 + v * 256;
    xv[v] = col < H ? ldg128(x + t * H + col) : make_uint4(0, 0, 0, 0);
    gv[v] = col < H ? ldg128(dy + t * H + col) : make_uint4(0, 0, 0, 0);
    if (kUnpacked) {
      const uint32_t* px = reinterpret_cast<const uint32_t*>(&xv[v]);
      const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv[v]);
#pragma unroll
      for (int q = 0; q < 4; ++q) xf[v][q] = bf16x2_to_float2(px[q]), gf[v][q] = bf16x2_to_float2(pg[q]);
    }
  }
  // dx[t] = sum_j dS[t,j] * Up[e]: the Up row of a pair is in registers for the dot product anyway, so the
  // input gradient is accumulated here too when the caller asks for it (dx != null)
  float2 dxa[HV][4];
#pragma unroll
  for (int v = 0; v < HV; ++v)
#pragma unroll
    for (int q = 0; q < 4; ++q) dxa[v][q] = make_float2(0.f, 0.f);
  bool bad = false;
  for (int j0 = 0; j0 < k; j0 += 32) {
    const int j = j0 + lane;
    int my_e = -1;
    float my_g = 0.f;
    if (j < k) {
      my_e = indices[t * k + j];
      my_g = weights[t * k + j];
      if (my_e < 0 || my_e >= N) bad = true, my_e = -1;
    }
    const int cnt = min(32, k - j0);
    float my_ds = 0.f, my_c = 0.f, my_dg = 0.f;
    for (int i = 0; i < cnt; i += UNR) {
      uint4 uv[UNR][HV], dv[UNR][HV];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int e = __shfl_sync(FULL_MASK, my_e, (i + u) & 31);
        const bool on = i + u < cnt && e >= 0;
#pragma unroll
        for (int v = 0; v < HV; ++v) {
          const int col = c0 + v * 256;
          const bool ld = on && col < H;
          uv[u][v] = ld ? ldg128(up + static_cast<int64_t>(e) * H + col) : make_uint4(0, 0, 0, 0);
          dv[u][v] = ld ? ldg128(down + static_cast<int64_t>(e) * H + col) : make_uint4(0, 0, 0, 0);
        }
      }
      float S[UNR], dA[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        float2 s2 = make_float2(0.f, 0.f), a2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int v = 0; v < HV; ++v) {
          if (kUnpacked) {
            s2 = dot8u(xf[v], uv[u][v], s2);
            a2 = dot8u(gf[v], dv[u][v], a2);
          } else {
            s2 = dot8f(xv[v], uv[u][v], s2);
            a2 = dot8f(gv[v], dv[u][v], a2);
          }
        }
        S[u] = s2.x + s2.y, dA[u] = a2.x + a2.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          S[u] += __shfl_xor_sync(FULL_MASK, S[u], o);
          dA[u] += __shfl_xor_sync(FULL_MASK, dA[u], o);
        }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        // S and dA are warp-uniform after the reduction: every lane forms dS (all of them need it for dx)
        const float gq = __shfl_sync(FULL_MASK, my_g, (i + u) & 31);
        const float sig = 1.0f / (1.0f + __expf(-S[u]));
        const float h = S[u] * sig;
        const float dsq = dA[u] * gq * (sig * (1.0f + S[u] * (1.0f - sig)));
        if (lane == i + u) {
          my_dg = dA[u] * h;
          my_c = my_g * h;
          my_ds = dsq;
        }
        if (dx != nullptr) {
#pragma unroll
          for (int v = 0; v < HV; ++v) axpy8f(dsq, uv[u][v], dxa[v]);  // rows of dead pairs were loaded as zeros
        }
      }
    }
    if (j < k) {
      const bool ok = my_e >= 0;
      ds[t * k + j] = ok ? my_ds : 0.f;
      cdown[t * k + j] = ok ? my_c : 0.f;
      dg[t * k + j] = ok ? my_dg : 0.f;
    }
  }
  if (dx != nullptr) {
#pragma unroll
    for (int v = 0; v < HV; ++v) {
      const int col = c0 + v * 256;
      if (col < H) {
        if (dx_f32) store8<true>(dx, t * H + col, dxa[v]);
        else store8<false>(dx, t * H + col, dxa[v]);
      }
    }
  }
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

// One warp per segment s of the schedule (expert expert_ids[s], sorted positions offsets[s] .. offsets[s+1]).
template <bool OUT_F32>
__global__ void __launch_bounds__(kThreads) expert_bwd_rows_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ ds,
    const float* __restrict__ cdown, const int32_t* __restrict__ sorted_pair_ids, const int32_t* __restrict__ expert_ids,
    const int32_t* __restrict__ offsets, const int32_t* __restrict__ num_segments, int64_t T, int k, int H, int compact,
    int long_threshold, int* __restrict__ long_count, void* __restrict__ d_up, void* __restrict__ d_down,
    int* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = lane_id();
  if (long_count && blockIdx.x == 0 && threadIdx.x == 0) *long_count = 0;  // filled by the long-segment kernel that follows
  const int64_t s = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (s >= *num_segments) return;
  const int begin = offsets[s], end = offsets[s + 1];
  if (end - begin > long_threshold) return;  // handled by the two long-segment kernels
  const int64_t row = compact ? s : static_cast<int64_t>(expert_ids[s]);
  bool bad = false;
  for (int c0 = lane * 8; c0 < H + lane * 8; c0 += 1024) {  // every lane makes the same number of trips
    float2 au[4][4], ad[4][4];
#pragma unroll
    for (int v = 0; v < 4; ++v)
#pragma unroll
      for (int q = 0; q < 4; ++q) au[v][q] = make_float2(0.f, 0.f), ad[v][q] = make_float2(0.f, 0.f);
    for (int p0 = begin; p0 < end; p0 += 32) {
      // lane l carries pair p0 + l of the segment
      const int p = p0 + lane;
      int my_t = -1;
      float my_s = 0.f, my_c = 0.f;
      if (p < end) {
        const int pid = sorted_pair_ids[p];
        const int64_t tok = pid / k;
        if (pid < 0 || tok >= T) bad = true;
        else my_t = static_cast<int>(tok), my_s = ds[pid], my_c = cdown[pid];
      }
      const int cnt = min(32, end - p0);
      for (int i = 0; i < cnt; ++i) {
        const int tok = __shfl_sync(FULL_MASK, my_t, i);
        const float cs = __shfl_sync(FULL_MASK, my_s, i), cc = __shfl_sync(FULL_MASK, my_c, i);
        if (tok < 0) continue;
        const __nv_bfloat16* xr = x + static_cast<int64_t>(tok) * H;
        const __nv_bfloat16* gr = dy + static_cast<int64_t>(tok) * H;
        uint4 xv[4], gv[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int col = c0 + v * 256;
          const bool ld = col < H;
          xv[v] = ld ? ldg128(xr + col) : make_uint4(0, 0, 0, 0);
          gv[v] = ld ? ldg128(gr + col) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          axpy8f(cs, xv[v], au[v]);
          axpy8f(cc, gv[v], ad[v]);
        }
      }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int col = c0 + v * 256;
      if (col < H) {
        store8<OUT_F32>(d_up, row * H + col, au[v]);
        store8<OUT_F32>(d_down, row * H + col, ad[v]);
      }
    }
  }
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_TOKEN_INDEX);
}

// ---- long segments ----------------------------------------------------------------------------
// An expert that receives thousands of pairs (skewed routing) would keep one warp busy for
// milliseconds.  Segments longer than C pairs are therefore summed in two levels:
//   expert_bwd_rows_long_kernel    block b owns the sorted positions [b*C, (b+1)*C), C = 64 ... 512 chosen by
//                                  the scratch size.  At most two long segments (longer than C) meet it (the
//                                  one covering its first position and the one covering its last); for each,
//                                  the block's C/64 warps sum their 64 positions apiece, combine through shared memory in warp order and
//                                  store one fp32 partial row pair in slot 2b (segment covers the block's
//                                  first position) or 2b+1.
//   expert_bwd_rows_reduce_kernel  one warp per long segment adds its partials in block order and writes
//                                  the gradient rows.
// Fixed assignment and fixed order: the sums are reproducible.
constexpr int kLongBlockMax = 512;  // positions per block: 64 per warp, 1 to 8 warps (C = 64, 128, 256 or 512)
constexpr int kLongCols = 256;      // columns per pass: one 128-bit load per lane
constexpr size_t kLongScratchBudget = size_t(256) << 20;

// index of the segment containing sorted position p: largest s with offsets[s] <= p
__device__ __forceinline__ int segment_of(const int32_t* __restrict__ offsets, int U, int p) {
  int lo = 0, hi = U - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (offsets[mid] <= p) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(kLongBlockMax / 2) expert_bwd_rows_long_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ ds,
    const float* __restrict__ cdown, const int32_t* __restrict__ sorted_pair_ids, const int32_t* __restrict__ offsets,
    const int32_t* __restrict__ num_segments, const int32_t* __restrict__ max_segment_len, int64_t P, int64_t T, int k, int H,
    int kLongBlock, int* __restrict__ long_count, int* __restrict__ long_list, float* __restrict__ scratch,
    int* __restrict__ status) {
  __shared__ float s_part[kLongBlockMax / 64][2][kLongCols];
  const int warps = blockDim.x >> 5;  // = kLongBlock / 64
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int U = *num_segments;
  if (U <= 0) return;
  if (max_segment_len && *max_segment_len <= kLongBlock) return;  // the usual case: no expert is that busy
  const int64_t lo = static_cast<int64_t>(blockIdx.x) * kLongBlock;
  if (lo >= P) return;
  const int64_t hi = (lo + kLongBlock < P) ? lo + kLongBlock : P;
  const int s_first = segment_of(offsets, U, static_cast<int>(lo));
  const int s_last = segment_of(offsets, U, static_cast<int>(hi - 1));
  bool bad = false;
  for (int which = 0; which < 2; ++which) {
    if (which == 1 && s_last == s_first) break;
    const int s = which == 0 ? s_first : s_last;
    const int begin = offsets[s], end = offsets[s + 1];
    if (end - begin <= kLongBlock) continue;  // block-uniform
    const int a = begin > lo ? begin : static_cast<int>(lo);
    const int c = end < hi ? end : static_cast<int>(hi);
    float* slot = scratch + (2 * static_cast<int64_t>(blockIdx.x) + which) * 2 * H;
    // the block holding the segment's first position enters it in the list the reduce kernel walks
    // (list order varies from run to run; every entry is reduced on its own, so results do not)
    if (threadIdx.x == 0 && begin >= lo) long_list[atomicAdd(long_count, 1)] = s;
    // this warp's positions: a + warp*64 + {lane, lane+32}
    int my_t[2];
    float my_s[2], my_c[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = a + warp * 64 + u * 32 + lane;
      my_t[u] = -1, my_s[u] = 0.f, my_c[u] = 0.f;
      if (p < c) {
        const int pid = sorted_pair_ids[p];
        const int64_t tok = pid / k;
        if (pid < 0 || tok >= T) bad = true;
        else my_t[u] = static_cast<int>(tok), my_s[u] = ds[pid], my_c[u] = cdown[pid];
      }
    }
    const int cnt = max(0, min(64, c - (a + warp * 64)));
    for (int c0 = 0; c0 < H; c0 += kLongCols) {
      const int col = c0 + lane * 8;
      float2 au[4], ad[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) au[q] = make_float2(0.f, 0.f), ad[q] = make_float2(0.f, 0.f);
      for (int i0 = 0; i0 < cnt; i0 += 4) {
        uint4 xv[4], gv[4];
        float cs[4], cc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u;
          const int src = i & 31;
          const int tok = (i < 32) ? __shfl_sync(FULL_MASK, my_t[0], src) : __shfl_sync(FULL_MASK, my_t[1], src);
          cs[u] = (i < 32) ? __shfl_sync(FULL_MASK, my_s[0], src) : __shfl_sync(FULL_MASK, my_s[1], src);
          cc[u] = (i < 32) ? __shfl_sync(FULL_MASK, my_c[0], src) : __shfl_sync(FULL_MASK, my_c[1], src);
          const bool ld = i < cnt && tok >= 0 && col < H;
          xv[u] = ld ? ldg128(x + static_cast<int64_t>(tok) * H + col) : make_uint4(0, 0, 0, 0);
          gv[u] = ld ? ldg128(dy + static_cast<int64_t>(tok) * H + col) : make_uint4(0, 0, 0, 0);
          if (!ld) cs[u] = 0.f, cc[u] = 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          axpy8f(cs[u], xv[u], au);
          axpy8f(cc[u], gv[u], ad);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        s_part[warp][0][lane * 8 + 2 * q] = au[q].x, s_part[warp][0][lane * 8 + 2 * q + 1] = au[q].y;
        s_part[warp][1][lane * 8 + 2 * q] = ad[q].x, s_part[warp][1][lane * 8 + 2 * q + 1] = ad[q].y;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < 2 * kLongCols; idx += blockDim.x) {
        const int tb = idx / kLongCols, cc2 = idx - tb * kLongCols;
        float sum = 0.f;
        for (int w = 0; w < warps; ++w) sum += s_part[w][tb][cc2];
        if (c0 + cc2 < H) slot[tb * H + c0 + cc2] = sum;
      }
      __syncthreads();
    }
  }
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_TOKEN_INDEX);
}

template <bool OUT_F32>
__global__ void __launch_bounds__(kThreads) expert_bwd_rows_reduce_kernel(
    const float* __restrict__ scratch, const int32_t* __restrict__ expert_ids, const int32_t* __restrict__ offsets,
    const int* __restrict__ long_count, const int* __restrict__ long_list, int H, int compact, int kLongBlock,
    void* __restrict__ d_up, void* __restrict__ d_down) {
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int count = *long_count;
  // blockIdx.y picks a tile of 256 columns, so a segment spread over hundreds of blocks is reduced by
  // H / 256 warps side by side; the partials are added in block order, four loads in flight
  const int c0 = blockIdx.y * 256 + lane * 8;
  if (c0 >= H) return;
  for (int i = blockIdx.x * kWarps + warp; i < count; i += gridDim.x * kWarps) {
    const int s = long_list[i];
    const int begin = offsets[s], end = offsets[s + 1];
    const int b0 = begin / kLongBlock, b1 = (end - 1) / kLongBlock;
    const int64_t row = compact ? s : static_cast<int64_t>(expert_ids[s]);
    float2 au[4], ad[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) au[q] = make_float2(0.f, 0.f), ad[q] = make_float2(0.f, 0.f);
    const int first_which = begin > b0 * kLongBlock ? 1 : 0;
    for (int b = b0; b <= b1; b += 4) {
      float4 u0[4], u1[4], d0[4], d1[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int bb = b + u;
        const bool on = bb <= b1;
        const int which = (bb == b0) ? first_which : 0;
        const float* slot = scratch + (2 * static_cast<int64_t>(on ? bb : b0) + which) * 2 * H;
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        u0[u] = on ? *reinterpret_cast<const float4*>(slot + c0) : z;
        u1[u] = on ? *reinterpret_cast<const float4*>(slot + c0 + 4) : z;
        d0[u] = on ? *reinterpret_cast<const float4*>(slot + H + c0) : z;
        d1[u] = on ? *reinterpret_cast<const float4*>(slot + H + c0 + 4) : z;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        au[0].x += u0[u].x, au[0].y += u0[u].y, au[1].x += u0[u].z, au[1].y += u0[u].w;
        au[2].x += u1[u].x, au[2].y += u1[u].y, au[3].x += u1[u].z, au[3].y += u1[u].w;
        ad[0].x += d0[u].x, ad[0].y += d0[u].y, ad[1].x += d0[u].z, ad[1].y += d0[u].w;
        ad[2].x += d1[u].x, ad[2].y += d1[u].y, ad[3].x += d1[u].z, ad[3].y += d1[u].w;
      }
    }
    store8<OUT_F32>(d_up, row * H + c0, au);
    store8<OUT_F32>(d_down, row * H + c0, ad);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" int omni_router_bwd(const float* dscores, const void* indices, int idx_is_i64, int64_t num_tokens, int sqrt_n,
                               int k, float* dlog_probs_x, float* dlog_probs_y, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && sqrt_n >= 1 && sqrt_n <= 1024 && k >= 0, "bad sizes (sqrt_n in [1, 1024])");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(dlog_probs_x && dlog_probs_y && status && (k == 0 || (dscores && indices)), "NULL argument");
  const unsigned grid = static_cast<unsigned>(ceil_div64(num_tokens, kWarps));
  const size_t smem = static_cast<size_t>(kWarps) * 2 * sqrt_n * sizeof(float);
  router_bwd_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(dscores, indices, idx_is_i64, num_tokens, sqrt_n,
                                                                                k, dlog_probs_x, dlog_probs_y, status);
  return check_launch("router_bwd_kernel");
}

extern "C" int omni_expert_bwd_dots_fuses_dx(int hidden) { return hidden <= 1024 ? 1 : 0; }

extern "C" int omni_expert_bwd_dots(const void* x, const void* up, const void* down, const void* dy, const float* weights,
                                    const int32_t* indices, int64_t num_tokens, int k, int hidden, int64_t num_experts,
                                    float* ds, float* cdown, float* dg, void* dx, int dx_dtype, int32_t* status, void* stream) {
  OMNI_REQUIRE(dx == nullptr || omni_expert_bwd_dots_fuses_dx(hidden),
               "dx can be fused for hidden <= 1024 only; pass NULL and use omni_expert_combine");
  OMNI_REQUIRE(dx == nullptr || dx_dtype == OMNI_F32 || dx_dtype == OMNI_BF16, "dx_dtype must be OMNI_F32 or OMNI_BF16");
  OMNI_REQUIRE(aligned16(dx), "dx must be 16-byte aligned");
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && hidden >= 8 && num_experts >= 1, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && up && down && dy && weights && indices && ds && cdown && dg && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up) && aligned16(down) && aligned16(dy), "x, up, down and dy must be 16-byte aligned");
  const unsigned grid = static_cast<unsigned>(ceil_div64(num_tokens, kWarps));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* ub = static_cast<const __nv_bfloat16*>(up);
  const auto* db = static_cast<const __nv_bfloat16*>(down);
  const auto* gb = static_cast<const __nv_bfloat16*>(dy);
#define OMNI_DOTS(HV_) \
  expert_bwd_dots_reg_kernel<HV_><<<grid, kThreads, 0, st>>>(xb, ub, db, gb, weights, indices, num_tokens, k, hidden, num_experts, ds, cdown, dg, dx, dx_dtype == OMNI_F32, status)
  if (hidden <= 256) OMNI_DOTS(1);
  else if (hidden <= 512) OMNI_DOTS(2);
  else if (hidden <= 1024) OMNI_DOTS(4);
  else  // wider rows: registers for two resident rows would cost more occupancy than the L1 re-reads do
    expert_bwd_dots_kernel<<<grid, kThreads, 0, st>>>(xb, ub, db, gb, weights, indices, num_tokens, k, hidden, num_experts, ds, cdown, dg, status);
#undef OMNI_DOTS
  return check_launch("expert_bwd_dots_kernel");
}

namespace {
// scratch layout: int32 count, int32 list[blocks] (padded to 256 bytes), then 2 partial row pairs per block
size_t long_header_bytes(int64_t num_pairs, int block) {
  return (static_cast<size_t>(ceil_div64(num_pairs, block) + 1) * sizeof(int32_t) + 255) / 256 * 256;
}
size_t long_scratch_need(int64_t num_pairs, int hidden, int block) {
  return long_header_bytes(num_pairs, block) +
         static_cast<size_t>(2 * ceil_div64(num_pairs, block)) * 2 * static_cast<size_t>(hidden) * sizeof(float);
}
}  // namespace

// Blocks of 256 sorted positions if their partial rows fit 256 MiB, of 512 otherwise.
extern "C" size_t omni_expert_bwd_rows_scratch_bytes(int64_t num_pairs, int hidden) {
  if (num_pairs <= 0 || hidden <= 0) return 0;
  const size_t fine = long_scratch_need(num_pairs, hidden, 256);
  return fine <= kLongScratchBudget ? fine : long_scratch_need(num_pairs, hidden, kLongBlockMax);
}

extern "C" int omni_expert_bwd_rows(const void* x, const void* dy, const float* ds, const float* cdown,
                                    const int32_t* sorted_pair_ids, const int32_t* expert_ids, const int32_t* offsets,
                                    const int32_t* num_segments, const int32_t* max_segment_len, int64_t max_segments,
                                    int64_t num_tokens, int k, int hidden, int compact, void* d_up, void* d_down, int out_dtype,
                                    void* scratch, size_t scratch_bytes, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && hidden >= 8 && max_segments >= 0, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  OMNI_REQUIRE(out_dtype == OMNI_F32 || out_dtype == OMNI_BF16, "out_dtype must be OMNI_F32 or OMNI_BF16");
  OMNI_REQUIRE(max_segments < (int64_t(1) << 31), "too many segments");
  const int64_t P = num_tokens * k;
  OMNI_REQUIRE(P < (int64_t(1) << 31), "too many pairs");
  if (num_tokens == 0 || max_segments == 0) return 0;
  OMNI_REQUIRE(x && dy && ds && cdown && sorted_pair_ids && expert_ids && offsets && num_segments && d_up && d_down && status,
               "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(dy) && aligned16(d_up) && aligned16(d_down), "x, dy, d_up and d_down must be 16-byte aligned");
  OMNI_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, "scratch must be 256-byte aligned");
  OMNI_REQUIRE(scratch == nullptr || scratch_bytes >= long_scratch_need(P, hidden, kLongBlockMax),
               "scratch too small: need at least %zu bytes", long_scratch_need(P, hidden, kLongBlockMax));
  // the finest split the given scratch has room for
  int long_block = kLongBlockMax;
  for (int block = 64; scratch && block < kLongBlockMax; block *= 2)
    if (long_scratch_need(P, hidden, block) <= scratch_bytes) { long_block = block; break; }
  const unsigned grid = static_cast<unsigned>(ceil_div64(max_segments, kWarps));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* gb = static_cast<const __nv_bfloat16*>(dy);
  const bool two_level = scratch != nullptr && P > long_block;
  // without a scratch every segment, however long, is summed by one warp
  const int long_threshold = two_level ? long_block : 0x7fffffff;
  int* long_count = two_level ? static_cast<int*>(scratch) : nullptr;
  int* long_list = two_level ? long_count + 1 : nullptr;
  float* partials = two_level ? reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + long_header_bytes(P, long_block)) : nullptr;
  if (out_dtype == OMNI_F32)
    expert_bwd_rows_kernel<true><<<grid, kThreads, 0, st>>>(xb, gb, ds, cdown, sorted_pair_ids, expert_ids, offsets, num_segments,
                                                            num_tokens, k, hidden, compact, long_threshold, long_count, d_up, d_down,
                                                            status);
  else
    expert_bwd_rows_kernel<false><<<grid, kThreads, 0, st>>>(xb, gb, ds, cdown, sorted_pair_ids, expert_ids, offsets, num_segments,
                                                             num_tokens, k, hidden, compact, long_threshold, long_count, d_up, d_down,
                                                             status);
  if (int e = check_launch("expert_bwd_rows_kernel")) return e;
  if (two_level) {
    expert_bwd_rows_long_kernel<<<static_cast<unsigned>(ceil_div64(P, long_block)), long_block / 2, 0, st>>>(
        xb, gb, ds, cdown, sorted_pair_ids, offsets, num_segments, max_segment_len, P, num_tokens, k, hidden, long_block, long_count,
        long_list, partials, status);
    if (int e = check_launch("expert_bwd_rows_long_kernel")) return e;
    const dim3 rgrid(64, ceil_div(hidden, 256));
    if (out_dtype == OMNI_F32)
      expert_bwd_rows_reduce_kernel<true><<<rgrid, kThreads, 0, st>>>(partials, expert_ids, offsets, long_count, long_list, hidden,
                                                                      compact, long_block, d_up, d_down);
    else
      expert_bwd_rows_reduce_kernel<false><<<rgrid, kThreads, 0, st>>>(partials, expert_ids, offsets, long_count, long_list, hidden,
                                                                       compact, long_block, d_up, d_down);
    return check_launch("expert_bwd_rows_reduce_kernel");
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Backward of the router front: logits z [T, 2n] -> BatchNorm (batch or running statistics, folded into
// scale / shift) -> log-softmax per axis -> scores[t,j] = lp[t, ix] + lp[t, n + iy].
//   g       = scatter of dscores into the 2n log-prob columns          (as in router_bwd_kernel)
//   dzhat   = g - exp(lp) * sum_axis(g)                                 (log-softmax backward, per axis)
//   eval:     dz = scale * dzhat
//   training: dz = scale * (dzhat - mean_t(dzhat) - zhat * mean_t(dzhat * zhat)),  zhat = z * scale + shift
// router_norm_bwd_kernel does everything per token and, in training, leaves dzhat in fp32 plus per-block
// column sums of dzhat and dzhat * zhat; router_norm_bwd_sums_kernel adds the block sums in block order;
// router_norm_bwd_apply_kernel forms dz.  No atomics.  Rows of at most 512 columns (n <= 256).
// ------------------------------------------------------------------------------------------------
namespace omni {
namespace {
constexpr int kNormTokensPerWarp = 2;
constexpr int kNormMaxCols = 512;

template <int VPL>
__global__ void __launch_bounds__(kThreads) router_norm_bwd_kernel(
    const float* __restrict__ dscores, const int32_t* __restrict__ indices, const float* __restrict__ lp,
    const float* __restrict__ logits, int64_t ld_logits, const float* __restrict__ scale, const float* __restrict__ shift,
    int64_t T, int n, int k, int training, float* __restrict__ dzhat, __nv_bfloat16* __restrict__ dz,
    float* __restrict__ partial /*[blocks, 2, 2n]*/, int* __restrict__ status) {
  __shared__ float s_g[kWarps][kNormMaxCols];
  __shared__ float s_red[kWarps][2][kNormMaxCols];
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int C = 2 * n;
  float* g = s_g[warp];
  float s1[VPL], s2[VPL], sc[VPL], sh[VPL];
#pragma unroll
  for (int e = 0; e < VPL; ++e) {
    const int c = lane + 32 * e;
    s1[e] = 0.f, s2[e] = 0.f;
    sc[e] = c < C ? scale[c] : 0.f;
    sh[e] = c < C ? shift[c] : 0.f;
  }
  bool bad = false;
  const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * kNormTokensPerWarp;
  for (int i = 0; i < kNormTokensPerWarp; ++i) {
    const int64_t t = t0 + i;
    if (t >= T) break;  // warp-uniform
    for (int c = lane; c < C; c += 32) g[c] = 0.f;
    __syncwarp();
    for (int j0 = 0; j0 < k; j0 += 32) {
      const int j = j0 + lane;
      int e_ = -1;
      float d = 0.f;
      if (j < k) {
        e_ = indices[t * k + j];
        d = dscores[t * k + j];
        if (e_ < 0 || e_ >= n * n) bad = true, e_ = -1;
      }
      const int ix = e_ < 0 ? -1 : e_ / n;
      const int iy = e_ < 0 ? -1 : n + (e_ - ix * n);
      const int cnt = min(32, k - j0);
      for (int q = 0; q < cnt; ++q) {
        const int bx = __shfl_sync(FULL_MASK, ix, q), by = __shfl_sync(FULL_MASK, iy, q);
        const float bd = __shfl_sync(FULL_MASK, d, q);
        if (bx >= 0) {
          if ((bx & 31) == lane) g[bx] += bd;
          if ((by & 31) == lane) g[by] += bd;
        }
      }
    }
    __syncwarp();
    float gv[VPL];
    float sum_x = 0.f, sum_y = 0.f;
#pragma unroll
    for (int e = 0; e < VPL; ++e) {
      const int c = lane + 32 * e;
      gv[e] = c < C ? g[c] : 0.f;
      if (c < n) sum_x += gv[e];
      else sum_y += gv[e];
    }
    sum_x = warp_sum(sum_x);
    sum_y = warp_sum(sum_y);
#pragma unroll
    for (int e = 0; e < VPL; ++e) {
      const int c = lane + 32 * e;
      if (c < C) {
        const float p = __expf(lp[t * C + c]);
        const float dh = gv[e] - p * (c < n ? sum_x : sum_y);
        if (training) {
          const float zh = __fmaf_rn(logits[t * ld_logits + c], sc[e], sh[e]);
          dzhat[t * C + c] = dh;
          s1[e] += dh;
          s2[e] = __fmaf_rn(dh, zh, s2[e]);
        } else {
          dz[t * C + c] = __float2bfloat16_rn(sc[e] * dh);
        }
      }
    }
    __syncwarp();
  }
  if (training) {
#pragma unroll
    for (int e = 0; e < VPL; ++e) {
      const int c = lane + 32 * e;
      if (c < C) s_red[warp][0][c] = s1[e], s_red[warp][1][c] = s2[e];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 2 * C; idx += blockDim.x) {
      const int which = idx / C, c = idx - which * C;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) sum += s_red[w][which][c];
      partial[(static_cast<int64_t>(blockIdx.x) * 2 + which) * C + c] = sum;
    }
  }
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

// One block per 32 of the 2C column sums: thread (slice, column) adds the block partials b = slice, slice + 8, ...
// and the eight slice sums are added in slice order: same result every run, 8 x shorter loops.
__global__ void __launch_bounds__(256) router_norm_bwd_sums_kernel(const float* __restrict__ partial, int blocks, int C, int64_t T,
                                                                   float* __restrict__ means /*[2, C]*/) {
  __shared__ float s_part[8][32];
  const int col = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int idx = blockIdx.x * 32 + col;
  float sum = 0.f;
  if (idx < 2 * C) {
    const int which = idx / C, c = idx - which * C;
#pragma unroll 4
    for (int b = slice; b < blocks; b += 8) sum += partial[(static_cast<int64_t>(b) * 2 + which) * C + c];
  }
  s_part[slice][col] = sum;
  __syncthreads();
  if (slice == 0 && idx < 2 * C) {
    float tot = 0.f;
#pragma unroll
    for (int s_ = 0; s_ < 8; ++s_) tot += s_part[s_][col];
    means[idx] = tot / static_cast<float>(T);
  }
}

__global__ void __launch_bounds__(256) router_norm_bwd_apply_kernel(const float* __restrict__ dzhat, const float* __restrict__ logits,
                                                                    int64_t ld_logits, const float* __restrict__ scale,
                                                                    const float* __restrict__ shift, const float* __restrict__ means,
                                                                    int64_t T, int C, __nv_bfloat16* __restrict__ dz) {
  const int64_t total = T * C;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / C;
    const int c = static_cast<int>(i - t * C);
    const float zh = __fmaf_rn(logits[t * ld_logits + c], scale[c], shift[c]);
    dz[i] = __float2bfloat16_rn(scale[c] * (dzhat[i] - means[c] - zh * means[C + c]));
  }
}
}  // namespace
}  // namespace omni

extern "C" size_t omni_router_norm_bwd_scratch_bytes(int64_t num_tokens, int sqrt_n) {
  if (num_tokens <= 0 || sqrt_n <= 0) return 0;
  const int64_t blocks = ceil_div64(num_tokens, kWarps * kNormTokensPerWarp);
  const size_t C = 2 * static_cast<size_t>(sqrt_n);
  // dzhat [T, C] + block sums [blocks, 2, C] + means [2, C]
  return (static_cast<size_t>(num_tokens) * C + static_cast<size_t>(blocks) * 2 * C + 2 * C) * sizeof(float);
}

extern "C" int omni_router_norm_bwd(const float* dscores, const int32_t* indices, const float* log_probs, const float* logits,
                                    int64_t ld_logits, const float* bn_scale, const float* bn_shift, int64_t num_tokens, int sqrt_n,
                                    int k, int training, void* dlogits, void* scratch, size_t scratch_bytes, int32_t* status,
                                    void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 0, "bad sizes");
  OMNI_REQUIRE(sqrt_n >= 1 && 2 * sqrt_n <= kNormMaxCols, "omni_router_norm_bwd handles sqrt_n <= %d, got %d", kNormMaxCols / 2, sqrt_n);
  OMNI_REQUIRE(ld_logits >= 2 * sqrt_n, "ld_logits %lld < 2*sqrt_n", static_cast<long long>(ld_logits));
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(log_probs && logits && bn_scale && bn_shift && dlogits && status && (k == 0 || (dscores && indices)), "NULL argument");
  OMNI_REQUIRE(!training || (scratch && scratch_bytes >= omni_router_norm_bwd_scratch_bytes(num_tokens, sqrt_n)),
               "scratch too small: need %zu bytes", omni_router_norm_bwd_scratch_bytes(num_tokens, sqrt_n));
  const int C = 2 * sqrt_n;
  const int64_t blocks = ceil_div64(num_tokens, kWarps * kNormTokensPerWarp);
  OMNI_REQUIRE(blocks < (int64_t(1) << 31), "too many tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* dzhat = training ? static_cast<float*>(scratch) : nullptr;
  float* partial = training ? dzhat + num_tokens * C : nullptr;
  float* means = training ? partial + blocks * 2 * C : nullptr;
  __nv_bfloat16* dz = static_cast<__nv_bfloat16*>(dlogits);
  if (C <= 128)
    router_norm_bwd_kernel<4><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(dscores, indices, log_probs, logits, ld_logits, bn_scale,
                                                                              bn_shift, num_tokens, sqrt_n, k, training, dzhat, dz,
                                                                              partial, status);
  else
    router_norm_bwd_kernel<16><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(dscores, indices, log_probs, logits, ld_logits,
                                                                               bn_scale, bn_shift, num_tokens, sqrt_n, k, training,
                                                                               dzhat, dz, partial, status);
  if (int e = check_launch("router_norm_bwd_kernel")) return e;
  if (!training) return 0;
  router_norm_bwd_sums_kernel<<<ceil_div(2 * C, 32), 256, 0, st>>>(partial, static_cast<int>(blocks), C, num_tokens, means);
  if (int e = check_launch("router_norm_bwd_sums_kernel")) return e;
  const int64_t total = num_tokens * C;
  const int64_t want = ceil_div64(total, 256);
  router_norm_bwd_apply_kernel<<<static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8), 256, 0, st>>>(
      dzhat, logits, ld_logits, bn_scale, bn_shift, means, num_tokens, C, dz);
  return check_launch("router_norm_bwd_apply_kernel");
}
