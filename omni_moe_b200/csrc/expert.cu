// Routed experts: y[t] = sum_j w[t,j] * silu(x[t] . Up[e[t,j]]) * Down[e[t,j]].
//
// expert_coef_kernel    walks the pairs in expert order (the output of the scheduler).  A warp owns
//                       a run of consecutive sorted positions, keeps the current expert's Up row in
//                       registers and only refetches it when the expert changes, so each Up row
//                       leaves HBM once; the token rows x[t] are re-read per pair, but x is k/4
//                       times smaller than the touched part of the table and lives in L2.
//                       Output: c[pair] = w * silu(x . up), fp32, at the pair's original place.
// expert_combine_kernel is token-centric: a warp owns (token, column slab), loops over the token's
//                       k pairs and accumulates c * Down[e] in fp32 registers, then writes the
//                       row once.  No atomics, no zero fill, fixed summation order.
// All row traffic is 128-bit loads, a warp reading 512 contiguous bytes per instruction.
#include <cstdlib>

#include "router_select.cuh"

namespace omni {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRun = 16;  // sorted positions per warp in expert_coef_kernel
constexpr int kCombineThreads = 128;
constexpr int kHot = 64;  // experts whose products with every token come from a dense GEMM (omni_expert_coef_hot)

__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
  const uint32_t* pa = reinterpret_cast<const uint32_t*>(&a);
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = bf16x2_to_float2(pa[i]), fb = bf16x2_to_float2(pb[i]);
    acc = __fmaf_rn(fa.x, fb.x, acc);
    acc = __fmaf_rn(fa.y, fb.y, acc);
  }
  return acc;
}

// Packed fp32 pairs: Blackwell issues two FMAs per instruction on a register pair (fma.rn.f32x2), and
// a bf16x2 word unpacks into exactly such a pair, so a row element costs 1 unpack op + 1/2 FMA issue.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// x row unpacked to fp32 pairs once per token: xf[v][q] = elements (2q, 2q+1) of vector v.
template <int HV>
__device__ __forceinline__ void unpack_row(const uint4 (&xv)[HV], float2 (&xf)[HV][4]) {
#pragma unroll
  for (int v = 0; v < HV; ++v) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&xv[v]);
#pragma unroll
    for (int q = 0; q < 4; ++q) xf[v][q] = bf16x2_to_float2(p[q]);
  }
}
__device__ __forceinline__ float2 dot8p(const float2 (&a)[4], const uint4& b, float2 acc) {
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc = fma2(a[i], bf16x2_to_float2(pb[i]), acc);
  return acc;
}
__device__ __forceinline__ void axpy8p(float c, const uint4& d, float2 (&acc)[4]) {
  const uint32_t* pd = reinterpret_cast<const uint32_t*>(&d);
  const float2 c2 = make_float2(c, c);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = fma2(c2, bf16x2_to_float2(pd[i]), acc[i]);
}

// HV = 128-bit vectors per lane; covers HV * 256 columns per slab.
template <int HV>
__global__ void __launch_bounds__(kThreads) expert_coef_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up, const float* __restrict__ weights,
    const int* __restrict__ perm, const int* __restrict__ sorted_experts, const int* __restrict__ pair_tokens,
    int64_t P, int64_t T, int k, int H, int64_t N, float* __restrict__ coef, int* status,
    const int* __restrict__ hot_ids, const float* __restrict__ hot_dots) {
  // weights == nullptr: the raw dot products x . Up[e] are written instead of w * silu(x . Up[e]) (a GPU that holds a
  // column slice of the tables: the partial products of all slices are added before the activation).
  // pair_tokens == nullptr: pairs come from a [T, k] routing table, pair p belongs to token p / k.
  // Otherwise pair p belongs to token pair_tokens[p] (pairs received from other GPUs).
  // hot_ids != nullptr: kHot ascending expert ids (padded with INT_MAX) followed by their count; the dot
  // products of those experts' Up rows with every token are already in hot_dots [T, kHot] (a dense GEMM),
  // so pairs on them gather nothing.
  const int lane = lane_id();
  const int64_t w0 = (static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5)) * kRun;
  if (w0 >= P) return;
  // lane i < kRun carries the metadata of sorted position w0 + i
  int my_pair = -1, my_e = -1, my_t = -1;
  float my_g = 0.f;
  if (lane < kRun && w0 + lane < P) {
    my_pair = perm[w0 + lane];
    my_e = sorted_experts[w0 + lane];
    if (my_pair >= 0 && my_pair < P) {
      my_g = weights ? weights[my_pair] : 1.f;
      my_t = pair_tokens ? pair_tokens[my_pair] : my_pair / k;
    }
  }
  const int count = (P - w0 < kRun) ? static_cast<int>(P - w0) : kRun;
  unsigned hot_mask = 0;
  if (hot_ids != nullptr && __ldg(hot_ids + kHot) > 0) {
    int col = -1;
    if (my_t >= 0 && my_t < T && my_e >= 0 && my_e < N) {
      int lo = 0;  // lower bound among kHot ascending ids
#pragma unroll
      for (int step = kHot / 2; step > 0; step >>= 1)
        if (__ldg(hot_ids + lo + step - 1) < my_e) lo += step;
      if (__ldg(hot_ids + lo) == my_e) col = lo;
    }
    if (col >= 0) {
      const float d = __ldg(hot_dots + static_cast<int64_t>(my_t) * kHot + col);
      coef[my_pair] = weights ? my_g * silu(d) : d;
    }
    hot_mask = __ballot_sync(FULL_MASK, col >= 0);
    if (hot_mask == (count >= 32 ? FULL_MASK : ((1u << count) - 1u))) return;
  }
  const int slabs = ceil_div(H, HV * 256);
  // Up rows stream through once; the token rows are gathered k times and should keep their place in L2
  const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
  int cur_e = -1;
  uint4 row[HV];
  bool bad_e = false, bad_t = false;
  if (slabs == 1) {
    // Common case, a whole row per lane set: the token row of pair i+1 is requested before pair i is
    // computed, so a warp always has two gathers in flight.
    const int c0 = lane * 8;
    auto fetch_x = [&](int i, uint4 (&dst)[HV]) {
      const int64_t t = __shfl_sync(FULL_MASK, my_t, i & 31);
      // never predicated (a predicated load lands in a conditional block and is not in flight with its neighbours):
      // a pair that is skipped reads row 0, a column past the end re-reads column 0 and meets a zero of the Up row
      const bool ok = t >= 0 && t < T && !((hot_mask >> i) & 1u);
      const __nv_bfloat16* xr = x + (ok ? t : 0) * H;
#pragma unroll
      for (int v = 0; v < HV; ++v) {
        const int c = c0 + v * 256;
        dst[v] = ldg128_hint(xr + (c < H ? c : 0), pol_keep);
      }
    };
    // one pair: the Up row of its expert (refetched only when the expert changes) against the token row xv
    auto one_pair = [&](int i, const uint4 (&xv)[HV]) {
      const int pair = __shfl_sync(FULL_MASK, my_pair, i);
      const int e = __shfl_sync(FULL_MASK, my_e, i);
      const float g = __shfl_sync(FULL_MASK, my_g, i);
      const int64_t t = __shfl_sync(FULL_MASK, my_t, i);
      const bool e_ok = e >= 0 && e < N, t_ok = pair >= 0 && t >= 0 && t < T;
      if ((hot_mask >> i) & 1u) {
        // done above from the dense products
      } else if (!e_ok) {
        bad_e = true;
        if (lane == 0 && pair >= 0 && pair < P) coef[pair] = 0.f;
      } else if (!t_ok) {
        bad_t = true;
      } else {
        if (e != cur_e) {
#pragma unroll
          for (int v = 0; v < HV; ++v) {
            const int c = c0 + v * 256;
            row[v] = c < H ? ldg128_hint(up + static_cast<int64_t>(e) * H + c, pol_stream) : make_uint4(0, 0, 0, 0);
          }
          cur_e = e;
        }
        float acc = 0.f;
#pragma unroll
        for (int v = 0; v < HV; ++v) acc = dot8(xv[v], row[v], acc);
        acc = warp_sum(acc);
        if (lane == 0) coef[pair] = weights ? g * silu(acc) : acc;
      }
    };
    {
      uint4 xcur[HV], xnext[HV];
      fetch_x(0, xcur);
      for (int i = 0; i < count; ++i) {
        fetch_x(i + 1, xnext);  // past the end of the run: lane i + 1 carries no token, row 0 is read (an L1 hit) and dropped
        one_pair(i, xcur);
#pragma unroll
        for (int v = 0; v < HV; ++v) xcur[v] = xnext[v];
      }
    }
  } else
  for (int i = 0; i < count; ++i) {
    const int pair = __shfl_sync(FULL_MASK, my_pair, i);
    const int e = __shfl_sync(FULL_MASK, my_e, i);
    const float g = __shfl_sync(FULL_MASK, my_g, i);
    const int64_t t = __shfl_sync(FULL_MASK, my_t, i);
    if ((hot_mask >> i) & 1u) continue;
    if (e < 0 || e >= N) { bad_e = true; if (lane == 0 && pair >= 0 && pair < P) coef[pair] = 0.f; continue; }
    if (pair < 0 || t < 0 || t >= T) { bad_t = true; continue; }
    float acc = 0.f;
    for (int s = 0; s < slabs; ++s) {
      const int c0 = s * HV * 256 + lane * 8;
      uint4 xv[HV];
#pragma unroll
      for (int v = 0; v < HV; ++v) {
        const int c = c0 + v * 256;
        xv[v] = c < H ? ldg128_hint(x + t * H + c, pol_keep) : make_uint4(0, 0, 0, 0);
      }
      if (e != cur_e || slabs > 1) {
#pragma unroll
        for (int v = 0; v < HV; ++v) {
          const int c = c0 + v * 256;
          row[v] = c < H ? ldg128_hint(up + static_cast<int64_t>(e) * H + c, pol_stream) : make_uint4(0, 0, 0, 0);
        }
        cur_e = e;
      }
#pragma unroll
      for (int v = 0; v < HV; ++v) acc = dot8(xv[v], row[v], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) coef[pair] = weights ? g * silu(acc) : acc;
  }
  if (bad_e && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
  if (bad_t && lane == 0) atomicOr(status, OMNI_ST_BAD_TOKEN_INDEX);
}

// Picks the experts that own long runs of the sorted pair list and copies their Up rows side by side, so that
// one dense GEMM gives their products with every token.  An expert qualifies when it fills a whole aligned window
// of `tau` sorted positions (any run of 2 * tau - 1 pairs does, none shorter than tau does); the first kHot such
// experts in sorted order are taken.  Every block repeats the scan (a few thousand loads) and block b then copies
// row b, so the list needs no second launch; unused slots get the id INT_MAX and a zero row.  The choice depends
// on the sorted list only, never on timing.  A list that is not sorted yields fewer or repeated ids, which costs
// speed only: the coefficient kernel takes a dense product only where the id matches exactly.
__global__ void __launch_bounds__(kThreads) hot_rows_kernel(const int* __restrict__ sorted_experts, int64_t P, int tau,
                                                            int64_t N, const __nv_bfloat16* __restrict__ up, int H,
                                                            int* __restrict__ hot_ids, __nv_bfloat16* __restrict__ hot_rows) {
  __shared__ int s_ids[kHot];
  __shared__ int s_warp[kWarps];
  __shared__ int s_count;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < kHot) s_ids[tid] = 0x7fffffff;
  if (tid == 0) s_count = 0;
  __syncthreads();
  const int64_t windows = P / tau;
  for (int64_t base = 0; base < windows; base += kThreads) {
    const int64_t j = base + tid;
    int e = -1;
    bool first_full = false;
    if (j < windows) {
      e = sorted_experts[j * tau];
      const int last = sorted_experts[(j + 1) * tau - 1];
      const int before = j > 0 ? sorted_experts[(j - 1) * tau] : -1;
      first_full = e == last && e >= 0 && e < N && !(j > 0 && before == e);
    }
    const unsigned m = __ballot_sync(FULL_MASK, first_full);
    if (lane == 0) s_warp[warp] = __popc(m);
    __syncthreads();
    int pos = s_count + __popc(m & ((1u << lane) - 1u));
    int total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      if (w < warp) pos += s_warp[w];
      total += s_warp[w];
    }
    if (first_full && pos < kHot) s_ids[pos] = e;
    __syncthreads();
    if (tid == 0) s_count += total;
    __syncthreads();
    if (s_count >= kHot) break;
  }
  const int b = blockIdx.x;
  const int id = s_ids[b];
  if (b == 0 && tid < kHot) hot_ids[tid] = s_ids[tid];
  if (b == 0 && tid == kHot) hot_ids[kHot] = min(s_count, kHot);
  uint4* dst = reinterpret_cast<uint4*>(hot_rows + static_cast<int64_t>(b) * H);
  const uint4* src = reinterpret_cast<const uint4*>(up + static_cast<int64_t>(id == 0x7fffffff ? 0 : id) * H);
  for (int c = tid; c < H / 8; c += kThreads) dst[c] = id == 0x7fffffff ? make_uint4(0, 0, 0, 0) : __ldg(src + c);
}

// Token-centric fusion of the two kernels above for tables that stay resident in L2: a warp owns one
// token, holds its x row in registers and walks its k pairs with the Up and the Down row of UNR
// pairs in flight; dot, SiLU, weight and the accumulation of c * Down happen in registers, nothing
// is scheduled and no coefficient round-trips through memory.  Every row is read k times in total,
// which is free while both tables live in L2 and wasteful once they do not (then the expert-ordered
// pair of kernels above reads each Up row from HBM once).
// Walks up to 32 pairs of one token: lane l carries pair l (expert my_e or -1, routing weight my_w).
// The Up and Down rows of UNR pairs are in flight at a time; dot, SiLU, weight and the accumulation
// of c * Down stay in registers.  coef_row, if not null, receives the cnt coefficients.
template <int HV>
__device__ __forceinline__ void gather_pairs(int my_e, float my_w, int cnt, int c0, int H, const float2 (&xf)[HV][4],
                                             const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
                                             float2 (&acc)[HV][4], float* coef_row) {
  constexpr int UNR = HV >= 8 ? 1 : 2;
  const int lane = lane_id();
  for (int j = 0; j < cnt; j += UNR) {
    uint4 uv[UNR][HV], dv[UNR][HV];
    float w[UNR];
    bool on[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int e = __shfl_sync(FULL_MASK, my_e, (j + u) & 31);
      w[u] = __shfl_sync(FULL_MASK, my_w, (j + u) & 31);
      on[u] = (j + u < cnt) && e >= 0;
#pragma unroll
      for (int v = 0; v < HV; ++v) {
        const int col = c0 + v * 256;
        const bool ld = on[u] && col < H;
        uv[u][v] = ld ? ldg128(up + static_cast<int64_t>(e) * H + col) : make_uint4(0, 0, 0, 0);
        dv[u][v] = ld ? ldg128(down + static_cast<int64_t>(e) * H + col) : make_uint4(0, 0, 0, 0);
      }
    }
    float dot[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      float2 d2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int v = 0; v < HV; ++v) d2 = dot8p(xf[v], uv[u][v], d2);
      dot[u] = d2.x + d2.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < UNR; ++u) dot[u] += __shfl_xor_sync(FULL_MASK, dot[u], o);
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const float c = on[u] ? w[u] * silu(dot[u]) : 0.f;
      if (coef_row && lane == 0 && j + u < cnt) coef_row[j + u] = c;
#pragma unroll
      for (int v = 0; v < HV; ++v) axpy8p(c, dv[u][v], acc[v]);
    }
  }
}

// Adds the optional residual row and writes one output row (fp32 or bf16).
template <int HV, bool OUT_F32>
__device__ __forceinline__ void store_row(float (&acc)[HV][8], int64_t t, int c0, int H, const void* residual, void* y);

// the same for accumulators kept as fp32 pairs
template <int HV, bool OUT_F32>
__device__ __forceinline__ void store_row(float2 (&acc2)[HV][4], int64_t t, int c0, int H, const void* residual, void* y) {
  float acc[HV][8];
#pragma unroll
  for (int v = 0; v < HV; ++v)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[v][2 * q] = acc2[v][q].x, acc[v][2 * q + 1] = acc2[v][q].y;
  store_row<HV, OUT_F32>(acc, t, c0, H, residual, y);
}

template <int HV, bool OUT_F32>
__device__ __forceinline__ void store_row(float (&acc)[HV][8], int64_t t, int c0, int H, const void* residual, void* y) {
#pragma unroll
  for (int v = 0; v < HV; ++v) {
    const int col = c0 + v * 256;
    if (col >= H) continue;
    const int64_t o = t * H + col;
    if (OUT_F32) {
      float4 a = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
      float4 b = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
      if (residual) {
        // plain loads: residual may be the output buffer itself (in-place add)
        const float4 ra = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(residual) + o);
        const float4 rb = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(residual) + o + 4);
        a.x += ra.x, a.y += ra.y, a.z += ra.z, a.w += ra.w;
        b.x += rb.x, b.y += rb.y, b.z += rb.z, b.w += rb.w;
      }
      float* yo = reinterpret_cast<float*>(y) + o;
      *reinterpret_cast<float4*>(yo) = a;
      *reinterpret_cast<float4*>(yo + 4) = b;
    } else {
      if (residual) {
        const uint4 rv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(residual) + o);
        const uint32_t* pr = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = bf16x2_to_float2(pr[q]);
          acc[v][2 * q] += f.x;
          acc[v][2 * q + 1] += f.y;
        }
      }
      uint4 o4;
      o4.x = float2_to_bf16x2(acc[v][0], acc[v][1]);
      o4.y = float2_to_bf16x2(acc[v][2], acc[v][3]);
      o4.z = float2_to_bf16x2(acc[v][4], acc[v][5]);
      o4.w = float2_to_bf16x2(acc[v][6], acc[v][7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(y) + o) = o4;
    }
  }
}

// Token-centric combine.  A warp owns (token, column slab of HV * 256 columns) and accumulates c * Down[e] over the
// token's pairs in fp32 registers, four rows in flight per step, then writes the slab once.
//   offsets == nullptr: the pairs of token t are entries [t * k, (t + 1) * k) of experts / coef (a [T, k] routing table);
//   otherwise: entries [offsets[t], offsets[t + 1]) of a pair list grouped by token (a GPU that holds a slice of the
//   tables and received only the pairs routed to its rows).
template <int HV, bool OUT_F32>
__global__ void __launch_bounds__(kCombineThreads) expert_combine_kernel(
    const __nv_bfloat16* __restrict__ down, const float* __restrict__ coef, const int* __restrict__ experts,
    const int* __restrict__ offsets, int64_t T, int k, int H, int64_t N, int slabs, const void* residual, void* y,
    int* status) {
  const int lane = lane_id();
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * (kCombineThreads / 32) + (threadIdx.x >> 5);
  const int64_t t = wid / slabs;
  const int slab = static_cast<int>(wid - t * slabs);
  if (t >= T) return;
  const int c0 = slab * HV * 256 + lane * 8;
  float2 acc[HV][4];
#pragma unroll
  for (int v = 0; v < HV; ++v)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[v][q] = make_float2(0.f, 0.f);
  bool bad = false;
  const int64_t lo = offsets ? static_cast<int64_t>(offsets[t]) : t * k;
  const int64_t hi = offsets ? static_cast<int64_t>(offsets[t + 1]) : lo + k;
  for (int64_t j0 = lo; j0 < hi; j0 += 32) {
    // lane l carries pair j0 + l of this token
    int my_e = -1;
    float my_c = 0.f;
    if (j0 + lane < hi) {
      my_e = experts[j0 + lane];
      my_c = coef[j0 + lane];
      if (my_e < 0 || my_e >= N) { bad = true; my_e = -1; }
    }
    const int cnt = static_cast<int>(hi - j0 < 32 ? hi - j0 : 32);
    constexpr int UNR = 4;  // rows in flight per step
    for (int j = 0; j < cnt; j += UNR) {
      uint4 dv[UNR][HV];
      float c[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int e = __shfl_sync(FULL_MASK, my_e, (j + u) & 31);
        c[u] = __shfl_sync(FULL_MASK, my_c, (j + u) & 31);
        const bool on = (j + u < cnt) && e >= 0;
        if (!on) c[u] = 0.f;
        // never predicated: a pair that is absent or invalid reads row 0 with coefficient 0, a column past the row's
        // end re-reads column 0 (its result is not stored).  Predicated loads here end up in conditional blocks, which
        // keeps the rows of a step from being in flight together (8 rows per step ran 2.7 times slower than 4).
        const __nv_bfloat16* rowp = down + static_cast<int64_t>(on ? e : 0) * H;
#pragma unroll
        for (int v = 0; v < HV; ++v) {
          const int col = c0 + v * 256;
          dv[u][v] = ldg128(rowp + (col < H ? col : 0));
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int v = 0; v < HV; ++v) axpy8p(c[u], dv[u][v], acc[v]);
    }
  }
  store_row<HV, OUT_F32>(acc, t, c0, H, residual, y);
  if (bad && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

template <int HV>
__device__ __forceinline__ void load_x_row(const __nv_bfloat16* __restrict__ x, int64_t t, int c0, int H, uint4 (&xv)[HV],
                                           float2 (&acc)[HV][4]) {
#pragma unroll
  for (int v = 0; v < HV; ++v) {
    const int col = c0 + v * 256;
    xv[v] = col < H ? ldg128(x + t * H + col) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[v][q] = make_float2(0.f, 0.f);
  }
}

template <int HV, bool OUT_F32>
__global__ void __launch_bounds__(kThreads) expert_fused_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
    const float* __restrict__ weights, const int* __restrict__ indices, int64_t T, int k, int H, int64_t N,
    const void* residual, void* y, float* __restrict__ coef, int* status) {
  const int lane = lane_id();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (t >= T) return;
  const int c0 = lane * 8;
  uint4 xv[HV];
  float2 acc[HV][4], xf[HV][4];
  load_x_row<HV>(x, t, c0, H, xv, acc);
  unpack_row<HV>(xv, xf);
  bool bad = false;
  for (int j0 = 0; j0 < k; j0 += 32) {
    int my_e = -1;
    float my_w = 0.f;
    if (j0 + lane < k) {
      my_e = indices[t * k + j0 + lane];
      my_w = weights[t * k + j0 + lane];
      if (my_e < 0 || my_e >= N) { bad = true; my_e = -1; }
    }
    gather_pairs<HV>(my_e, my_w, min(32, k - j0), c0, H, xf, up, down, acc, coef ? coef + t * k + j0 : nullptr);
  }
  store_row<HV, OUT_F32>(acc, t, c0, H, residual, y);
  if (bad && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

// Router selection and routed experts in one kernel: the warp that owns a token first picks its k
// experts from the token's router logits (BatchNorm fold, log-softmax, product-key top-k: see
// router_select.cuh) and then gathers their rows.  The selection is arithmetic on a few hundred
// values and runs in the shadow of other warps' row gathers, so it costs no extra pass over
// memory and no launch.  Lane r % 32 ends the selection holding rank r, which is exactly the
// layout gather_pairs wants.
template <int HV, int VPL, int CPL>
__global__ void __launch_bounds__(kThreads, HV <= 4 ? 2 : 1) expert_routed_kernel(
    const sel::TopkArgs a, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up,
    const __nv_bfloat16* __restrict__ down, int H, int64_t N, const void* residual, void* y) {
  __shared__ sel::WarpScratch<VPL, CPL> s_warp[kWarps];
  __shared__ sel::RegionTable s_region;
  sel::build_region_table(s_region, a.kk, a.k, kWarps);
  pdl_wait();  // everything above is shared-memory set-up; the logits and y come from earlier kernels
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (t >= a.T) return;
  const int c0 = lane * 8, k = a.k;
  uint32_t rkey[sel::kMaxK / 32], rflat[sel::kMaxK / 32];
  sel::select_token<VPL, CPL, true>(a, t, s_warp[warp], s_region.cell, rkey, rflat);
  // k <= 32 here (checked by the host), so rank r lives in lane r
  int my_e = -1;
  float my_w = 0.f;
  if (lane < k) {
    const float sc = key_to_float(rkey[0]);
    my_w = expf(sc);
    my_e = static_cast<int>(rflat[0]);  // < sqrt_n^2 <= N by construction
    const int64_t o = t * k + lane;
    if (a.scores) a.scores[o] = sc;
    if (a.indices) reinterpret_cast<int32_t*>(a.indices)[o] = my_e;
    if (a.weights) a.weights[o] = my_w;
    if (my_e >= N) my_e = -1;
  }
  float2 acc[HV][4], xf[HV][4];
  {
    uint4 xv[HV];
    load_x_row<HV>(x, t, c0, H, xv, acc);
    unpack_row<HV>(xv, xf);
  }
  gather_pairs<HV>(my_e, my_w, k, c0, H, xf, up, down, acc, nullptr);
  store_row<HV, false>(acc, t, c0, H, residual, y);
}

// mma.sync m16n8k16, bf16 operands, fp32 accumulate: D (16 x 8) += A (16 x 16, row major) * B (16 x 8, column major).
// Fragments (g = lane / 4, t = lane % 4): a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1], a2 = A[g][2t+8, 2t+9],
// a3 = A[g+8][2t+8, 2t+9]; b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g]; d0, d1 = D[g][2t, 2t+1], d2, d3 = D[g+8][2t, 2t+1].
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// L2 prefetch of a contiguous range: nothing reaches the SM.
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Router selection + routed experts, for rows of exactly HV * 256 columns (256, 512 or 1024) and k <= 32: the k dot
// products of a token on the tensor cores, and the two stages of a token handed out dynamically.
//
// Dots.  The 16 x H block "Up rows of 16 selected experts" is the A operand of mma.sync.m16n8k16 and the token's x
// row, repeated in every column, the B operand, so D[e][.] = x . Up[e].  No shared-memory staging of the rows is
// needed: the contraction index may be permuted freely as long as both operands agree, so lane (g, t) simply loads 32
// contiguous bytes (16 columns) of row g and of row g + 8 - four lanes cover a whole 128-byte line - and uses the
// eight 32-bit words, two at a time, as (a0, a2) / (a1, a3) of four MMAs; the matching B words are the same 32 bytes
// of the x row, which the warp keeps in shared memory (every lane group reads them: a broadcast).  Per 16 bytes of
// an Up row this is half a load and half an MMA instead of eight unpack operations and four packed FMAs.
// The k-term sum of Down rows stays on the CUDA cores (its contraction index is the row index, which mma.sync
// could only take through a transposing copy in shared memory); every lane owns 8 contiguous columns per 256.
// Experts that are not valid (index >= N, ranks beyond k) are replaced by a valid row with weight 0, so no load in
// the loops is predicated.
//
// Scheduling.  The selection of a token is arithmetic with long dependency chains (~5 us for a warp) and the gather
// is bound by the latency and the bandwidth of L2 (~8 us for a warp).  With one token per warp, both in a row, the
// warps of an SM run in step - everybody selects, then everybody gathers - and a token count that is not a multiple
// of the resident warps leaves most of them idle for a whole second round.  Here one block per SM owns a
// contiguous range of tokens and its 16 warps take tasks from two counters in shared memory: "gather the next
// token whose selection is finished" if there is one, otherwise "select the next unselected token".  The memory
// system stays busy while other warps select, and the work is spread over the warps in units of half a token.
#ifdef OMNI_TUNING
}  // namespace
__device__ long long g_dyn_prof[160 * 16 * 8];  // tuning builds only: per-warp clocks by part
namespace {
#define OMNI_TIC(v) const long long v = clock64()
#define OMNI_TOC(acc, v) acc += clock64() - v
#else
#define OMNI_TIC(v)
#define OMNI_TOC(acc, v)
#endif
constexpr int kDynWarps = 16;
constexpr int kDynTokens = 32;  // tokens per block at most
constexpr uint32_t kDynSpinLimit = 1u << 20;

struct RoutedRecord {
  int e[32];    // expert row by rank (a valid row wherever the weight is 0)
  float w[32];  // routing weight by rank
};

// Lane r brings the expert row and the routing weight of rank r (a valid row with weight 0 where there is none).
template <int HV>
__device__ __forceinline__ void gather_token_tc(int my_e, float my_w, int k, int64_t t, const __nv_bfloat16* __restrict__ x,
                                                const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
                                                uint4* xrow, const void* residual, void* y, long long* pr) {
  constexpr int H = HV * 256;
  const int lane = lane_id();
  const int gq = lane >> 2, tq = lane & 3;
  OMNI_TIC(cx);
  uint4 xv[HV];
#pragma unroll
  for (int v = 0; v < HV; ++v) xv[v] = ldg128(x + t * H + v * 256 + lane * 8);
  __syncwarp();  // the previous user of xrow (this warp) is done with it
#pragma unroll
  for (int v = 0; v < HV; ++v) xrow[v * 32 + lane] = xv[v];
  __syncwarp();
  float2 acc[HV][4];
#pragma unroll
  for (int v = 0; v < HV; ++v)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[v][q] = make_float2(0.f, 0.f);
  const uint4* xs = xrow + 2 * tq;
  OMNI_TOC(pr[0], cx);
  for (int base = 0; base < k; base += 16) {
    OMNI_TIC(cd);
    // ---- dots of the 16 experts base .. base + 15: rows gq and gq + 8 of the tile belong to this lane group
    const int e_a = __shfl_sync(FULL_MASK, my_e, (base + gq) & 31), e_b = __shfl_sync(FULL_MASK, my_e, (base + gq + 8) & 31);
    const float w_a = __shfl_sync(FULL_MASK, my_w, (base + gq) & 31), w_b = __shfl_sync(FULL_MASK, my_w, (base + gq + 8) & 31);
    const uint4* ra = reinterpret_cast<const uint4*>(up + static_cast<int64_t>(e_a) * H) + 2 * tq;
    const uint4* rb = reinterpret_cast<const uint4*>(up + static_cast<int64_t>(e_b) * H) + 2 * tq;
    float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
    for (int s = 0; s < H / 64; ++s) {  // 64 columns per step: 16 per lane of a group
      const uint4 a0 = __ldg(ra + 8 * s), a1 = __ldg(ra + 8 * s + 1);
      const uint4 b0 = __ldg(rb + 8 * s), b1 = __ldg(rb + 8 * s + 1);
      const uint4 x0 = xs[8 * s], x1 = xs[8 * s + 1];
      mma_bf16_16816(d[0], a0.x, b0.x, a0.y, b0.y, x0.x, x0.y);
      mma_bf16_16816(d[1], a0.z, b0.z, a0.w, b0.w, x0.z, x0.w);
      mma_bf16_16816(d[0], a1.x, b1.x, a1.y, b1.y, x1.x, x1.y);
      mma_bf16_16816(d[1], a1.z, b1.z, a1.w, b1.w, x1.z, x1.w);
    }
    // every column of D holds the same dot: d[.][0] is expert base + gq, d[.][2] expert base + gq + 8
    const float c_a = w_a * silu(d[0][0] + d[1][0]);
    const float c_b = w_b * silu(d[0][2] + d[1][2]);
    OMNI_TOC(pr[1], cd);
    OMNI_TIC(ca_);
    // ---- y += c[j] * Down[e[j]], UNR rows in flight
    constexpr int UNR = HV >= 4 ? 4 : 8;  // 16 x 16-byte loads per lane in flight
    const int cnt = min(16, k - base);
    for (int j = 0; j < cnt; j += UNR) {
      uint4 dv[UNR][HV];
      float c[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int jj = j + u;  // may run past cnt (but stays below 16): those ranks carry weight 0 and a valid row
        const int e = __shfl_sync(FULL_MASK, my_e, (base + jj) & 31);
        const float ca = __shfl_sync(FULL_MASK, c_a, (jj & 7) * 4), cb = __shfl_sync(FULL_MASK, c_b, (jj & 7) * 4);
        c[u] = (jj & 8) ? cb : ca;
        if (jj >= cnt) c[u] = 0.f;  // ranks of the next tile, if any, are not part of this one
        const uint4* row = reinterpret_cast<const uint4*>(down + static_cast<int64_t>(e) * H) + lane;
#pragma unroll
        for (int v = 0; v < HV; ++v) dv[u][v] = __ldg(row + v * 32);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int v = 0; v < HV; ++v) axpy8p(c[u], dv[u][v], acc[v]);
    }
    OMNI_TOC(pr[2], ca_);
  }
  OMNI_TIC(cs);
  store_row<HV, false>(acc, t, lane * 8, H, residual, y);
  OMNI_TOC(pr[3], cs);
}

// The routed experts of tokens whose routing is already known (indices / weights in memory), one warp per token, dots
// on the tensor cores as above.  bf16 output; the caller's residual is added.
template <int HV>
__global__ void __launch_bounds__(kThreads, 2) expert_fused_tc_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
    const float* __restrict__ weights, const int* __restrict__ indices, int64_t T, int k, int64_t N, const void* residual,
    void* y, int* status) {
  constexpr int H = HV * 256;
  __shared__ __align__(16) uint4 s_x[kWarps][HV * 32];
  if (threadIdx.x < 2) {  // this block's share of both tables into L2, as a stream (they are weights: no dependency)
    const int64_t total = N * H * 2;
    const int64_t share = ((total + gridDim.x - 1) / gridDim.x + 255) & ~int64_t(255);
    const int64_t lo = share * blockIdx.x, hi = min(total, lo + share);
    const unsigned char* tab = reinterpret_cast<const unsigned char*>(threadIdx.x == 0 ? up : down);
    for (int64_t o = lo; o < hi; o += 16384) l2_prefetch_bulk(tab + o, static_cast<uint32_t>(min(int64_t(16384), hi - o)));
  }
  pdl_wait();  // the routing and y come from earlier kernels
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (t >= T) return;
  int my_e = 0;
  float my_w = 0.f;
  bool valid = false, bad = false;
  if (lane < k) {
    my_e = indices[t * k + lane];
    my_w = weights[t * k + lane];
    valid = my_e >= 0 && my_e < N;
    bad = !valid;
  }
  const unsigned ok_mask = __ballot_sync(FULL_MASK, valid);
  const int safe = ok_mask ? __shfl_sync(FULL_MASK, my_e, __ffs(ok_mask) - 1) : 0;  // a row that exists
  if (!valid) my_e = safe, my_w = 0.f;
  long long pr[8];
  gather_token_tc<HV>(my_e, my_w, k, t, x, up, down, s_x[warp], residual, y, pr);
  if (__any_sync(FULL_MASK, bad) && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

template <int HV, int VPL, int CPL>
__global__ void __launch_bounds__(kDynWarps * 32, 1) expert_routed_dyn_kernel(
    const sel::TopkArgs a, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up,
    const __nv_bfloat16* __restrict__ down, int64_t N, int tok_per_block, const void* residual, void* y, int* status) {
  constexpr int H = HV * 256;
  using Scratch = sel::WarpScratch<VPL, CPL, 32>;  // k <= 32: at most 32 sub-keys kept per axis
  __shared__ Scratch s_warp[kDynWarps];
  __shared__ sel::RegionTable s_region;
  __shared__ int s_sel_next, s_gat_next, s_abort;
  __shared__ int s_ready[kDynTokens];
  extern __shared__ __align__(16) unsigned char s_dyn[];
  uint4* s_x = reinterpret_cast<uint4*>(s_dyn);  // [kDynWarps][HV * 32]
  RoutedRecord* s_rec = reinterpret_cast<RoutedRecord*>(s_dyn + kDynWarps * HV * 32 * sizeof(uint4));  // [kDynTokens]
  if (threadIdx.x < kDynTokens) s_ready[threadIdx.x] = 0;
  if (threadIdx.x == 0) s_sel_next = 0, s_gat_next = 0, s_abort = 0;
  sel::build_region_table(s_region, a.kk, a.k, kDynWarps);  // ends with a block barrier
  // The tables are weights, not the output of an earlier kernel: every block asks for its share of both to be streamed
  // into L2 now, so that the row gathers below, which arrive in routing order, find them there.
  if (threadIdx.x < 2) {
    const int64_t total = N * H * 2;  // bytes of one table
    const int64_t share = ((total + gridDim.x - 1) / gridDim.x + 255) & ~int64_t(255);
    const int64_t lo = share * blockIdx.x, hi = min(total, lo + share);
    const unsigned char* tab = reinterpret_cast<const unsigned char*>(threadIdx.x == 0 ? up : down);
    for (int64_t o = lo; o < hi; o += 16384) l2_prefetch_bulk(tab + o, static_cast<uint32_t>(min(int64_t(16384), hi - o)));
  }
  pdl_wait();  // the logits and y come from earlier kernels
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * tok_per_block;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(tok_per_block), a.T - t0));
  const int k = a.k;
  uint32_t idle = 0;
  long long pr[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // x row, dots, output, store, select, idle, tasks, total (tuning builds)
#ifdef OMNI_TUNING
  const long long pr_t0 = clock64();
#endif
  while (true) {
    // lane 0 picks the task: 1 = gather token idx, 2 = select token idx, 0 = nothing to do right now, -1 = finished
    int task = 0, idx = 0;
    if (lane == 0) {
      const int g = *reinterpret_cast<volatile int*>(&s_gat_next);
      if (g >= ntok || *reinterpret_cast<volatile int*>(&s_abort)) {
        task = -1;
      } else {
        const bool can_gather = *reinterpret_cast<volatile int*>(&s_ready[g]) != 0;
        const bool can_select = *reinterpret_cast<volatile int*>(&s_sel_next) < ntok;
        // half of the warps prefer to gather, the other half to select, so that the two kinds of work overlap
        const bool want_select = can_select && (!can_gather || warp >= kDynWarps / 2);
        if (want_select) {
          const int s = atomicAdd(&s_sel_next, 1);
          if (s < ntok) task = 2, idx = s;
          else task = 3;
        } else if (can_gather) {
          if (atomicCAS(&s_gat_next, g, g + 1) == g) task = 1, idx = g;
          else task = 3;  // another warp took it: look again
        }
      }
    }
    task = __shfl_sync(FULL_MASK, task, 0);
    idx = __shfl_sync(FULL_MASK, idx, 0);
    if (task < 0) break;
    if (task == 1) {
      __threadfence_block();  // the record was written before the flag
      gather_token_tc<HV>(s_rec[idx].e[lane], s_rec[idx].w[lane], k, t0 + idx, x, up, down, s_x + warp * (HV * 32), residual, y, pr);
      pr[6] += 1;
      idle = 0;
    } else if (task == 2) {
      OMNI_TIC(cq);
      const int64_t t = t0 + idx;
      uint32_t rkey[sel::kMaxK / 32], rflat[sel::kMaxK / 32];
      sel::select_token<VPL, CPL, true, Scratch>(a, t, s_warp[warp], s_region.cell, rkey, rflat);
      // k <= 32 (checked by the host), so rank r lives in lane r
      int my_e = 0;
      float my_w = 0.f;
      bool valid = false;
      if (lane < k) {
        const float sc = key_to_float(rkey[0]);
        my_w = expf(sc);
        my_e = static_cast<int>(rflat[0]);  // < sqrt_n^2 <= N by construction
        const int64_t o = t * k + lane;
        if (a.scores) a.scores[o] = sc;
        if (a.indices) reinterpret_cast<int32_t*>(a.indices)[o] = my_e;
        if (a.weights) a.weights[o] = my_w;
        valid = my_e >= 0 && my_e < N;
      }
      const unsigned ok_mask = __ballot_sync(FULL_MASK, valid);
      const int safe = ok_mask ? __shfl_sync(FULL_MASK, my_e, __ffs(ok_mask) - 1) : 0;  // a row that exists
      s_rec[idx].e[lane] = valid ? my_e : safe;
      s_rec[idx].w[lane] = valid ? my_w : 0.f;
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&s_ready[idx]) = 1;
      }
      idle = 0;
      OMNI_TOC(pr[4], cq);
      pr[6] += 1000;
    } else if (task == 0) {
      OMNI_TIC(ci);
      // every token is being selected by some other warp and none is ready yet: those warps never wait, so this ends;
      // the limit only guards against a defect
      __nanosleep(200);
      if (++idle > kDynSpinLimit) {
        if (lane == 0) {
          s_abort = 1;
          if (status) atomicOr(status, OMNI_ST_WAIT_TIMEOUT);
        }
        break;
      }
      OMNI_TOC(pr[5], ci);
    }
  }
#ifdef OMNI_TUNING
  if (lane == 0 && blockIdx.x < 160) {
    pr[7] = clock64() - pr_t0;
    for (int i = 0; i < 8; ++i) g_dyn_prof[(blockIdx.x * 16 + warp) * 8 + i] = pr[i];
  }
#endif
}

// fp32 operands end to end (x, both tables, output): the accuracy path for callers that hold float32 tensors and
// expect float32 arithmetic (the reference computes in the dtype of its inputs, omni_moe/ops/triton/omni_expert.py:13-168).
// One warp per token, two passes: the k coefficients w * silu(x . Up[e]) first (kept in shared memory), then the sum of
// Down rows one slab of 1024 columns at a time (8 float4 accumulators per lane).  CUDA cores only: there is no fp32
// tensor-core path, and this is a compatibility kernel, not a tuned one.
__global__ void __launch_bounds__(kThreads) expert_fused_f32_kernel(
    const float* __restrict__ x, const float* __restrict__ up, const float* __restrict__ down, const float* __restrict__ weights,
    const int* __restrict__ indices, int64_t T, int k, int H, int64_t N, const float* residual, float* y, int* status) {
  __shared__ float s_c[kWarps][sel::kMaxK];
  __shared__ int s_e[kWarps][sel::kMaxK];
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (t >= T) return;
  const float4* xr = reinterpret_cast<const float4*>(x + t * H);
  const int h4 = H >> 2;
  bool bad = false;
  for (int j = 0; j < k; ++j) {
    const int e = indices[t * k + j];
    float c = 0.f;
    if (e < 0 || e >= N) {
      bad = true;
    } else {
      const float4* ur = reinterpret_cast<const float4*>(up + static_cast<int64_t>(e) * H);
      float a0 = 0.f, a1 = 0.f;
      for (int i = lane; i < h4; i += 64) {
        const float4 p = __ldg(xr + i), q = __ldg(ur + i);
        a0 = __fmaf_rn(p.x, q.x, a0), a0 = __fmaf_rn(p.y, q.y, a0), a0 = __fmaf_rn(p.z, q.z, a0), a0 = __fmaf_rn(p.w, q.w, a0);
        if (i + 32 < h4) {
          const float4 p2 = __ldg(xr + i + 32), q2 = __ldg(ur + i + 32);
          a1 = __fmaf_rn(p2.x, q2.x, a1), a1 = __fmaf_rn(p2.y, q2.y, a1), a1 = __fmaf_rn(p2.z, q2.z, a1), a1 = __fmaf_rn(p2.w, q2.w, a1);
        }
      }
      const float dot = warp_sum(a0 + a1);
      c = weights[t * k + j] * (dot / (1.0f + expf(-dot)));
    }
    if (lane == 0) s_c[warp][j] = c, s_e[warp][j] = (e < 0 || e >= N) ? 0 : e;
  }
  __syncwarp();
  for (int c0 = 0; c0 < h4; c0 += 256) {  // 256 float4 = 1024 columns per slab, 8 float4 per lane
    float4 acc[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      const float c = s_c[warp][j];
      const float4* dr = reinterpret_cast<const float4*>(down + static_cast<int64_t>(s_e[warp][j]) * H) + c0 + lane;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        if (c0 + lane + v * 32 < h4) {
          const float4 d = __ldg(dr + v * 32);
          acc[v].x = __fmaf_rn(c, d.x, acc[v].x), acc[v].y = __fmaf_rn(c, d.y, acc[v].y);
          acc[v].z = __fmaf_rn(c, d.z, acc[v].z), acc[v].w = __fmaf_rn(c, d.w, acc[v].w);
        }
      }
    }
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const int i = c0 + lane + v * 32;
      if (i < h4) {
        float4 o = acc[v];
        if (residual) {
          const float4 r = *(reinterpret_cast<const float4*>(residual + t * H) + i);  // plain load: may be y itself
          o.x += r.x, o.y += r.y, o.z += r.z, o.w += r.w;
        }
        *(reinterpret_cast<float4*>(y + t * H) + i) = o;
      }
    }
  }
  if (bad && lane == 0) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// OMNI_MOE_B200_ROUTED=legacy: dot products on the CUDA cores, one token per warp, for every shape
bool routed_legacy() {
  static const bool v = [] {
    const char* e = getenv("OMNI_MOE_B200_ROUTED");
    return e && e[0] == 'l';
  }();
  return v;
}

}  // namespace
}  // namespace omni

using namespace omni;

static int launch_expert_coef(const void* x, const void* up, const float* weights, const int32_t* sorted_pair_ids,
                              const int32_t* sorted_experts, int64_t num_tokens, int k, int hidden,
                              int64_t num_experts, float* coef, int32_t* status, void* stream, const int* hot_ids,
                              const float* hot_dots, bool raw = false) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && hidden >= 8 && num_experts >= 1, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  const int64_t P = num_tokens * k;
  if (P == 0) return 0;
  OMNI_REQUIRE(x && up && (weights || raw) && sorted_pair_ids && sorted_experts && coef && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up), "x and up must be 16-byte aligned");
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* ub = static_cast<const __nv_bfloat16*>(up);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div64(ceil_div64(P, kRun), kWarps));
#define OMNI_COEF(HV)                                                                                         \
  expert_coef_kernel<HV><<<grid, kThreads, 0, st>>>(xb, ub, weights, sorted_pair_ids, sorted_experts, nullptr, P,     \
                                                   num_tokens, k, hidden, num_experts, coef, status, hot_ids, hot_dots)
  if (hidden <= 256) OMNI_COEF(1);
  else if (hidden <= 512) OMNI_COEF(2);
  else if (hidden <= 1024) OMNI_COEF(4);
  else if (hidden <= 2048) OMNI_COEF(8);
  else OMNI_COEF(16);
#undef OMNI_COEF
  return check_launch("expert_coef_kernel");
}

extern "C" int omni_expert_dots(const void* x, const void* up, const int32_t* sorted_pair_ids, const int32_t* sorted_experts,
                                int64_t num_tokens, int k, int hidden, int64_t num_experts, float* dots, int32_t* status,
                                void* stream) {
  return launch_expert_coef(x, up, nullptr, sorted_pair_ids, sorted_experts, num_tokens, k, hidden, num_experts, dots, status,
                            stream, nullptr, nullptr, true);
}

extern "C" int omni_expert_coef(const void* x, const void* up, const float* weights, const int32_t* sorted_pair_ids,
                                const int32_t* sorted_experts, int64_t num_tokens, int k, int hidden,
                                int64_t num_experts, float* coef, int32_t* status, void* stream) {
  return launch_expert_coef(x, up, weights, sorted_pair_ids, sorted_experts, num_tokens, k, hidden, num_experts, coef,
                            status, stream, nullptr, nullptr);
}

namespace {
constexpr int64_t kHotIdsBytes = 1024;  // kHot ids + the count, padded so that the rows behind them stay aligned
int64_t hot_rows_bytes(int hidden) { return static_cast<int64_t>(kHot) * hidden * 2; }
}  // namespace

extern "C" int64_t omni_expert_coef_hot_workspace(int64_t num_tokens, int hidden) {
  if (num_tokens < 0 || hidden < 8) return 0;
  return kHotIdsBytes + hot_rows_bytes(hidden) + num_tokens * kHot * static_cast<int64_t>(sizeof(float));
}

extern "C" int omni_expert_coef_hot(const void* x, const void* up, const float* weights, const int32_t* sorted_pair_ids,
                                    const int32_t* sorted_experts, int64_t num_tokens, int k, int hidden,
                                    int64_t num_experts, int64_t min_run, float* coef, void* workspace,
                                    int64_t workspace_bytes, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && hidden >= 8 && hidden % 8 == 0 && num_experts >= 1, "bad sizes");
  const int64_t P = num_tokens * k;
  if (P == 0) return 0;
  OMNI_REQUIRE(x && up && weights && sorted_pair_ids && sorted_experts && coef && status && workspace, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up) && aligned16(workspace), "x, up and workspace must be 16-byte aligned");
  OMNI_REQUIRE(workspace_bytes >= omni_expert_coef_hot_workspace(num_tokens, hidden),
               "workspace holds %lld bytes, omni_expert_coef_hot_workspace asks for %lld",
               static_cast<long long>(workspace_bytes),
               static_cast<long long>(omni_expert_coef_hot_workspace(num_tokens, hidden)));
  if (min_run <= 0) min_run = num_tokens / 32 > 512 ? num_tokens / 32 : 512;
  OMNI_REQUIRE(min_run < (int64_t(1) << 30), "min_run out of range");
  char* ws = static_cast<char*>(workspace);
  int* hot_ids = reinterpret_cast<int*>(ws);
  auto* hot_rows = reinterpret_cast<__nv_bfloat16*>(ws + kHotIdsBytes);
  float* hot_dots = reinterpret_cast<float*>(ws + kHotIdsBytes + hot_rows_bytes(hidden));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  hot_rows_kernel<<<kHot, kThreads, 0, st>>>(sorted_experts, P, static_cast<int>(min_run), num_experts,
                                             static_cast<const __nv_bfloat16*>(up), hidden, hot_ids, hot_rows);
  if (int e = check_launch("hot_rows_kernel")) return e;
  // products of every token with the kHot rows: [T, kHot] fp32, two halves of kHot / 2 columns side by side
  // (skipped on the device when no expert qualified)
  if (int e = router_gate_if(x, hot_rows, hot_rows + static_cast<int64_t>(kHot / 2) * hidden, num_tokens, hidden, kHot / 2,
                             hot_dots, hot_ids + kHot, status, stream))
    return e;
  return launch_expert_coef(x, up, weights, sorted_pair_ids, sorted_experts, num_tokens, k, hidden, num_experts, coef,
                            status, stream, hot_ids, hot_dots);
}

// Column slab of the combine by row length.  Four rows of a 1024-column slab in flight per warp at 127 registers keeps
// 16 warps on an SM; wider slabs or more rows per step leave fewer warps and were slower at every measured shape.
static int launch_combine(const __nv_bfloat16* db, const float* coef, const int32_t* experts, const int32_t* offsets,
                          int64_t num_tokens, int k, int hidden, int64_t num_experts, const void* residual, void* y,
                          int out_dtype, int32_t* status, cudaStream_t st) {
  const int hv = hidden <= 256 ? 1 : hidden <= 512 ? 2 : 4;
  const int slabs = ceil_div(hidden, hv * 256);
  const unsigned grid = static_cast<unsigned>(ceil_div64(num_tokens * slabs, kCombineThreads / 32));
#define OMNI_COMB(HV)                                                                                                  \
  do {                                                                                                                 \
    if (out_dtype == OMNI_F32)                                                                                         \
      expert_combine_kernel<HV, true><<<grid, kCombineThreads, 0, st>>>(db, coef, experts, offsets, num_tokens, k, hidden, \
                                                                        num_experts, slabs, residual, y, status);      \
    else                                                                                                               \
      expert_combine_kernel<HV, false><<<grid, kCombineThreads, 0, st>>>(db, coef, experts, offsets, num_tokens, k, hidden, \
                                                                         num_experts, slabs, residual, y, status);     \
  } while (0)
  if (hv == 1) OMNI_COMB(1);
  else if (hv == 2) OMNI_COMB(2);
  else OMNI_COMB(4);
#undef OMNI_COMB
  return check_launch("expert_combine_kernel");
}

extern "C" int omni_expert_combine(const void* down, const float* coef, const int32_t* indices, int64_t num_tokens,
                                   int k, int hidden, int64_t num_experts, const void* residual, void* y,
                                   int out_dtype, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && hidden >= 8 && num_experts >= 1, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  OMNI_REQUIRE(out_dtype == OMNI_F32 || out_dtype == OMNI_BF16, "out_dtype must be OMNI_F32 or OMNI_BF16");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(down && coef && indices && y && status, "NULL argument");
  OMNI_REQUIRE(aligned16(down) && aligned16(y) && aligned16(residual), "down, y and residual must be 16-byte aligned");
  const auto* db = static_cast<const __nv_bfloat16*>(down);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return launch_combine(db, coef, indices, nullptr, num_tokens, k, hidden, num_experts, residual, y, out_dtype, status, st);
}

extern "C" int omni_expert_fused(const void* x, const void* up, const void* down, const float* weights,
                                 const int32_t* indices, int64_t num_tokens, int k, int hidden, int64_t num_experts,
                                 const void* residual, void* y, int out_dtype, float* coef, int32_t* status,
                                 void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && hidden >= 8 && num_experts >= 1, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  OMNI_REQUIRE(hidden <= 2048, "omni_expert_fused keeps a whole row in registers: hidden <= 2048, got %d "
               "(use omni_schedule + omni_expert_coef + omni_expert_combine)", hidden);
  OMNI_REQUIRE(out_dtype == OMNI_F32 || out_dtype == OMNI_BF16, "out_dtype must be OMNI_F32 or OMNI_BF16");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && up && down && weights && indices && y && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up) && aligned16(down) && aligned16(y) && aligned16(residual),
               "x, up, down, y and residual must be 16-byte aligned");
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* ub = static_cast<const __nv_bfloat16*>(up);
  const auto* db = static_cast<const __nv_bfloat16*>(down);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div64(num_tokens, kWarps));
  if (!routed_legacy() && out_dtype == OMNI_BF16 && coef == nullptr && k <= 32 &&
      (hidden == 256 || hidden == 512 || hidden == 1024)) {
    // dots on the tensor cores; output bits differ from the CUDA-core kernel below (another summation order)
    if (hidden == 256)
      launch_after_predecessor(expert_fused_tc_kernel<1>, dim3(grid), dim3(kThreads), 0, st, xb, ub, db, weights, indices,
                               num_tokens, k, num_experts, residual, y, status);
    else if (hidden == 512)
      launch_after_predecessor(expert_fused_tc_kernel<2>, dim3(grid), dim3(kThreads), 0, st, xb, ub, db, weights, indices,
                               num_tokens, k, num_experts, residual, y, status);
    else
      launch_after_predecessor(expert_fused_tc_kernel<4>, dim3(grid), dim3(kThreads), 0, st, xb, ub, db, weights, indices,
                               num_tokens, k, num_experts, residual, y, status);
    return check_launch("expert_fused_tc_kernel");
  }
#define OMNI_FUSED(HV)                                                                                                 \
  do {                                                                                                                 \
    if (out_dtype == OMNI_F32)                                                                                         \
      expert_fused_kernel<HV, true><<<grid, kThreads, 0, st>>>(xb, ub, db, weights, indices, num_tokens, k, hidden,    \
                                                               num_experts, residual, y, coef, status);                 \
    else                                                                                                               \
      expert_fused_kernel<HV, false><<<grid, kThreads, 0, st>>>(xb, ub, db, weights, indices, num_tokens, k, hidden,   \
                                                                num_experts, residual, y, coef, status);                \
  } while (0)
  if (hidden <= 256) OMNI_FUSED(1);
  else if (hidden <= 512) OMNI_FUSED(2);
  else if (hidden <= 1024) OMNI_FUSED(4);
  else OMNI_FUSED(8);
#undef OMNI_FUSED
  return check_launch("expert_fused_kernel");
}

extern "C" int omni_route_expert_fused(const float* logits, int64_t ld_logits, const float* bn_scale,
                                       const float* bn_shift, const void* x, const void* up, const void* down,
                                       int64_t num_tokens, int sqrt_n, int k, int hidden, int64_t num_experts,
                                       const void* residual, void* y, float* scores, int32_t* indices,
                                       float* weights, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && hidden >= 8 && hidden % 8 == 0 && hidden <= 2048,
               "hidden must be a multiple of 8 in [8, 2048], got %d", hidden);
  OMNI_REQUIRE(sqrt_n >= 1 && sqrt_n <= 256, "omni_route_expert_fused: sqrt_n must be in [1, 256], got %d", sqrt_n);
  OMNI_REQUIRE(k >= 1 && static_cast<int64_t>(k) <= static_cast<int64_t>(sqrt_n) * sqrt_n, "k out of range: %d", k);
  OMNI_REQUIRE(static_cast<int64_t>(sqrt_n) * sqrt_n <= num_experts, "the tables have fewer than sqrt_n^2 rows");
  OMNI_REQUIRE(ld_logits >= 2 * sqrt_n, "ld_logits %lld < 2*sqrt_n", static_cast<long long>(ld_logits));
  OMNI_REQUIRE((bn_scale == nullptr) == (bn_shift == nullptr), "bn_scale and bn_shift must be given together");
  sel::TopkArgs a{};
  a.in_x = logits, a.in_dtype = OMNI_F32, a.ld_in = ld_logits, a.bn_scale = bn_scale, a.bn_shift = bn_shift;
  a.T = num_tokens, a.n = sqrt_n, a.k = k, a.kk = sqrt_n < k ? sqrt_n : k;
  a.cells = sel::region_cells(a.kk, k);
  a.scores = scores, a.indices = indices, a.idx_is_i64 = 0, a.weights = weights;
  OMNI_REQUIRE(k <= 32 && a.cells <= 128, "omni_route_expert_fused handles k <= 32 (got %d, %d candidate cells); "
               "use omni_router_logits_topk + omni_expert_fused", k, a.cells);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(logits && x && up && down && y, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up) && aligned16(down) && aligned16(y) && aligned16(residual),
               "x, up, down, y and residual must be 16-byte aligned");
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* ub = static_cast<const __nv_bfloat16*>(up);
  const auto* db = static_cast<const __nv_bfloat16*>(down);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div64(num_tokens, kWarps));
  if (!routed_legacy() && (hidden == 256 || hidden == 512 || hidden == 1024)) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    int tpb = static_cast<int>(ceil_div64(num_tokens, sms));
    tpb = tpb < 1 ? 1 : (tpb > kDynTokens ? kDynTokens : tpb);
    const unsigned dgrid = static_cast<unsigned>(ceil_div64(num_tokens, tpb));
    const size_t dyn = static_cast<size_t>(kDynWarps) * (hidden / 8) * sizeof(uint4) + kDynTokens * sizeof(RoutedRecord);
#define OMNI_ROUTED_DYN(HV, VPL, CPL)                                                                                      \
  do {                                                                                                                     \
    static OncePerDevice once;                                                                                             \
    if (once.first() && cudaFuncSetAttribute(expert_routed_dyn_kernel<HV, VPL, CPL>,                                       \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,                                   \
                                             kDynWarps * HV * 32 * 16 + kDynTokens * sizeof(RoutedRecord)) != cudaSuccess) \
      return fail(-3, "expert_routed_dyn_kernel: cannot reserve its shared memory");                                       \
    launch_after_predecessor(expert_routed_dyn_kernel<HV, VPL, CPL>, dim3(dgrid), dim3(kDynWarps * 32), dyn, st, a, xb, ub, \
                             db, num_experts, tpb, residual, y, status);                                                    \
  } while (0)
#define OMNI_ROUTED_DYN_HV(VPL, CPL)                        \
  do {                                                      \
    if (hidden == 256) OMNI_ROUTED_DYN(1, VPL, CPL);        \
    else if (hidden == 512) OMNI_ROUTED_DYN(2, VPL, CPL);   \
    else OMNI_ROUTED_DYN(4, VPL, CPL);                      \
  } while (0)
    const bool small = a.cells <= 64;
    if (sqrt_n <= 64) {
      if (small) OMNI_ROUTED_DYN_HV(2, 2);
      else OMNI_ROUTED_DYN_HV(2, 4);
    } else {
      if (small) OMNI_ROUTED_DYN_HV(8, 2);
      else OMNI_ROUTED_DYN_HV(8, 4);
    }
#undef OMNI_ROUTED_DYN_HV
#undef OMNI_ROUTED_DYN
    return check_launch("expert_routed_dyn_kernel");
  }
#define OMNI_ROUTED(HV, VPL, CPL) \
  launch_after_predecessor(expert_routed_kernel<HV, VPL, CPL>, dim3(grid), dim3(kThreads), 0, st, a, xb, ub, db, hidden, \
                           num_experts, residual, y)
#define OMNI_ROUTED_HV(VPL, CPL)                  \
  do {                                            \
    if (hidden <= 256) OMNI_ROUTED(1, VPL, CPL);  \
    else if (hidden <= 512) OMNI_ROUTED(2, VPL, CPL);  \
    else if (hidden <= 1024) OMNI_ROUTED(4, VPL, CPL); \
    else OMNI_ROUTED(8, VPL, CPL);                \
  } while (0)
  const bool small_cells = a.cells <= 64;
  if (sqrt_n <= 64) {
    if (small_cells) OMNI_ROUTED_HV(2, 2);
    else OMNI_ROUTED_HV(2, 4);
  } else {
    if (small_cells) OMNI_ROUTED_HV(8, 2);
    else OMNI_ROUTED_HV(8, 4);
  }
#undef OMNI_ROUTED_HV
#undef OMNI_ROUTED
  return check_launch("expert_routed_kernel");
}

extern "C" int omni_expert_coef_pairs(const void* x, const void* up, const int32_t* pair_tokens, const float* pair_weights,
                                      const int32_t* sorted_pair_ids, const int32_t* sorted_experts, int64_t num_pairs,
                                      int64_t num_tokens, int hidden, int64_t num_experts, float* coef,
                                      int32_t* status, void* stream) {
  OMNI_REQUIRE(num_pairs >= 0 && num_tokens >= 0 && hidden >= 8 && num_experts >= 1, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  OMNI_REQUIRE(num_pairs < (int64_t(1) << 31), "too many pairs");
  if (num_pairs == 0) return 0;
  OMNI_REQUIRE(x && up && pair_tokens && pair_weights && sorted_pair_ids && sorted_experts && coef && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up), "x and up must be 16-byte aligned");
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* ub = static_cast<const __nv_bfloat16*>(up);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div64(ceil_div64(num_pairs, kRun), kWarps));
#define OMNI_COEFP(HV)                                                                                               \
  expert_coef_kernel<HV><<<grid, kThreads, 0, st>>>(xb, ub, pair_weights, sorted_pair_ids, sorted_experts, pair_tokens, \
                                                   num_pairs, num_tokens, 1, hidden, num_experts, coef, status, nullptr, nullptr)
  if (hidden <= 256) OMNI_COEFP(1);
  else if (hidden <= 512) OMNI_COEFP(2);
  else if (hidden <= 1024) OMNI_COEFP(4);
  else if (hidden <= 2048) OMNI_COEFP(8);
  else OMNI_COEFP(16);
#undef OMNI_COEFP
  return check_launch("expert_coef_kernel (pair list)");
}

extern "C" int omni_expert_combine_segments(const void* down, const float* coef, const int32_t* pair_experts,
                                            const int32_t* token_offsets, int64_t num_tokens, int hidden,
                                            int64_t num_experts, const void* residual, void* y, int out_dtype,
                                            int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && hidden >= 8 && num_experts >= 1, "bad sizes");
  OMNI_REQUIRE(hidden % 8 == 0, "hidden must be a multiple of 8, got %d", hidden);
  OMNI_REQUIRE(out_dtype == OMNI_F32 || out_dtype == OMNI_BF16, "out_dtype must be OMNI_F32 or OMNI_BF16");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(down && token_offsets && y && status, "NULL argument");
  OMNI_REQUIRE(aligned16(down) && aligned16(y) && aligned16(residual), "down, y and residual must be 16-byte aligned");
  const auto* db = static_cast<const __nv_bfloat16*>(down);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return launch_combine(db, coef, pair_experts, token_offsets, num_tokens, 0, hidden, num_experts, residual, y, out_dtype,
                        status, st);
}

extern "C" int omni_expert_fused_f32(const float* x, const float* up, const float* down, const float* weights,
                                     const int32_t* indices, int64_t num_tokens, int k, int hidden, int64_t num_experts,
                                     const float* residual, float* y, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && k <= sel::kMaxK && hidden >= 4 && num_experts >= 1, "bad sizes (k <= %d)", sel::kMaxK);
  OMNI_REQUIRE(hidden % 4 == 0, "hidden must be a multiple of 4, got %d", hidden);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && up && down && weights && indices && y && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(up) && aligned16(down) && aligned16(y) && aligned16(residual),
               "x, up, down, y and residual must be 16-byte aligned");
  const unsigned grid = static_cast<unsigned>(ceil_div64(num_tokens, kWarps));
  expert_fused_f32_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, up, down, weights, indices, num_tokens, k,
                                                                                   hidden, num_experts, residual, y, status);
  return check_launch("expert_fused_f32_kernel");
}

#ifdef OMNI_TUNING
// tuning builds only: the per-warp cycle counters of the latest expert_routed_dyn_kernel launch (160 x 16 x 8 words)
extern "C" OMNI_API int omni_debug_routed_profile(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, omni::g_dyn_prof, sizeof(long long) * 160 * 16 * 8) == cudaSuccess ? 0 : -3;
}
#endif
