// Product-key router selection: one warp per token.
//
// Per token the kernel holds the two sub-key rows in registers, extracts the kk = min(sqrt_n, k)
// best sub-keys of each axis (score descending, index ascending), and then searches the kk x kk
// candidate sums for the k best (sum descending, flat expert index ascending).
//
// Search pruning.  In rank space (i = rank on x, j = rank on y) a cell can only be among the k
// best if (i+1)*(j+1) <= k, because every cell it dominates scores at least as much.  Only those
// ~k*ln(k) cells are materialised.  fp32 rounding can make a dominated cell *tie* with a cell
// outside that region, and the tie rule (lower flat index) could then prefer the outside cell, so
// after the pruned search the kernel tests the first cell outside the region in every row against
// the k-th score; a token that shows such a tie is redone by an exact scan over all kk x kk cells.
#include "common.cuh"

namespace omni {
namespace {

constexpr int kMaxK = 128;
constexpr int kWarpsPerBlock = 4;
constexpr int kMaxCells = 704;  // cells with (i+1)(j+1) <= 128 in a 128 x 128 grid: 642

struct TopkArgs {
  const void* in_x;      // PRE: logits row base (x axis at column 0); else log-probs x
  const void* in_y;      // PRE: unused; else log-probs y
  int in_dtype;          // OMNI_F32 / OMNI_BF16 / OMNI_F16 (PRE: always f32)
  int64_t ld_in;         // row stride in elements
  const float* bn_scale; // PRE only, may be null
  const float* bn_shift;
  float* lp_out;         // PRE only, may be null: [T, 2n]
  int64_t T;
  int n, k, kk, cells;
  float* scores;
  void* indices;
  int idx_is_i64;
  float* weights;
};

__device__ __forceinline__ float load_as_float(const void* base, int dtype, int64_t i) {
  if (dtype == OMNI_F32) return __ldg(reinterpret_cast<const float*>(base) + i);
  if (dtype == OMNI_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
}

// Extracts the kk largest of a row spread over the warp (element e of lane l is sub-key e*32+l;
// key 0 marks "absent").  Writes sorted scores and sub-key indices to shared memory.
template <int VPL>
__device__ __forceinline__ void axis_select(uint32_t (&key)[VPL], int kk, float* s_out, int* i_out) {
  const int lane = lane_id();
  uint32_t lmax = 0;
#pragma unroll
  for (int e = 0; e < VPL; ++e) lmax = max(lmax, key[e]);
  for (int r = 0; r < kk; ++r) {
    const uint32_t m = __reduce_max_sync(FULL_MASK, lmax);
    uint32_t mine = 0xffffffffu;
    if (lmax == m) {
#pragma unroll
      for (int e = VPL - 1; e >= 0; --e)
        if (key[e] == m) mine = e * 32 + lane;
    }
    const uint32_t w = __reduce_min_sync(FULL_MASK, mine);
    if (lane == 0) {
      s_out[r] = key_to_float(m);
      i_out[r] = static_cast<int>(w);
    }
    if ((w & 31u) == static_cast<uint32_t>(lane)) {
      lmax = 0;
#pragma unroll
      for (int e = 0; e < VPL; ++e) {
        if (e == static_cast<int>(w >> 5)) key[e] = 0;
        lmax = max(lmax, key[e]);
      }
    }
    __syncwarp();
  }
}

// Small rows (at most 64 entries, two per lane): rank every entry by counting the entries that beat
// it.  The entries are made distinct by packing (score key, ~index) into 64 bits, so the ranks are a
// permutation; there is no cross-lane dependency chain, only broadcast reads of shared memory.
// Returns the rank of `mine` among the 64 packed entries in `all`.
__device__ __forceinline__ int rank_among_64(const unsigned long long* all, unsigned long long mine) {
  int rank = 0;
  const ulonglong2* p = reinterpret_cast<const ulonglong2*>(all);
#pragma unroll 8
  for (int q = 0; q < 32; ++q) {
    const ulonglong2 o = p[q];
    rank += (o.x > mine) + (o.y > mine);
  }
  return rank;
}

template <int VPL, int CPL, bool PRE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) router_topk_kernel(const TopkArgs a) {
  constexpr bool kSmallAxis = VPL == 2;   // n <= 64: rank by counting instead of selection rounds
  constexpr bool kSmallCells = CPL == 2;  // <= 64 candidate cells: likewise
  __shared__ __align__(16) unsigned long long s_pack[(kSmallAxis || kSmallCells) ? kWarpsPerBlock : 1][64];
  __shared__ uint32_t s_rk[kSmallCells ? kWarpsPerBlock : 1][kSmallCells ? 64 : 1];
  __shared__ uint32_t s_rf[kSmallCells ? kWarpsPerBlock : 1][kSmallCells ? 64 : 1];
  __shared__ float s_sx[kWarpsPerBlock][kMaxK], s_sy[kWarpsPerBlock][kMaxK];
  __shared__ int s_ix[kWarpsPerBlock][kMaxK], s_iy[kWarpsPerBlock][kMaxK];
  __shared__ uint16_t s_cell[kMaxCells];  // i | j << 8 for each cell of the pruned region
  __shared__ int s_rowstart[kMaxK + 1];

  const int lane = lane_id();
  const int warp = threadIdx.x >> 5;
  const int n = a.n, k = a.k, kk = a.kk;

  // Region table, shared by the block: row i keeps columns [0, min(kk, k/(i+1))).
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < kk; ++i) {
      s_rowstart[i] = acc;
      acc += min(kk, k / (i + 1));
    }
    s_rowstart[kk] = acc;
  }
  __syncthreads();
  for (int i = warp; i < kk; i += kWarpsPerBlock) {
    const int st = s_rowstart[i], cnt = s_rowstart[i + 1] - st;
    for (int j = lane; j < cnt; j += 32) s_cell[st + j] = static_cast<uint16_t>(i | (j << 8));
  }
  __syncthreads();

  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (t >= a.T) return;
  float* sx = s_sx[warp];
  float* sy = s_sy[warp];
  int* ix = s_ix[warp];
  int* iy = s_iy[warp];

  // ---- per-axis rows -> sorted best kk --------------------------------------------------
#pragma unroll 1
  for (int axis = 0; axis < 2; ++axis) {
    uint32_t key[VPL];
    if (PRE) {
      const float* row = reinterpret_cast<const float*>(a.in_x) + t * a.ld_in + axis * n;
      float v[VPL];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < VPL; ++e) {
        const int c = e * 32 + lane;
        if (c < n) {
          float z = __ldg(row + c);
          if (a.bn_scale) z = __fmaf_rn(z, __ldg(a.bn_scale + axis * n + c), __ldg(a.bn_shift + axis * n + c));
          v[e] = z;
          mx = fmaxf(mx, z);
        } else {
          v[e] = -INFINITY;
        }
      }
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < VPL; ++e)
        if (e * 32 + lane < n) sum += expf(v[e] - mx);
      sum = warp_sum(sum);
      const float lse = logf(sum);
#pragma unroll
      for (int e = 0; e < VPL; ++e) {
        const int c = e * 32 + lane;
        if (c < n) {
          const float lp = (v[e] - mx) - lse;
          if (a.lp_out) a.lp_out[t * (2 * n) + axis * n + c] = lp;
          key[e] = float_to_key(lp);
        } else {
          key[e] = 0;
        }
      }
    } else {
      const void* base = axis == 0 ? a.in_x : a.in_y;
#pragma unroll
      for (int e = 0; e < VPL; ++e) {
        const int c = e * 32 + lane;
        key[e] = c < n ? float_to_key(load_as_float(base, a.in_dtype, t * a.ld_in + c)) : 0u;
      }
    }
    if constexpr (kSmallAxis) {
      unsigned long long mine[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t c = e * 32 + lane;
        mine[e] = (static_cast<unsigned long long>(key[e]) << 32) | (0xffffffffu - c);
        s_pack[warp][c] = mine[e];
      }
      __syncwarp();
      float* so = axis == 0 ? sx : sy;
      int* io = axis == 0 ? ix : iy;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int r = rank_among_64(s_pack[warp], mine[e]);
        if (r < kk) so[r] = key_to_float(key[e]), io[r] = e * 32 + lane;
      }
      __syncwarp();
    } else {
      axis_select<VPL>(key, kk, axis == 0 ? sx : sy, axis == 0 ? ix : iy);
    }
  }
  __syncwarp();

  // ---- pruned candidate search ----------------------------------------------------------
  uint32_t ckey[CPL], cflat[CPL];
  uint32_t lmax = 0;
#pragma unroll
  for (int q = 0; q < CPL; ++q) {
    const int c = q * 32 + lane;
    if (c < a.cells) {
      const int cell = s_cell[c];
      const int i = cell & 0xff, j = cell >> 8;
      ckey[q] = float_to_key(__fadd_rn(sx[i], sy[j]));
      cflat[q] = static_cast<uint32_t>(ix[i]) * n + iy[j];
    } else {
      ckey[q] = 0;
      cflat[q] = 0xffffffffu;
    }
    lmax = max(lmax, ckey[q]);
  }
  uint32_t rkey[kMaxK / 32], rflat[kMaxK / 32];
#pragma unroll
  for (int s = 0; s < kMaxK / 32; ++s) rkey[s] = 0, rflat[s] = 0;
  uint32_t last_key = 0;
  if constexpr (kSmallCells) {
    unsigned long long mine[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      // padding cells have key 0 and can never outrank a real one; real cells differ in `flat`
      mine[q] = (static_cast<unsigned long long>(ckey[q]) << 32) | (0xffffffffu - cflat[q]);
      s_pack[warp][q * 32 + lane] = mine[q];
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int r = rank_among_64(s_pack[warp], mine[q]);
      if (r < k && ckey[q] != 0) s_rk[warp][r] = ckey[q], s_rf[warp][r] = cflat[q];
    }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int r = s * 32 + lane;
      if (r < k) rkey[s] = s_rk[warp][r], rflat[s] = s_rf[warp][r];
    }
    last_key = s_rk[warp][k - 1];
  } else
  for (int r = 0; r < k; ++r) {
    const uint32_t m = __reduce_max_sync(FULL_MASK, lmax);
    uint32_t mine = 0xffffffffu;
    if (lmax == m) {
#pragma unroll
      for (int q = 0; q < CPL; ++q)
        if (ckey[q] == m) mine = min(mine, cflat[q]);
    }
    const uint32_t w = __reduce_min_sync(FULL_MASK, mine);
    if (lane == (r & 31)) {
#pragma unroll
      for (int s = 0; s < kMaxK / 32; ++s)
        if (s == (r >> 5)) rkey[s] = m, rflat[s] = w;
    }
    if (mine == w && lmax == m) {  // flat indices are unique, so exactly one lane owns the winner
      lmax = 0;
#pragma unroll
      for (int q = 0; q < CPL; ++q) {
        if (ckey[q] == m && cflat[q] == w) ckey[q] = 0;
        lmax = max(lmax, ckey[q]);
      }
    }
    last_key = m;
    __syncwarp();
  }

  // ---- did a cell outside the region tie with the k-th score? -----------------------------
  bool tie = false;
  for (int i = lane; i < kk; i += 32) {
    const int j0 = min(kk, k / (i + 1));
    if (j0 < kk && float_to_key(__fadd_rn(sx[i], sy[j0])) >= last_key) tie = true;
  }
  if (__any_sync(FULL_MASK, tie)) {
    // Exact scan: round r takes the best cell that comes after the previous winner in the order
    // (key descending, flat ascending).
    uint32_t pk = 0xffffffffu, pf = 0;
    bool first = true;
    for (int r = 0; r < k; ++r) {
      uint32_t bk = 0, bf = 0xffffffffu;
      for (int c = lane; c < kk * kk; c += 32) {
        const int i = c / kk, j = c - i * kk;
        const uint32_t key = float_to_key(__fadd_rn(sx[i], sy[j]));
        const uint32_t flat = static_cast<uint32_t>(ix[i]) * n + iy[j];
        const bool after = first || key < pk || (key == pk && flat > pf);
        if (after && (key > bk || (key == bk && flat < bf))) bk = key, bf = flat;
      }
      const uint32_t m = __reduce_max_sync(FULL_MASK, bk);
      const uint32_t w = __reduce_min_sync(FULL_MASK, bk == m ? bf : 0xffffffffu);
      if (lane == (r & 31)) {
#pragma unroll
        for (int s = 0; s < kMaxK / 32; ++s)
          if (s == (r >> 5)) rkey[s] = m, rflat[s] = w;
      }
      pk = m, pf = w, first = false;
    }
  }

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

int region_cells(int kk, int k) {
  int c = 0;
  for (int i = 0; i < kk; ++i) c += (k / (i + 1) < kk) ? k / (i + 1) : kk;
  return c;
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
    static bool carveout_set = false;                                                                           \
    if (!carveout_set) {                                                                                        \
      cudaFuncSetAttribute(router_topk_kernel<VPL, CPL_, PRE>, cudaFuncAttributePreferredSharedMemoryCarveout,  \
                           cudaSharedmemCarveoutMaxShared);                                                     \
      carveout_set = true;                                                                                      \
    }                                                                                                           \
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
  if (a.n <= 256) return launch_cpl<8, PRE>(a, st);
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
