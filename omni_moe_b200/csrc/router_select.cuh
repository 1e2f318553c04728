// Per-token product-key selection, shared by the stand-alone router kernel and by the fused
// router + routed-experts kernel.  One warp works on one token.
//
// The warp holds the two sub-key rows in registers, extracts the kk = min(sqrt_n, k) best sub-keys
// of each axis (score descending, index ascending), and then searches the kk x kk candidate sums
// for the k best (sum descending, flat expert index ascending).
//
// Search pruning.  In rank space (i = rank on x, j = rank on y) a cell can only be among the k
// best if (i+1)*(j+1) <= k, because every cell it dominates scores at least as much.  Only those
// ~k*ln(k) cells are materialised.  fp32 rounding can make a dominated cell *tie* with a cell
// outside that region, and the tie rule (lower flat index) could then prefer the outside cell, so
// after the pruned search the first cell outside the region in every row is tested against the
// k-th score; a token that shows such a tie is redone by an exact scan over all kk x kk cells.
#pragma once

#include "common.cuh"

namespace omni {
namespace sel {

constexpr int kMaxK = 128;
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


// Shared memory of one warp.
template <int VPL, int CPL>
struct WarpScratch {
  static constexpr bool kSmall = (VPL == 2) || (CPL == 2);
  __align__(16) unsigned long long pack[kSmall ? 64 : 2];
  uint32_t rk[CPL == 2 ? 64 : 1], rf[CPL == 2 ? 64 : 1];
  float sx[kMaxK], sy[kMaxK];
  int ix[kMaxK], iy[kMaxK];
};

// Shared memory of the block: the cells of the pruned region, i | j << 8 each.
struct RegionTable {
  uint16_t cell[kMaxCells];
  int rowstart[kMaxK + 1];
};

// Builds the region table (row i keeps columns [0, min(kk, k/(i+1)))).  All threads of the block
// must call it; it ends with a block barrier.
__device__ __forceinline__ void build_region_table(RegionTable& rt, int kk, int k, int warps_per_block) {
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < kk; ++i) {
      rt.rowstart[i] = acc;
      acc += min(kk, k / (i + 1));
    }
    rt.rowstart[kk] = acc;
  }
  __syncthreads();
  for (int i = warp; i < kk; i += warps_per_block) {
    const int st = rt.rowstart[i], cnt = rt.rowstart[i + 1] - st;
    for (int j = lane; j < cnt; j += 32) rt.cell[st + j] = static_cast<uint16_t>(i | (j << 8));
  }
  __syncthreads();
}

// Selects the k experts of token t.  On return lane (r % 32) holds, in slot r / 32, the score key
// (see float_to_key) and the flat expert index of rank r.
template <int VPL, int CPL, bool PRE>
__device__ __forceinline__ void select_token(const TopkArgs& a, int64_t t, WarpScratch<VPL, CPL>& w,
                                             const uint16_t* cell_table, uint32_t (&rkey)[kMaxK / 32],
                                             uint32_t (&rflat)[kMaxK / 32]) {
  constexpr bool kSmallAxis = VPL == 2;   // n <= 64: rank by counting instead of selection rounds
  constexpr bool kSmallCells = CPL == 2;  // <= 64 candidate cells: likewise
  const int lane = lane_id();
  const int n = a.n, k = a.k, kk = a.kk;
  float* sx = w.sx;
  float* sy = w.sy;
  int* ix = w.ix;
  int* iy = w.iy;

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
        w.pack[c] = mine[e];
      }
      __syncwarp();
      float* so = axis == 0 ? sx : sy;
      int* io = axis == 0 ? ix : iy;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int r = rank_among_64(w.pack, mine[e]);
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
      const int cell = cell_table[c];
      const int i = cell & 0xff, j = cell >> 8;
      ckey[q] = float_to_key(__fadd_rn(sx[i], sy[j]));
      cflat[q] = static_cast<uint32_t>(ix[i]) * n + iy[j];
    } else {
      ckey[q] = 0;
      cflat[q] = 0xffffffffu;
    }
    lmax = max(lmax, ckey[q]);
  }
#pragma unroll
  for (int s = 0; s < kMaxK / 32; ++s) rkey[s] = 0, rflat[s] = 0;
  uint32_t last_key = 0;
  if constexpr (kSmallCells) {
    unsigned long long mine[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      // padding cells have key 0 and can never outrank a real one; real cells differ in `flat`
      mine[q] = (static_cast<unsigned long long>(ckey[q]) << 32) | (0xffffffffu - cflat[q]);
      w.pack[q * 32 + lane] = mine[q];
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int r = rank_among_64(w.pack, mine[q]);
      if (r < k && ckey[q] != 0) w.rk[r] = ckey[q], w.rf[r] = cflat[q];
    }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int r = s * 32 + lane;
      if (r < k) rkey[s] = w.rk[r], rflat[s] = w.rf[r];
    }
    last_key = w.rk[k - 1];
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

}

inline int region_cells(int kk, int k) {
  int c = 0;
  for (int i = 0; i < kk; ++i) c += (k / (i + 1) < kk) ? k / (i + 1) : kk;
  return c;
}

}  // namespace sel
}  // namespace omni
