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

#ifdef OMNI_TUNING
// tuning builds only: clocks spent by all warps in the parts of select_token (rows, axis selection, candidates,
// final ranking, tie check), and the number of tokens
__device__ unsigned long long g_sel_prof[4096 * 8];  // spread over 4096 slots so that the adds do not queue up
#define SEL_SLOT ((blockIdx.x * 4 + (threadIdx.x >> 5)) & 4095)
#define SEL_TIC(v) const long long v = clock64()
#define SEL_TOC(i, v) if (lane_id() == 0) atomicAdd(&g_sel_prof[SEL_SLOT * 8 + i], static_cast<unsigned long long>(clock64() - v))
#else
#define SEL_TIC(v)
#define SEL_TOC(i, v)
#endif

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


// Final stage of warp_select_sorted: the K winners sit packed (key << 32 | ~id, all distinct) in s_tmp[0, K);
// lane l ranks the entries l, 32 + l, ... (NS of them) by counting the winners that beat them.
template <int NS, bool AS_FLOAT>
__device__ __forceinline__ void rank_winners(unsigned long long* s_tmp, int K, uint32_t* out_key, uint32_t* out_id) {
  const int lane = lane_id();
  unsigned long long mine[NS];
  int rank[NS];
#pragma unroll
  for (int q = 0; q < NS; ++q) {
    const int r = q * 32 + lane;
    mine[q] = r < K ? s_tmp[r] : 0ull;
    rank[q] = 0;
  }
  if ((K & 1) && lane == 0) s_tmp[K] = 0ull;  // K <= kMaxK - 1 when odd: the pairwise reads may touch one slot past the end
  __syncwarp();
  const ulonglong2* p = reinterpret_cast<const ulonglong2*>(s_tmp);
  const int pairs = (K + 1) >> 1;
  for (int j = 0; j < pairs; ++j) {
    const ulonglong2 o = p[j];
#pragma unroll
    for (int q = 0; q < NS; ++q) rank[q] += (o.x > mine[q]) + (o.y > mine[q]);
  }
#pragma unroll
  for (int q = 0; q < NS; ++q) {
    if (q * 32 + lane < K) {
      const uint32_t kq = static_cast<uint32_t>(mine[q] >> 32);
      out_key[rank[q]] = AS_FLOAT ? __float_as_uint(key_to_float(kq)) : kq;
      out_id[rank[q]] = 0xffffffffu - static_cast<uint32_t>(mine[q]);
    }
  }
}

// Sorted top-K of the E * 32 entries a warp holds in registers (entry = 32-bit key, larger wins, and a
// 32-bit id that is unique among the entries, smaller wins on equal keys; key 0 = absent).
//   1. radix select: a bitwise search for the K-th largest key tau (per step every lane counts its
//      entries >= trial, one warp reduction adds the counts); only the bits in which the largest and
//      the smallest key differ are searched;
//   2. entries equal to tau are admitted by ascending id until K entries are in (a second bitwise
//      search, on the ids, only when more entries tie at tau than there is room for);
//   3. the K admitted entries are compacted into shared memory and ranked by counting.
// out_key[r], out_id[r] receive rank r (AS_FLOAT: the key converted back to its float).
template <int E, bool AS_FLOAT, bool FEW = false>
__device__ __forceinline__ void warp_select_sorted(const uint32_t (&key)[E], const uint32_t (&id)[E], int K,
                                                   unsigned long long* s_tmp /*[kMaxK]*/, uint32_t* out_key,
                                                   uint32_t* out_id) {
  const int lane = lane_id();
  if (FEW && K <= 16) {
    // Shortcut for few winners (compiled in only where the caller asks: it costs registers): the K-th largest of the 32 per-lane maxima is a lower bound of the K-th
    // largest entry (K lanes hold an entry at least that large).  Usually only a few more than K entries
    // reach it; if at most 64 do, they are compacted and ranked by counting like a small row, with the
    // same (key, id) order as the general path.  Otherwise (many ties) the general path below runs.
    uint32_t lmax = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) lmax = max(lmax, key[e]);
    // rank of this lane's maximum among the 32 (ties: lower lane first), read back as eight 128-bit words
    uint32_t* s_max = reinterpret_cast<uint32_t*>(s_tmp);
    s_max[lane] = lmax;
    __syncwarp();
    int lrank = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint4 o = reinterpret_cast<const uint4*>(s_max)[q];
      const int j = 4 * q;
      lrank += (o.x > lmax) || (o.x == lmax && j < lane);
      lrank += (o.y > lmax) || (o.y == lmax && j + 1 < lane);
      lrank += (o.z > lmax) || (o.z == lmax && j + 2 < lane);
      lrank += (o.w > lmax) || (o.w == lmax && j + 3 < lane);
    }
    const unsigned who = __ballot_sync(FULL_MASK, lrank == K - 1);
    const uint32_t bound = __shfl_sync(FULL_MASK, lmax, __ffs(who) - 1);
    int cnt = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) cnt += (key[e] >= bound) && key[e] != 0;
    const int total = __reduce_add_sync(FULL_MASK, cnt);
    if (bound != 0 && total <= 64) {
      const unsigned lt_mask = (1u << lane) - 1u;
      __syncwarp();  // every lane has read s_max
      int base = 0;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const bool in = (key[e] >= bound) && key[e] != 0;
        const unsigned m = __ballot_sync(FULL_MASK, in);
        if (in) s_tmp[base + __popc(m & lt_mask)] = (static_cast<unsigned long long>(key[e]) << 32) | (0xffffffffu - id[e]);
        base += __popc(m);
      }
      if ((total & 1) && lane == 0) s_tmp[total] = 0ull;  // the pairwise reads below may touch one slot past the end
      __syncwarp();
      // rank the `total` candidates among themselves (distinct packed values): slot lane and, if there are
      // more than 32, slot 32 + lane; only the live slots are compared against
      const int pairs = (total + 1) >> 1;
      const int slots = total > 32 ? 2 : 1;
      for (int q = 0; q < slots; ++q) {
        const int slot = q * 32 + lane;
        const unsigned long long mine = slot < total ? s_tmp[slot] : 0ull;
        int r = 0;
        const ulonglong2* p = reinterpret_cast<const ulonglong2*>(s_tmp);
        for (int j = 0; j < pairs; ++j) {
          const ulonglong2 o = p[j];
          r += (o.x > mine) + (o.y > mine);
        }
        if (slot < total && r < K) {
          const uint32_t kq = static_cast<uint32_t>(mine >> 32);
          out_key[r] = AS_FLOAT ? __float_as_uint(key_to_float(kq)) : kq;
          out_id[r] = 0xffffffffu - static_cast<uint32_t>(mine);
        }
      }
      __syncwarp();
      return;
    }
    __syncwarp();  // s_max is dead before the general path reuses the scratch
  }
  uint32_t kmax = 0, kmin = 0xffffffffu;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    kmax = max(kmax, key[e]);
    if (key[e]) kmin = min(kmin, key[e]);
  }
  kmax = __reduce_max_sync(FULL_MASK, kmax);
  kmin = __reduce_min_sync(FULL_MASK, kmin);
  const uint32_t diff = kmax ^ kmin;
  uint32_t tau = kmax;
  if (diff) {
    const int hb = 31 - __clz(diff);  // highest bit in which present keys differ
    tau = hb == 31 ? 0u : (kmax >> (hb + 1)) << (hb + 1);
    for (int bit = hb; bit >= 0; --bit) {
      const uint32_t trial = tau | (1u << bit);
      int c = 0;
#pragma unroll
      for (int e = 0; e < E; ++e) c += key[e] >= trial;
      c = __reduce_add_sync(FULL_MASK, c);
      if (c >= K) tau = trial;
      // exactly K keys reach the prefix found so far: they are the K winners whatever the lower bits of the K-th
      // key are (tau is then a lower bound of it, not the key itself; the admission below only asks key >= tau)
      if (c == K) break;
    }
  }
  int c_gt = 0, c_eq = 0;
#pragma unroll
  for (int e = 0; e < E; ++e) c_gt += key[e] > tau, c_eq += key[e] == tau;
  c_gt = __reduce_add_sync(FULL_MASK, c_gt);
  c_eq = __reduce_add_sync(FULL_MASK, c_eq);
  const int room = K - c_gt;  // entries equal to tau that are admitted (>= 1)
  uint32_t id_thr = 0xffffffffu;
  if (c_eq > room) {
    uint32_t lo = 0;  // becomes the room-th smallest id among the ties
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t trial = lo | (1u << bit);
      int c = 0;
#pragma unroll
      for (int e = 0; e < E; ++e) c += (key[e] == tau) && (id[e] < trial);
      if (__reduce_add_sync(FULL_MASK, c) < room) lo = trial;
    }
    id_thr = lo;
  }
  const unsigned lt_mask = (1u << lane) - 1u;
  int base = 0;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const bool in = key[e] > tau || (key[e] == tau && id[e] <= id_thr);
    const unsigned m = __ballot_sync(FULL_MASK, in);
    if (in) s_tmp[base + __popc(m & lt_mask)] = (static_cast<unsigned long long>(key[e]) << 32) | (0xffffffffu - id[e]);
    base += __popc(m);
  }
  __syncwarp();
  // rank the K admitted entries among themselves; NS = ceil(K / 32) slots per lane, two entries per shared-memory read
  const int nslot = (K + 31) >> 5;
  if (nslot == 1) rank_winners<1, AS_FLOAT>(s_tmp, K, out_key, out_id);
  else if (nslot == 2) rank_winners<2, AS_FLOAT>(s_tmp, K, out_key, out_id);
  else rank_winners<kMaxK / 32, AS_FLOAT>(s_tmp, K, out_key, out_id);
  __syncwarp();
}

// Shared memory of one warp.  KCAP bounds kk = min(sqrt_n, k), the sub-keys kept per axis; a kernel that
// only serves small k can shrink it.
template <int VPL, int CPL, int KCAP = kMaxK>
struct WarpScratch {
  static constexpr bool kAllSmall = (VPL == 2) && (CPL == 2);
  __align__(16) unsigned long long pack[kAllSmall ? 64 : kMaxK];  // ranking scratch
  uint32_t rk[CPL == 2 ? 64 : kMaxK], rf[CPL == 2 ? 64 : kMaxK];  // selected (score key, flat index) by rank
  float sx[KCAP], sy[KCAP];
  int ix[KCAP], iy[KCAP];
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
// The same ranking on the 32-bit keys alone (half the compare work).  Entries with equal keys get
// equal ranks, so the caller must check that the ranks it uses are distinct and fall back to the
// packed 64-bit ranking when they are not.
__device__ __forceinline__ int rank32_among_64(const uint32_t* all, uint32_t mine) {
  int rank = 0;
  const uint4* p = reinterpret_cast<const uint4*>(all);
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    const uint4 o = p[q];
    rank += (o.x > mine) + (o.y > mine) + (o.z > mine) + (o.w > mine);
  }
  return rank;
}
// True if, over the warp, exactly `want` of the given ranks are below `want` and they are all
// different (want <= 32): then the `want` best entries are strictly ordered by key alone.
__device__ __forceinline__ bool ranks_distinct(int r0, int r1, int want) {
  const unsigned bits = (r0 < want ? 1u << r0 : 0u) | (r1 < want ? 1u << r1 : 0u);
  const unsigned mask = __reduce_or_sync(FULL_MASK, bits);
  const int cnt = __reduce_add_sync(FULL_MASK, (r0 < want) + (r1 < want));
  return cnt == want && __popc(mask) == want;
}

// Both axes of a token at once, for rows of at most 64 logits (two per lane) and kk <= 32: loads, BatchNorm fold,
// log-softmax and the rank-by-counting of the two axes are written side by side, so that their dependency chains
// (two warp reductions, a logarithm, the ranking) overlap instead of following one another.  Same arithmetic, in the
// same order per axis, as the one-axis-at-a-time code in select_token.  Returns a mask of the axes whose best kk
// sub-keys are strictly ordered by key alone and were written to (sx, ix) / (sy, iy); an axis with a tie among its
// best kk is left to the caller's exact path.
template <class Scratch>
__device__ __forceinline__ unsigned select_axes_small(const TopkArgs& a, int64_t t, Scratch& w) {
  const int lane = lane_id();
  const int n = a.n, kk = a.kk;
  const float* row = reinterpret_cast<const float*>(a.in_x) + t * a.ld_in;
  float v[2][2];
#pragma unroll
  for (int ax = 0; ax < 2; ++ax)
#pragma unroll
    for (int e = 0; e < 2; ++e) v[ax][e] = (e * 32 + lane) < n ? __ldg(row + ax * n + e * 32 + lane) : -INFINITY;
  if (a.bn_scale) {
    float sc[2][2], sh[2][2];
#pragma unroll
    for (int ax = 0; ax < 2; ++ax)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int c = e * 32 + lane;
        sc[ax][e] = c < n ? __ldg(a.bn_scale + ax * n + c) : 1.f;
        sh[ax][e] = c < n ? __ldg(a.bn_shift + ax * n + c) : 0.f;
      }
#pragma unroll
    for (int ax = 0; ax < 2; ++ax)
#pragma unroll
      for (int e = 0; e < 2; ++e) v[ax][e] = __fmaf_rn(v[ax][e], sc[ax][e], sh[ax][e]);
  }
  float mx[2], sum[2], lse[2];
#pragma unroll
  for (int ax = 0; ax < 2; ++ax) mx[ax] = fmaxf(fmaxf(-INFINITY, v[ax][0]), v[ax][1]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int ax = 0; ax < 2; ++ax) mx[ax] = fmaxf(mx[ax], __shfl_xor_sync(FULL_MASK, mx[ax], o));
#pragma unroll
  for (int ax = 0; ax < 2; ++ax) {
    sum[ax] = 0.f;
#pragma unroll
    for (int e = 0; e < 2; ++e)
      if (e * 32 + lane < n) sum[ax] += __expf(v[ax][e] - mx[ax]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int ax = 0; ax < 2; ++ax) sum[ax] += __shfl_xor_sync(FULL_MASK, sum[ax], o);
#pragma unroll
  for (int ax = 0; ax < 2; ++ax) lse[ax] = logf(sum[ax]);
  uint32_t key[2][2];
  uint32_t* k32 = reinterpret_cast<uint32_t*>(w.pack);  // 64 keys of the x axis, then 64 of the y axis
#pragma unroll
  for (int ax = 0; ax < 2; ++ax)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int c = e * 32 + lane;
      if (c < n) {
        const float lp = (v[ax][e] - mx[ax]) - lse[ax];
        if (a.lp_out) a.lp_out[t * (2 * n) + ax * n + c] = lp;
        key[ax][e] = float_to_key(lp);
      } else {
        key[ax][e] = 0;
      }
      k32[ax * 64 + c] = key[ax][e];
    }
  __syncwarp();
  int r[2][2];
#pragma unroll
  for (int ax = 0; ax < 2; ++ax)
#pragma unroll
    for (int e = 0; e < 2; ++e) r[ax][e] = rank32_among_64(k32 + ax * 64, key[ax][e]);
  unsigned done = 0;
#pragma unroll
  for (int ax = 0; ax < 2; ++ax) {
    if (ranks_distinct(r[ax][0], r[ax][1], kk)) {
      float* so = ax == 0 ? w.sx : w.sy;
      int* io = ax == 0 ? w.ix : w.iy;
      if (r[ax][0] < kk) so[r[ax][0]] = key_to_float(key[ax][0]), io[r[ax][0]] = lane;
      if (r[ax][1] < kk) so[r[ax][1]] = key_to_float(key[ax][1]), io[r[ax][1]] = 32 + lane;
      done |= 1u << ax;
    }
  }
  __syncwarp();
  return done;
}

template <int VPL, int CPL, bool PRE, class Scratch = WarpScratch<VPL, CPL>>
__device__ __forceinline__ void select_token(const TopkArgs& a, int64_t t, Scratch& w,
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
  unsigned axes_done = 0;
  if constexpr (kSmallAxis && PRE) {
    if (kk <= 32) axes_done = select_axes_small(a, t, w);  // both axes side by side; ties are left to the loop below
  }
#pragma unroll 1
  for (int axis = 0; axis < 2; ++axis) {
    if ((axes_done >> axis) & 1) continue;
    uint32_t key[VPL];
    SEL_TIC(c_rows);
    if (PRE) {
      const float* row = reinterpret_cast<const float*>(a.in_x) + t * a.ld_in + axis * n;
      float v[VPL];
      float mx = -INFINITY;
      // Every load of the row is issued before any value is used (predicated loads, no branch in between): with a
      // load and its use in the same conditional block the compiler keeps them in program order and the row costs
      // VPL memory round trips instead of one.
#pragma unroll
      for (int e = 0; e < VPL; ++e) {
        const int c = e * 32 + lane;
        v[e] = c < n ? __ldg(row + c) : -INFINITY;
      }
      if (a.bn_scale) {
        float sc[VPL], sh[VPL];
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
          const int c = e * 32 + lane;
          sc[e] = c < n ? __ldg(a.bn_scale + axis * n + c) : 1.f;
          sh[e] = c < n ? __ldg(a.bn_shift + axis * n + c) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < VPL; ++e) v[e] = __fmaf_rn(v[e], sc[e], sh[e]);  // columns past n stay -inf
      }
#pragma unroll
      for (int e = 0; e < VPL; ++e) mx = fmaxf(mx, v[e]);
      mx = warp_max(mx);
      SEL_TOC(6, c_rows);  // tuning: loads + max only
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < VPL; ++e)
        if (e * 32 + lane < n) sum += __expf(v[e] - mx);  // ex2-based: 2 ulp, the sum only shifts all log-probs
      sum = warp_sum(sum);
      const float lse = logf(sum);
      SEL_TOC(7, c_rows);  // tuning: ... + exp / sum / log
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
      // one loop per element type, loads first (see above): a type test per element would put every load behind a branch
      float f[VPL];
      if (a.in_dtype == OMNI_F32) {
        const float* p = reinterpret_cast<const float*>(base) + t * a.ld_in;
#pragma unroll
        for (int e = 0; e < VPL; ++e) f[e] = (e * 32 + lane) < n ? __ldg(p + e * 32 + lane) : 0.f;
      } else if (a.in_dtype == OMNI_BF16) {
        const unsigned short* p = reinterpret_cast<const unsigned short*>(base) + t * a.ld_in;
        unsigned short h[VPL];
#pragma unroll
        for (int e = 0; e < VPL; ++e) h[e] = (e * 32 + lane) < n ? __ldg(p + e * 32 + lane) : static_cast<unsigned short>(0);
#pragma unroll
        for (int e = 0; e < VPL; ++e) f[e] = __uint_as_float(static_cast<uint32_t>(h[e]) << 16);
      } else {
        const __half* p = reinterpret_cast<const __half*>(base) + t * a.ld_in;
        __half h[VPL];
#pragma unroll
        for (int e = 0; e < VPL; ++e) h[e] = (e * 32 + lane) < n ? __ldg(p + e * 32 + lane) : __half(0.f);
#pragma unroll
        for (int e = 0; e < VPL; ++e) f[e] = __half2float(h[e]);
      }
#pragma unroll
      for (int e = 0; e < VPL; ++e) key[e] = (e * 32 + lane) < n ? float_to_key(f[e]) : 0u;
    }
    SEL_TOC(0, c_rows);
    SEL_TIC(c_axis);
    if constexpr (kSmallAxis) {
      float* so = axis == 0 ? sx : sy;
      int* io = axis == 0 ? ix : iy;
      bool done = false;
      if (kk <= 32) {  // fast path: rank on the keys alone, valid when no tie touches the best kk
        uint32_t* k32 = reinterpret_cast<uint32_t*>(w.pack);
        k32[lane] = key[0], k32[32 + lane] = key[1];
        __syncwarp();
        const int r0 = rank32_among_64(k32, key[0]), r1 = rank32_among_64(k32, key[1]);
        done = ranks_distinct(r0, r1, kk);
        if (done) {
          if (r0 < kk) so[r0] = key_to_float(key[0]), io[r0] = lane;
          if (r1 < kk) so[r1] = key_to_float(key[1]), io[r1] = 32 + lane;
        }
        __syncwarp();
      }
      if (!done) {
        unsigned long long mine[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t c = e * 32 + lane;
          mine[e] = (static_cast<unsigned long long>(key[e]) << 32) | (0xffffffffu - c);
          w.pack[c] = mine[e];
        }
        __syncwarp();
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int r = rank_among_64(w.pack, mine[e]);
          if (r < kk) so[r] = key_to_float(key[e]), io[r] = e * 32 + lane;
        }
        __syncwarp();
      }
    } else {
      uint32_t sub[VPL];
#pragma unroll
      for (int e = 0; e < VPL; ++e) sub[e] = e * 32 + lane;
      warp_select_sorted<VPL, true, (VPL <= 8)>(key, sub, kk, w.pack, reinterpret_cast<uint32_t*>(axis == 0 ? sx : sy),
                                    reinterpret_cast<uint32_t*>(axis == 0 ? ix : iy));
    }
    SEL_TOC(1, c_axis);
  }
  __syncwarp();
  SEL_TIC(c_cand);

  // ---- pruned candidate search ----------------------------------------------------------
  uint32_t ckey[CPL], cflat[CPL];
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
  }
#pragma unroll
  for (int s = 0; s < kMaxK / 32; ++s) rkey[s] = 0, rflat[s] = 0;
  uint32_t last_key = 0;
  SEL_TOC(2, c_cand);
  SEL_TIC(c_rank);
  if constexpr (kSmallCells) {
    bool done = false;
    if (k <= 32) {  // fast path on the score keys alone (see the axis selection above)
      uint32_t* k32 = reinterpret_cast<uint32_t*>(w.pack);
      k32[lane] = ckey[0], k32[32 + lane] = ckey[1];
      __syncwarp();
      const int r0 = rank32_among_64(k32, ckey[0]), r1 = rank32_among_64(k32, ckey[1]);
      done = ranks_distinct(r0, r1, k);
      if (done) {
        if (r0 < k) w.rk[r0] = ckey[0], w.rf[r0] = cflat[0];
        if (r1 < k) w.rk[r1] = ckey[1], w.rf[r1] = cflat[1];
      }
      __syncwarp();
    }
    if (!done) {
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
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int r = s * 32 + lane;
      if (r < k) rkey[s] = w.rk[r], rflat[s] = w.rf[r];
    }
    last_key = w.rk[k - 1];
  } else {
    warp_select_sorted<CPL, false>(ckey, cflat, k, w.pack, w.rk, w.rf);
#pragma unroll
    for (int s = 0; s < kMaxK / 32; ++s) {
      const int r = s * 32 + lane;
      if (r < k) rkey[s] = w.rk[r], rflat[s] = w.rf[r];
    }
    last_key = w.rk[k - 1];
  }

  SEL_TOC(3, c_rank);
  SEL_TIC(c_tie);
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
  SEL_TOC(4, c_tie);
#ifdef OMNI_TUNING
  if (lane_id() == 0) atomicAdd(&g_sel_prof[SEL_SLOT * 8 + 5], 1ull);
#endif
}

inline int region_cells(int kk, int k) {
  int c = 0;
  for (int i = 0; i < kk; ++i) c += (k / (i + 1) < kk) ? k / (i + 1) : kk;
  return c;
}

}  // namespace sel
}  // namespace omni
