// Expert-centric scheduling: a stable least-significant-digit radix sort of the (token, expert)
// pairs by expert id, followed by the CSR description of the expert segments.
//
// One digit pass = three kernels and no inter-block waiting:
//   radix_count   every tile (a contiguous run of pairs) histograms its digit into shared memory
//                 and writes its column of the [bins x tiles] count matrix.
//   radix_scan    one warp per bin row turns the row into exclusive prefixes over the tiles; the
//                 block that finishes last scans the bin totals ("last block done", nobody spins).
//   radix_scatter every tile ranks its pairs inside the tile with warp match operations
//                 (order preserving) and writes key and pair id to
//                 bin_base[digit] + tile_prefix[digit][tile] + rank.
// Digits are at most 11 bits wide, so expert tables up to 2^22 rows need two passes.
//
// The segment description is two more kernels: count segment heads per tile (+ last-block
// scan), then write expert ids / offsets / token ids / permuted weights (+ last-block maximum
// segment length).
#include "common.cuh"

namespace omni {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxBits = 11;
constexpr int kMaxBins = 1 << kMaxBits;

// workspace header (int32 words)
enum { HDR_TICKET0 = 0, HDR_WORDS = 16 };  // one ticket counter per kernel that uses "last block done"

struct Plan {
  int64_t P;
  int passes, bits[3], ipt, tile, tiles;
  size_t off_keysA, off_valsA, off_keysB, off_valsB, off_hist, off_binbase, off_tilecnt, total;
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

Plan make_plan(int64_t P, int64_t N) {
  Plan p{};
  p.P = P;
  int key_bits = 1;
  while ((int64_t(1) << key_bits) < N) ++key_bits;
  p.passes = ceil_div(key_bits, kMaxBits);
  // distribute the bits evenly over the passes: the first passes get the ceiling
  int left = key_bits;
  for (int i = 0; i < p.passes; ++i) {
    p.bits[i] = ceil_div(left, p.passes - i);
    left -= p.bits[i];
  }
  p.ipt = (P >= int64_t(148) * 2 * kThreads * 16) ? 16 : 4;
  p.tile = kThreads * p.ipt;
  p.tiles = static_cast<int>(ceil_div64(P > 0 ? P : 1, p.tile));
  size_t o = HDR_WORDS * sizeof(int32_t);
  o = align_up(o, 256);
  const size_t arr = align_up(static_cast<size_t>(P > 0 ? P : 1) * 4, 256);
  p.off_keysA = o, o += arr;
  p.off_valsA = o, o += arr;
  p.off_keysB = o, o += arr;
  p.off_valsB = o, o += arr;
  p.off_hist = o, o += align_up(static_cast<size_t>(kMaxBins) * p.tiles * 4, 256);
  p.off_binbase = o, o += align_up(static_cast<size_t>(2 * kMaxBins) * 4, 256);  // bin_base, bin_total
  p.off_tilecnt = o, o += align_up(static_cast<size_t>(p.tiles + 1) * 4, 256);
  p.total = o;
  return p;
}

// IPT keys of one thread at positions first + i * stride, all requested before any is used: one loop per key width
// (a width test per element would put every load behind a branch, and loads behind branches are issued one memory
// round trip after the other).  Positions at or past P yield `fill`.
template <int IPT>
__device__ __forceinline__ void load_keys(const void* keys, int is_i64, int64_t first, int64_t stride, int64_t P, int fill,
                                          int (&out)[IPT]) {
  if (is_i64) {
    const int64_t* k = reinterpret_cast<const int64_t*>(keys);
    int64_t v[IPT];
#pragma unroll
    for (int i = 0; i < IPT; ++i) v[i] = (first + i * stride) < P ? k[first + i * stride] : static_cast<int64_t>(fill);
#pragma unroll
    for (int i = 0; i < IPT; ++i) out[i] = static_cast<int>(v[i]);
  } else {
    const int32_t* k = reinterpret_cast<const int32_t*>(keys);
#pragma unroll
    for (int i = 0; i < IPT; ++i) out[i] = (first + i * stride) < P ? k[first + i * stride] : fill;
  }
}

// Block-wide exclusive scan of one int per thread; returns the exclusive prefix, total via reference.
__device__ __forceinline__ int block_exclusive_scan(int v, int* s_warp /*[kWarps]*/, int& total) {
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(FULL_MASK, inc, o);
    if (lane >= o) inc += y;
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  int wbase = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const int c = s_warp[w];
    if (w < warp) wbase += c;
    tot += c;
  }
  __syncthreads();
  total = tot;
  return wbase + inc - v;
}

// ---- pass kernel 1: per-tile digit histogram ---------------------------------------------------
template <int IPT>
__global__ void __launch_bounds__(kThreads) radix_count_kernel(
    const void* keys, int key_is_i64, int64_t P, int shift, int bits, int check_range, int num_experts,
    int* hist /*[bins][tiles]*/, int* status) {
  __shared__ int s_hist[kMaxBins];
  const int bins = 1 << bits, tiles = gridDim.x, tile = blockIdx.x;
  for (int b = threadIdx.x; b < bins; b += kThreads) s_hist[b] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(tile) * (kThreads * IPT);
  bool bad = false;
  int e[IPT];
  load_keys<IPT>(keys, key_is_i64, base + threadIdx.x, kThreads, P, 0, e);
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int64_t p = base + i * kThreads + threadIdx.x;
    if (p < P) {
      if (check_range && (e[i] < 0 || e[i] >= num_experts)) bad = true;
      atomicAdd(&s_hist[(static_cast<unsigned>(e[i]) >> shift) & (bins - 1)], 1);
    }
  }
  if (bad) atomicOr(status, OMNI_ST_BAD_EXPERT_INDEX);
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kThreads) hist[static_cast<size_t>(b) * tiles + tile] = s_hist[b];
}

// ---- pass kernel 2: exclusive prefixes of the count matrix ------------------------------------
// One warp per bin row: every lane owns a contiguous chunk of the row, sums it (independent loads),
// the lane sums are scanned across the warp, and the chunk is walked again to write the exclusive
// prefixes.  The block that finishes last scans the bin totals into bin_base.
__global__ void __launch_bounds__(kThreads) radix_scan_kernel(int* hist /*[bins][tiles]*/, int tiles, int bins,
                                                             int* bin_total /*[bins]*/, int* bin_base /*[bins]*/,
                                                             int* ticket) {
  __shared__ int s_scan[kWarps];
  __shared__ int s_last;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const int b = blockIdx.x * kWarps + warp;
  if (b < bins) {
    int* row = hist + static_cast<size_t>(b) * tiles;
    // chunk per lane, a multiple of 4 so that rows whose length is a multiple of 4 can move as int4
    const int per = ceil_div(ceil_div(tiles, 32), 4) * 4;
    const int lo = min(tiles, lane * per), hi = min(tiles, lo + per);
    const bool vec = (tiles & 3) == 0;  // then lo, hi and the row start are 16-byte aligned
    int sum = 0;
    if (vec) {
      const int4* r4 = reinterpret_cast<const int4*>(row + lo);
      const int n4 = (hi - lo) >> 2;
#pragma unroll 8
      for (int i = 0; i < n4; ++i) {
        const int4 v = r4[i];
        sum += v.x + v.y + v.z + v.w;
      }
    } else {
      for (int t = lo; t < hi; ++t) sum += row[t];
    }
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(FULL_MASK, inc, o);
      if (lane >= o) inc += y;
    }
    int run = inc - sum;
    if (vec) {
      int4* r4 = reinterpret_cast<int4*>(row + lo);
      const int n4 = (hi - lo) >> 2;
#pragma unroll 8
      for (int i = 0; i < n4; ++i) {
        const int4 v = r4[i];
        int4 o;
        o.x = run, o.y = run + v.x, o.z = o.y + v.y, o.w = o.z + v.z;
        run = o.w + v.w;
        r4[i] = o;
      }
    } else {
      for (int t = lo; t < hi; ++t) {
        const int v = row[t];
        row[t] = run;
        run += v;
      }
    }
    if (lane == 31) bin_total[b] = inc;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // exclusive scan of the bin totals (bins <= 2048 = 8 per thread)
  constexpr int PER = kMaxBins / kThreads;
  volatile int* tot = bin_total;
  int loc[PER], sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int bb = threadIdx.x * PER + j;
    loc[j] = bb < bins ? tot[bb] : 0;
    sum += loc[j];
  }
  int total;
  int run = block_exclusive_scan(sum, s_scan, total);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int bb = threadIdx.x * PER + j;
    if (bb < bins) bin_base[bb] = run;
    run += loc[j];
  }
  if (threadIdx.x == 0) *ticket = 0;  // ready for the next use of this counter
}

// ---- pass kernel 3: stable in-tile ranking + scatter --------------------------------------
template <int IPT>
__global__ void __launch_bounds__(kThreads) radix_scatter_kernel(
    const void* keys, int key_is_i64, const int* vals /*null: identity*/, int64_t P, int shift, int bits,
    const int* hist, const int* bin_base, int* out_keys, int* out_vals) {
  extern __shared__ uint16_t s_cnt[];  // [kWarps][bins]: pairs of each digit seen so far by each warp
  const int bins = 1 << bits, tiles = gridDim.x, tile = blockIdx.x;
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  for (int b = threadIdx.x; b < kWarps * bins; b += kThreads) s_cnt[b] = 0;
  __syncthreads();
  // warp w owns the contiguous run [w * 32 * IPT, (w + 1) * 32 * IPT) of the tile, item i of lane
  // l sits at offset i * 32 + l, so walking i upward visits the pairs in ascending pair order.
  const int64_t wbase = static_cast<int64_t>(tile) * (kThreads * IPT) + warp * (32 * IPT);
  uint16_t* cnt = s_cnt + warp * bins;
  int key[IPT], val[IPT];
  uint16_t rank[IPT];
  const unsigned lt_mask = (1u << lane) - 1u;
  // all loads of the tile first (see load_keys), then the order-preserving ranking, which is sequential by nature
  load_keys<IPT>(keys, key_is_i64, wbase + lane, 32, P, 0, key);
  if (vals) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) val[i] = (wbase + i * 32 + lane) < P ? vals[wbase + i * 32 + lane] : 0;
  } else {
#pragma unroll
    for (int i = 0; i < IPT; ++i) val[i] = static_cast<int>(wbase + i * 32 + lane);
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int64_t p = wbase + i * 32 + lane;
    const bool ok = p < P;
    const int d = ok ? ((static_cast<unsigned>(key[i]) >> shift) & (bins - 1)) : bins;  // bins = "none"
    const unsigned peers = __match_any_sync(FULL_MASK, d);
    const int before = ok ? cnt[d] : 0;
    __syncwarp();
    if (ok && (peers & lt_mask) == 0) cnt[d] = static_cast<uint16_t>(before + __popc(peers));
    __syncwarp();
    rank[i] = static_cast<uint16_t>(before + __popc(peers & lt_mask));
  }
  __syncthreads();
  // per digit: exclusive prefix over the warps (warp order = pair order)
  for (int b = threadIdx.x; b < bins; b += kThreads) {
    int run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = s_cnt[w * bins + b];
      s_cnt[w * bins + b] = static_cast<uint16_t>(run);
      run += c;
    }
  }
  __syncthreads();
  int dst[IPT];
#pragma unroll
  for (int i = 0; i < IPT; ++i) {  // the offsets of all items first: two dependent-free gathers per item
    const int d = (static_cast<unsigned>(key[i]) >> shift) & (bins - 1);
    dst[i] = bin_base[d] + hist[static_cast<size_t>(d) * tiles + tile] + cnt[d] + rank[i];
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int64_t p = wbase + i * 32 + lane;
    if (p < P) {
      out_keys[dst[i]] = key[i];
      out_vals[dst[i]] = val[i];
    }
  }
}

// ---- segments kernel 1: heads per tile + last-block scan ------------------------------------
template <int IPT>
__global__ void __launch_bounds__(kThreads) segment_count_kernel(const int* sorted_keys, int64_t P, int* tile_cnt /*[tiles+1]*/,
                                                                 int* ticket, int* meta) {
  __shared__ int s_scan[kWarps];
  __shared__ int s_last;
  const int tiles = gridDim.x, tile = blockIdx.x;
  const int64_t base = static_cast<int64_t>(tile) * (kThreads * IPT) + static_cast<int64_t>(threadIdx.x) * IPT;
  int heads = 0;
  int kv[IPT + 1];  // kv[i] = key at base + i - 1: every load before the first comparison
#pragma unroll
  for (int i = 0; i <= IPT; ++i) {
    const int64_t q = base + i - 1;
    kv[i] = (q >= 0 && q < P) ? sorted_keys[q] : -1;
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int64_t p = base + i;
    if (p < P && (p == 0 || kv[i + 1] != kv[i])) ++heads;
  }
  int total;
  block_exclusive_scan(heads, s_scan, total);
  if (threadIdx.x == 0) {
    tile_cnt[tile] = total;
    __threadfence();
    s_last = (atomicAdd(ticket, 1) == tiles - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // last block: exclusive scan of tile_cnt in place, U to meta[0]
  volatile int* tc = tile_cnt;
  int carry = 0;
  for (int t0 = 0; t0 < tiles; t0 += kThreads) {
    const int t = t0 + threadIdx.x;
    const int v = t < tiles ? tc[t] : 0;
    int tot;
    const int ex = block_exclusive_scan(v, s_scan, tot);
    if (t < tiles) tc[t] = carry + ex;
    carry += tot;
  }
  if (threadIdx.x == 0) {
    tc[tiles] = carry;
    meta[0] = carry;
    *ticket = 0;
  }
}

// ---- segments kernel 2: write the description -------------------------------------------------
template <int IPT>
__global__ void __launch_bounds__(kThreads) segment_write_kernel(
    const int* sorted_keys, const int* perm, int64_t P, int k, const void* weights, int wbytes,
    const int* tile_cnt, int* token_ids, void* sorted_weights, int* expert_ids, int* offsets,
    int* ticket, int* meta) {
  __shared__ int s_scan[kWarps];
  __shared__ int s_last;
  const int tiles = gridDim.x, tile = blockIdx.x;
  const int64_t base = static_cast<int64_t>(tile) * (kThreads * IPT) + static_cast<int64_t>(threadIdx.x) * IPT;
  int keyv[IPT];
  bool head[IPT];
  int heads = 0;
  int kv[IPT + 1], pr[IPT];  // keys at base - 1 .. base + IPT - 1 and the permutation: every load before its first use
#pragma unroll
  for (int i = 0; i <= IPT; ++i) {
    const int64_t q = base + i - 1;
    kv[i] = (q >= 0 && q < P) ? sorted_keys[q] : -1;
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) pr[i] = (base + i) < P ? perm[base + i] : 0;
  if (sorted_weights) {  // the permuted weights: gathers that depend on pr only
    if (wbytes == 4) {
      uint32_t wv[IPT];
#pragma unroll
      for (int i = 0; i < IPT; ++i) wv[i] = (base + i) < P ? reinterpret_cast<const uint32_t*>(weights)[pr[i]] : 0u;
#pragma unroll
      for (int i = 0; i < IPT; ++i)
        if (base + i < P) reinterpret_cast<uint32_t*>(sorted_weights)[base + i] = wv[i];
    } else {
      uint16_t wv[IPT];
#pragma unroll
      for (int i = 0; i < IPT; ++i) wv[i] = (base + i) < P ? reinterpret_cast<const uint16_t*>(weights)[pr[i]] : uint16_t(0);
#pragma unroll
      for (int i = 0; i < IPT; ++i)
        if (base + i < P) reinterpret_cast<uint16_t*>(sorted_weights)[base + i] = wv[i];
    }
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int64_t p = base + i;
    head[i] = false;
    if (p < P) {
      keyv[i] = kv[i + 1];
      head[i] = (p == 0) || (kv[i + 1] != kv[i]);
      heads += head[i];
      if (token_ids) token_ids[p] = pr[i] / k;
    }
  }
  int total;
  int r = tile_cnt[tile] + block_exclusive_scan(heads, s_scan, total);
  if (offsets) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (head[i]) {
        if (expert_ids) expert_ids[r] = keyv[i];
        offsets[r] = static_cast<int>(base + i);
        ++r;
      }
    }
  }
  if (!offsets) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1) == tiles - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // last block: offsets[U] = P and the longest segment
  const int U = tile_cnt[tiles];
  volatile int* off = offsets;
  if (threadIdx.x == 0) off[U] = static_cast<int>(P);
  __syncthreads();
  int mx = 0;
  for (int s = threadIdx.x; s < U; s += kThreads) mx = max(mx, off[s + 1] - off[s]);
  mx = __reduce_max_sync(FULL_MASK, mx);
  if (lane_id() == 0) s_scan[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 0; w < kWarps; ++w) mx = max(mx, s_scan[w]);
    meta[1] = mx;
    *ticket = 0;
  }
}

template <int IPT>
int run(const Plan& pl, const void* indices, int idx_is_i64, const void* weights, int wbytes, int k, int64_t N,
        int* perm, int* sorted_experts, int* token_ids, void* sorted_weights, int* expert_ids, int* offsets,
        int* meta, char* ws, cudaStream_t st) {
  int* hdr = reinterpret_cast<int*>(ws);
  int* keysA = reinterpret_cast<int*>(ws + pl.off_keysA);
  int* valsA = reinterpret_cast<int*>(ws + pl.off_valsA);
  int* keysB = reinterpret_cast<int*>(ws + pl.off_keysB);
  int* valsB = reinterpret_cast<int*>(ws + pl.off_valsB);
  int* hist = reinterpret_cast<int*>(ws + pl.off_hist);
  int* binbase = reinterpret_cast<int*>(ws + pl.off_binbase);
  int* bintotal = binbase + kMaxBins;
  int* tilecnt = reinterpret_cast<int*>(ws + pl.off_tilecnt);
  cudaMemsetAsync(hdr, 0, HDR_WORDS * sizeof(int), st);
  cudaMemsetAsync(meta, 0, 4 * sizeof(int), st);
  const void* in_keys = indices;
  int in_i64 = idx_is_i64;
  const int* in_vals = nullptr;
  int shift = 0;
  for (int pass = 0; pass < pl.passes; ++pass) {
    const bool last = pass == pl.passes - 1;
    int* ok = last ? sorted_experts : (pass == 0 ? keysA : keysB);
    int* ov = last ? perm : (pass == 0 ? valsA : valsB);
    const int bits = pl.bits[pass];
    radix_count_kernel<IPT><<<pl.tiles, kThreads, 0, st>>>(in_keys, in_i64, pl.P, shift, bits, pass == 0,
                                                         static_cast<int>(N), hist, meta + 2);
    radix_scan_kernel<<<ceil_div(1 << bits, kWarps), kThreads, 0, st>>>(hist, pl.tiles, 1 << bits, bintotal, binbase,
                                                                        hdr + HDR_TICKET0);
    const size_t smem = static_cast<size_t>(kWarps) * (size_t(1) << bits) * sizeof(uint16_t);
    radix_scatter_kernel<IPT><<<pl.tiles, kThreads, smem, st>>>(in_keys, in_i64, in_vals, pl.P, shift, bits, hist, binbase, ok, ov);
    in_keys = ok, in_i64 = 0, in_vals = ov;
    shift += bits;
  }
  if (!offsets && !token_ids && !sorted_weights) return check_launch("omni_schedule kernels");  // permutation only
  segment_count_kernel<IPT><<<pl.tiles, kThreads, 0, st>>>(sorted_experts, pl.P, tilecnt, hdr + HDR_TICKET0, meta);
  segment_write_kernel<IPT><<<pl.tiles, kThreads, 0, st>>>(sorted_experts, perm, pl.P, k, weights, wbytes, tilecnt, token_ids,
                                                         sorted_weights, expert_ids, offsets, hdr + HDR_TICKET0, meta);
  return check_launch("omni_schedule kernels");
}

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" size_t omni_schedule_workspace_bytes(int64_t num_pairs, int64_t num_experts) {
  if (num_pairs < 0 || num_experts < 1) return 0;
  return make_plan(num_pairs, num_experts).total;
}

extern "C" int omni_schedule(const void* indices, int idx_is_i64, const void* weights, int weight_elem_bytes,
                             int64_t num_tokens, int k, int64_t num_experts, int32_t* sorted_pair_ids,
                             int32_t* sorted_experts, int32_t* token_ids, void* sorted_weights,
                             int32_t* expert_ids, int32_t* offsets, int32_t* meta, void* workspace,
                             size_t workspace_bytes, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1, "num_tokens must be >= 0 and k >= 1");
  OMNI_REQUIRE(num_experts >= 1 && num_experts <= (int64_t(1) << 30), "num_experts must be in [1, 2^30]");
  const int64_t P = num_tokens * k;
  OMNI_REQUIRE(P < (int64_t(1) << 31) - 65536, "too many (token, expert) pairs: %lld", static_cast<long long>(P));
  OMNI_REQUIRE(meta, "meta must not be NULL");
  OMNI_REQUIRE((sorted_weights == nullptr) || (weights != nullptr), "sorted_weights needs weights");
  OMNI_REQUIRE(weights == nullptr || weight_elem_bytes == 2 || weight_elem_bytes == 4, "weight_elem_bytes must be 2 or 4");
  OMNI_REQUIRE((expert_ids == nullptr) || (offsets != nullptr), "expert_ids needs offsets");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (P == 0) {
    cudaMemsetAsync(meta, 0, 4 * sizeof(int), st);
    if (offsets) cudaMemsetAsync(offsets, 0, sizeof(int), st);
    return check_launch("omni_schedule (empty)");
  }
  OMNI_REQUIRE(indices && sorted_pair_ids && sorted_experts, "indices, sorted_pair_ids and sorted_experts must not be NULL");
  const Plan pl = make_plan(P, num_experts);
  OMNI_REQUIRE(workspace && workspace_bytes >= pl.total, "workspace too small: need %zu bytes", pl.total);
  OMNI_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  char* ws = static_cast<char*>(workspace);
  if (pl.ipt == 16)
    return run<16>(pl, indices, idx_is_i64, weights, weight_elem_bytes, k, num_experts, sorted_pair_ids, sorted_experts,
                   token_ids, sorted_weights, expert_ids, offsets, meta, ws, st);
  return run<4>(pl, indices, idx_is_i64, weights, weight_elem_bytes, k, num_experts, sorted_pair_ids, sorted_experts,
                token_ids, sorted_weights, expert_ids, offsets, meta, ws, st);
}

// ---------------------------------------------------------------------------------------------
// Scheduling without caller-provided scratch
// ---------------------------------------------------------------------------------------------
namespace omni {
namespace {

constexpr int64_t kStaticMaxPairs = 262144;            // largest T*k the built-in scratch can sort
constexpr size_t kStaticBytes = 6 * 1024 * 1024 + 512 * 1024;  // 6.5 MiB, held by every GPU that loads the library

// The scratch lives in the library image, not on the heap.  In host code this name is only a handle
// for the symbol: the device address has to be asked for with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
void* g_static_ptr[kMaxDevices] = {};

// Device address of the built-in scratch on the current device (looked up once per device).
int static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(-2, "cannot identify the current CUDA device");
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return fail(-2, "cudaGetSymbolAddress(built-in scratch) failed: %s", cudaGetErrorString(e));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return 0;
}

}  // namespace
}  // namespace omni

extern "C" int64_t omni_schedule_static_max_pairs(void) { return kStaticMaxPairs; }

extern "C" int omni_schedule_static(const void* indices, int idx_is_i64, const void* weights, int weight_elem_bytes,
                                    int64_t num_tokens, int k, int64_t num_experts, int32_t* sorted_pair_ids,
                                    int32_t* sorted_experts, int32_t* token_ids, void* sorted_weights,
                                    int32_t* expert_ids, int32_t* offsets, int32_t* meta, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1, "num_tokens must be >= 0 and k >= 1");
  const int64_t P = num_tokens * k;
  OMNI_REQUIRE(P <= kStaticMaxPairs,
               "omni_schedule_static sorts at most %lld (token, expert) pairs with its built-in scratch, got %lld; "
               "use omni_schedule with a caller-provided workspace",
               static_cast<long long>(kStaticMaxPairs), static_cast<long long>(P));
  OMNI_REQUIRE(num_experts >= 1 && num_experts <= (int64_t(1) << 30), "num_experts must be in [1, 2^30]");
  OMNI_REQUIRE(make_plan(P, num_experts).total <= kStaticBytes, "built-in scratch too small for this problem");
  void* ws = nullptr;
  if (int e = static_scratch(&ws)) return e;
  // Same kernels as omni_schedule; the counters that must start at zero are cleared on the stream
  // at the start of every call, the rest of the scratch is overwritten before it is read.
  return omni_schedule(indices, idx_is_i64, weights, weight_elem_bytes, num_tokens, k, num_experts, sorted_pair_ids,
                       sorted_experts, token_ids, sorted_weights, expert_ids, offsets, meta, ws, kStaticBytes, stream);
}
