// bf16 GEMMs of the layer on the 5th-generation tensor cores: D[M, N] = A[M, K] . B[N, K]^T.
//
// Both operands are K-major (row-major activations and nn.Linear weights), so a tile of either is
// `rows x 64` bf16 = rows x 128 bytes, fetched by one TMA box with the 128-byte swizzle and fed to
// tcgen05.mma straight from shared memory.  The accumulator lives in tensor memory (TMEM); the
// epilogue warps read it back with tcgen05.ld and apply the fused tail of the op:
//   EPI_F32     store fp32 (router gate logits; B comes from two weight matrices, x and y axis)
//   EPI_SWIGLU  B tile = 128 rows of Wg next to 128 rows of Wu; writes silu(g) * u as bf16
//   EPI_RES     adds an optional fp32 residual, writes bf16 (down projection + expert states)
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer (one lane): fills a ring of shared-memory stages
//   warp 1      allocates TMEM; one lane issues tcgen05.mma and commits to the stage / accumulator barriers
//   warps 2-9   epilogue: a warp may read the 32 TMEM lanes (= tile rows) its warp id modulo 4 selects;
//               two warps share a lane quarter and split the columns
// Two accumulators alternate, so the epilogue of tile i overlaps the MMAs of tile i+1.
// In the CTA-pair kernels the bf16 output (and the fp32 router logits) leave through a swizzled shared-memory
// staging buffer per epilogue warp and TMA stores (store_tile_tma); outputs that do not qualify and the
// single-CTA kernels store from registers with 256-bit accesses (store_tile).
//
// Every mbarrier wait is bounded.  A wait that runs out sets OMNI_ST_WAIT_TIMEOUT in the status
// word and raises a CTA-wide abort flag that turns all later waits into no-ops, so the kernel still
// drains, frees its TMEM and returns; the results of such a launch are garbage and the host sees the flag.
// The MLP GEMMs normally run the CTA-pair variant further down (cta_group::2).
// No load in this file uses cluster multicast.
#include <cstdlib>

#include "tcgen05.cuh"

namespace omni {
namespace {

using namespace tc;
constexpr int kEpiWarps = 8;  // two per TMEM lane quarter, each draining half of the columns
constexpr int kThreads = 64 + 32 * kEpiWarps;

enum { EPI_F32 = 0, EPI_SWIGLU = 1, EPI_RES = 2, EPI_SWIGLU_CLAMP = 3 };
// EPI_SWIGLU_CLAMP is EPI_SWIGLU with gate and up limited to [-limit, limit] before the activation; a
// separate instantiation, so the kernels of the common no-clamp case are compiled without it.
__host__ __device__ constexpr bool is_swiglu(int epi) { return epi == EPI_SWIGLU || epi == EPI_SWIGLU_CLAMP; }

struct GemmArgs {
  int M, N, K;          // N: logical output columns (EPI_SWIGLU: activation columns; EPI_F32 dual: per-axis columns)
  int dual;             // EPI_F32: 1 = two B matrices of N rows each, outputs side by side (ldc >= 2N)
  int tiles_m, tiles_n; // tiles_n counts tiles over all axes
  int tiles_n_axis;     // tiles per axis (EPI_F32 dual), else tiles_n
  float limit;          // EPI_SWIGLU_CLAMP: gate and up are limited to [-limit, limit] before the activation
  void* out;
  int64_t ldo;
  const float* residual;  // EPI_RES
  int64_t ldr;
  int tma_out;            // pair kernel: 1 = bf16 output tiles leave through shared memory and TMA stores
  int tma_logits;         // pair kernel: 1 = the fp32 router logits do too (tensor map tm_lg)
  void* gu_out;           // EPI_SWIGLU: if set, [M, 2N] bf16 that also receives the gate | up pre-activations
  int64_t ldgu;
  // router tile columns of the fused gate/up + router-gate launch (pair kernel, EPI_SWIGLU only)
  int router_tiles;       // tile columns holding router sub-keys (0 = none); they come first in tile order
  int router_n;           // sqrt_n; kernels without router tiles and with a transposed B: k_split (0 = one B matrix)
  float* logits;          // [M, 2 * sqrt_n]
  const int* enable;      // gemm_kernel: if set and *enable == 0 the launch does nothing (decided by an earlier kernel)
  int* status;
#ifdef OMNI_TUNING
  long long* prof;  // tuning builds: per-CTA cycle counters (8 words per CTA), normally null
  int knobs;        // tuning builds: 1 = no TMA loads (MMAs run on stale tiles), 2 = no MMAs; normally 0
  int grid_limit;   // tuning builds: cap on CTAs (pairs for the pair kernel); 0 = none
#endif
};

// The cycle counters and switches used while tuning exist only in builds with -DOMNI_TUNING; in the default build
// they are compile-time constants and every branch on them disappears.
#ifdef OMNI_TUNING
#define G_PROF (g.prof)
#define G_KNOBS (g.knobs)
#define G_GRID_LIMIT (g.grid_limit)
#else
#define G_PROF (static_cast<long long*>(nullptr))
#define G_KNOBS 0
#define G_GRID_LIMIT 0
#endif

// Cycle accounting for tuning builds: adds the cycles spent in `stmt` to `acc` when profiling is on.
#ifdef OMNI_TUNING
#define OMNI_TIMED(acc, stmt)                 \
  do {                                        \
    if (g.prof) {                             \
      const long long t0_ = clock64();        \
      stmt;                                   \
      acc += clock64() - t0_;                 \
    } else {                                  \
      stmt;                                   \
    }                                         \
  } while (0)
#else
#define OMNI_TIMED(acc, stmt) \
  do {                        \
    stmt;                     \
  } while (0)
#endif

// Tile order.  Tiles are handed out in groups of kGroupM tile rows: inside a group the column index
// advances slowest within a row block, so the CTAs running at any moment share a few A tiles and a few
// B tiles, and a group's A rows stay in L2 while the whole width of B sweeps past them.  (With plain
// row-fastest order a 65536-token activation matrix is re-read from HBM once per tile column.)
constexpr int kGroupM = 8;
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kGroupM * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int rows = min(kGroupM, tiles_m - first_m);  // the last group may be short
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

template <int BN>
struct Cfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;  // two accumulators; 128, 256 or 512: powers of two
  static constexpr int kBarBytes = 1024;
  static constexpr int kSmem = kStages * kStage + kBarBytes + 1024;  // + slack to align the base to 1024
};

// 256-bit store of eight 32-bit words (a whole 32-byte sector); ptr must be 32-byte aligned.
__device__ __forceinline__ void st256(void* ptr, const uint32_t (&p)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(p[0]), "r"(p[1]), "r"(p[2]), "r"(p[3]),
               "r"(p[4]), "r"(p[5]), "r"(p[6]), "r"(p[7])
               : "memory");
}

// silu(gate) * up of one 32-column chunk.  CLAMP limits gate and up to [-limit, limit] first, as the
// reference's activation does (compute_silu_mul, omni_moe/ops/triton/omni_mlp.py:54-61); the registers
// keep the unclamped values (the training forward saves those).
template <bool CLAMP>
__device__ __forceinline__ void swiglu_chunk(const uint32_t (&ra)[32], const uint32_t (&rb)[32], float limit, float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float a = __uint_as_float(ra[i]), b = __uint_as_float(rb[i]);
    if (CLAMP) a = fminf(fmaxf(a, -limit), limit), b = fminf(fmaxf(b, -limit), limit);
    v[i] = silu_fast(a) * b;
  }
}

// Drains this warp's share of one accumulator tile: its 32 rows (TMEM lane quarter) and the column
// chunks [c_begin, c_begin + 32 * NCH).  The TMEM load of chunk i+1 and the residual fetch of
// chunk i are in flight while chunk i-1 is converted and stored.
// taddr: TMEM address of column 0 of the accumulator in this warp's lane quarter; row: global row
// of this thread; output columns start at col_tile and are clipped to col_lim.
template <int BN, int EPI, int NCH>
__device__ __forceinline__ void store_tile(uint32_t taddr, int row, int col_tile, int col_lim, int c_begin, const GemmArgs& g) {
  uint32_t ra[32], rb[32];
  tmem_ld32_async(taddr + c_begin, ra);
  if (is_swiglu(EPI)) tmem_ld32_async(taddr + BN / 2 + c_begin, rb);
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = c_begin + 32 * ch;
    const int col0 = col_tile + c;
    const bool live = row < g.M && col0 < col_lim;
    const bool full = col0 + 32 <= col_lim;
    float4 res[8];
    const bool vec_res = EPI == EPI_RES && g.residual && live && full && (g.ldr & 3) == 0;
    if (vec_res) {
      const float* r = g.residual + static_cast<int64_t>(row) * g.ldr + col0;
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = __ldg(reinterpret_cast<const float4*>(r) + i);
    }
    float v[32];
    tmem_ld_wait(ra);
    if (is_swiglu(EPI)) {
      tmem_ld_wait(rb);
      swiglu_chunk<EPI == EPI_SWIGLU_CLAMP>(ra, rb, g.limit, v);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
    }
    if (is_swiglu(EPI) && g.gu_out != nullptr && live) {
      // training: keep the pre-activations for the backward (gate in columns [0, N), up in [N, 2N))
      __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(g.gu_out) + static_cast<int64_t>(row) * g.ldgu + col0;
      __nv_bfloat16* ou = og + g.N;
      if (full && (g.ldgu & 15) == 0 && (g.N & 15) == 0 && (reinterpret_cast<uintptr_t>(g.gu_out) & 31) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 16) {
          uint32_t pg[8], pu[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            pg[q] = float2_to_bf16x2(__uint_as_float(ra[i + 2 * q]), __uint_as_float(ra[i + 2 * q + 1]));
            pu[q] = float2_to_bf16x2(__uint_as_float(rb[i + 2 * q]), __uint_as_float(rb[i + 2 * q + 1]));
          }
          st256(og + i, pg);
          st256(ou + i, pu);
        }
      } else if (full && (g.ldgu & 7) == 0 && (g.N & 7) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 pg, pu;
          pg.x = float2_to_bf16x2(__uint_as_float(ra[i]), __uint_as_float(ra[i + 1]));
          pg.y = float2_to_bf16x2(__uint_as_float(ra[i + 2]), __uint_as_float(ra[i + 3]));
          pg.z = float2_to_bf16x2(__uint_as_float(ra[i + 4]), __uint_as_float(ra[i + 5]));
          pg.w = float2_to_bf16x2(__uint_as_float(ra[i + 6]), __uint_as_float(ra[i + 7]));
          pu.x = float2_to_bf16x2(__uint_as_float(rb[i]), __uint_as_float(rb[i + 1]));
          pu.y = float2_to_bf16x2(__uint_as_float(rb[i + 2]), __uint_as_float(rb[i + 3]));
          pu.z = float2_to_bf16x2(__uint_as_float(rb[i + 4]), __uint_as_float(rb[i + 5]));
          pu.w = float2_to_bf16x2(__uint_as_float(rb[i + 6]), __uint_as_float(rb[i + 7]));
          *reinterpret_cast<uint4*>(og + i) = pg;
          *reinterpret_cast<uint4*>(ou + i) = pu;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {  // static indices: the accumulator registers must not move to local memory
          if (col0 + i < col_lim) {
            og[i] = __float2bfloat16_rn(__uint_as_float(ra[i]));
            ou[i] = __float2bfloat16_rn(__uint_as_float(rb[i]));
          }
        }
      }
    }
    if (ch + 1 < NCH) {
      tmem_ld32_async(taddr + c + 32, ra);
      if (is_swiglu(EPI)) tmem_ld32_async(taddr + BN / 2 + c + 32, rb);
    }
    if (!live) continue;
    if (EPI == EPI_F32) {
      float* o = reinterpret_cast<float*>(g.out) + static_cast<int64_t>(row) * g.ldo + col0;
      if (full && (g.ldo & 7) == 0 && (col0 & 7) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 31) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint32_t p[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) p[q] = __float_as_uint(v[i + q]);
          st256(o + i, p);
        }
      } else if (full && (g.ldo & 3) == 0 && (col0 & 3) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
        for (int i = 0; i < 32 && col0 + i < col_lim; ++i) o[i] = v[i];
      }
    } else {
      if (EPI == EPI_RES && g.residual) {
        if (vec_res) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            v[4 * i] += res[i].x, v[4 * i + 1] += res[i].y, v[4 * i + 2] += res[i].z, v[4 * i + 3] += res[i].w;
        } else {
          const float* r = g.residual + static_cast<int64_t>(row) * g.ldr + col0;
          for (int i = 0; i < 32 && col0 + i < col_lim; ++i) v[i] += r[i];
        }
      }
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + static_cast<int64_t>(row) * g.ldo + col0;
      if (full && (g.ldo & 15) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 31) == 0) {
        // 32 consecutive bf16 of this row = 64 bytes: two 256-bit stores, each a whole 32-byte sector
#pragma unroll
        for (int i = 0; i < 32; i += 16) {
          uint32_t p[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) p[q] = float2_to_bf16x2(v[i + 2 * q], v[i + 2 * q + 1]);
          st256(o + i, p);
        }
      } else if (full && (g.ldo & 7) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 p;
          p.x = float2_to_bf16x2(v[i], v[i + 1]);
          p.y = float2_to_bf16x2(v[i + 2], v[i + 3]);
          p.z = float2_to_bf16x2(v[i + 4], v[i + 5]);
          p.w = float2_to_bf16x2(v[i + 6], v[i + 7]);
          *reinterpret_cast<uint4*>(o + i) = p;
        }
      } else {
        for (int i = 0; i < 32 && col0 + i < col_lim; ++i) o[i] = __float2bfloat16_rn(v[i]);
      }
    }
  }
}

// The same drain with the output leaving through shared memory: every pair of 32-column chunks (64 bf16
// = 128 bytes per row) is written into the warp's 32-row staging buffer in the 128-byte swizzle the
// tensor map expects (16-byte piece j of row r sits at piece j ^ (r % 8): no bank conflicts although a
// lane owns a row), and one lane hands the 32 x 64 box to the TMA engine.  The global writes are then
// whole 128-byte lines issued by the copy engine instead of 32 scattered sectors per warp instruction,
// rows and columns outside the matrix are clipped by the tensor map, and the warp goes on draining
// while the box is on its way.  row0: global row of lane 0; stg: shared-memory address of the warp's
// 4 KB staging buffer (1024-byte aligned).  bf16 outputs only (EPI_SWIGLU, EPI_RES); NCH even.
template <int BN, int EPI, int NCH>
__device__ __forceinline__ void store_tile_tma(uint32_t taddr, int row0, int col_tile, int col_lim, int c_begin, const GemmArgs& g,
                                               const CUtensorMap* tm_out, uint32_t stg) {
  static_assert(NCH % 2 == 0 && EPI != EPI_F32, "bf16 slabs of two chunks");
  const int lane = lane_id();
  const int row = row0 + lane;
  uint32_t ra[32], rb[32];
  tmem_ld32_async(taddr + c_begin, ra);
  if (is_swiglu(EPI)) tmem_ld32_async(taddr + BN / 2 + c_begin, rb);
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = c_begin + 32 * ch;
    const int col0 = col_tile + c;
    const bool live = row < g.M && col0 < col_lim;
    const bool full = col0 + 32 <= col_lim;
    float v[32];
    tmem_ld_wait(ra);
    if (is_swiglu(EPI)) {
      tmem_ld_wait(rb);
      swiglu_chunk<EPI == EPI_SWIGLU_CLAMP>(ra, rb, g.limit, v);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
    }
    if (is_swiglu(EPI) && g.gu_out != nullptr && live) {
      __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(g.gu_out) + static_cast<int64_t>(row) * g.ldgu + col0;
      __nv_bfloat16* ou = og + g.N;
      if (full && (g.ldgu & 15) == 0 && (g.N & 15) == 0 && (reinterpret_cast<uintptr_t>(g.gu_out) & 31) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 16) {
          uint32_t pg[8], pu[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            pg[q] = float2_to_bf16x2(__uint_as_float(ra[i + 2 * q]), __uint_as_float(ra[i + 2 * q + 1]));
            pu[q] = float2_to_bf16x2(__uint_as_float(rb[i + 2 * q]), __uint_as_float(rb[i + 2 * q + 1]));
          }
          st256(og + i, pg);
          st256(ou + i, pu);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (col0 + i < col_lim) {
            og[i] = __float2bfloat16_rn(__uint_as_float(ra[i]));
            ou[i] = __float2bfloat16_rn(__uint_as_float(rb[i]));
          }
        }
      }
    }
    if (ch + 1 < NCH) {
      tmem_ld32_async(taddr + c + 32, ra);
      if (is_swiglu(EPI)) tmem_ld32_async(taddr + BN / 2 + c + 32, rb);
    }
    if (EPI == EPI_RES && g.residual && live) {
      if (full && (g.ldr & 3) == 0) {
        const float4* r4 = reinterpret_cast<const float4*>(g.residual + static_cast<int64_t>(row) * g.ldr + col0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 t4 = __ldg(r4 + i);
          v[4 * i] += t4.x, v[4 * i + 1] += t4.y, v[4 * i + 2] += t4.z, v[4 * i + 3] += t4.w;
        }
      } else {
        const float* r = g.residual + static_cast<int64_t>(row) * g.ldr + col0;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i < col_lim) v[i] += r[i];
      }
    }
    if ((ch & 1) == 0) {
      // a new slab: the box sent from this buffer before must have been read out
      if (lane == 0) bulk_wait_read_all();
      __syncwarp();
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int piece = ((ch & 1) * 4 + q) ^ (lane & 7);
      st_shared_v4(stg + lane * 128 + piece * 16, float2_to_bf16x2(v[8 * q], v[8 * q + 1]), float2_to_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                   float2_to_bf16x2(v[8 * q + 4], v[8 * q + 5]), float2_to_bf16x2(v[8 * q + 6], v[8 * q + 7]));
    }
    if ((ch & 1) == 1) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(tm_out, stg, col0 - 32, row0);
        bulk_commit_group();
      }
    }
  }
}

// fp32 variant for the router logits: a chunk of 32 columns is 128 bytes per row, one box per chunk through
// the same staging buffer.  NCH chunks starting at TMEM column offset 0 of `taddr`; output columns
// col_tile + 32 * ch.  The tensor map clips rows; the caller guarantees the columns are inside the axis.
template <int NCH>
__device__ __forceinline__ void store_logits_tma(uint32_t taddr, int row0, int col_tile, const CUtensorMap* tm_lg, uint32_t stg) {
  const int lane = lane_id();
  uint32_t ra[32];
  tmem_ld32_async(taddr, ra);
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    uint32_t v[32];
    tmem_ld_wait(ra);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = ra[i];
    if (ch + 1 < NCH) tmem_ld32_async(taddr + 32 * (ch + 1), ra);
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int piece = q ^ (lane & 7);
      st_shared_v4(stg + lane * 128 + piece * 16, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tm_lg, stg, col_tile + 32 * ch, row0);
      bulk_commit_group();
    }
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                           const __grid_constant__ CUtensorMap tm_b0,
                                                           const __grid_constant__ CUtensorMap tm_b1,
                                                           const GemmArgs g) {
  using C = Cfg<BN>;
  if (g.enable != nullptr && *g.enable == 0) return;  // every thread of every CTA, before anything is allocated
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t sA = base;
  const uint32_t sB = base + C::kStages * C::kStageA;
  uint8_t* bar_ptr = base_ptr + C::kStages * C::kStage;
  const uint32_t bars = base + C::kStages * C::kStage;
  // barrier map (8 bytes each): full[s], empty[s], tmem_full[2], tmem_empty[2]; then tmem base, abort flag
  const uint32_t bar_full = bars;
  const uint32_t bar_empty = bars + 8 * C::kStages;
  const uint32_t bar_tfull = bars + 16 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ptr + 16 * C::kStages + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 16 * C::kStages + 40);

  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int num_tiles = g.tiles_m * g.tiles_n;
  const int kblocks = ceil_div(g.K, BK);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b0);
    prefetch_tmap(&tm_b1);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      long long p_wait = 0;
      bool dead = false;
      const long long p_t0 = clock64();
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, g.tiles_m, g.tiles_n, tm, tn);
        const int axis = tn / g.tiles_n_axis, tj = tn - axis * g.tiles_n_axis;
        for (int kb = 0; kb < kblocks; ++kb) {
          bool ok;
          OMNI_TIMED(p_wait, ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, g.status));
          if (!ok) { dead = true; break; }
          const uint32_t full = bar_full + 8 * stage;
          mbar_arrive_expect_tx(full, C::kStage);
          tma_load_2d(sA + stage * C::kStageA, &tm_a, kb * BK, tm * BM, full);
          const uint32_t dstB = sB + stage * C::kStageB;
          if (is_swiglu(EPI)) {
            tma_load_2d(dstB, &tm_b0, kb * BK, tj * (BN / 2), full);
            tma_load_2d(dstB + (BN / 2) * BK * 2, &tm_b1, kb * BK, tj * (BN / 2), full);
          } else {
            tma_load_2d(dstB, axis == 0 ? &tm_b0 : &tm_b1, kb * BK, tj * BN, full);
          }
          if (++stage == C::kStages) stage = 0, phase ^= 1;
        }
        if (dead) break;
      }
      if (G_PROF) G_PROF[blockIdx.x * 16 + 3] = p_wait, G_PROF[blockIdx.x * 16 + 4] = clock64() - p_t0;
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      long long m_full = 0, m_tempty = 0;
      bool dead = false;
      const uint64_t adesc0 = make_smem_desc(sA), bdesc0 = make_smem_desc(sB);
      const long long m_t0 = clock64();
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        OMNI_TIMED(m_tempty, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, g.status));
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          bool ok;
          OMNI_TIMED(m_full, ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status));
          if (!ok) { dead = true; break; }
          tc_fence_after();
          // descriptors of consecutive stages differ only in the start-address field (16-byte units)
          const uint64_t adesc = adesc0 + static_cast<uint64_t>(stage * (C::kStageA >> 4));
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(stage * (C::kStageB >> 4));
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            // advancing K by 16 bf16 = 32 bytes = 2 units of the start-address field
            umma_bf16(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, (kb | ks) != 0);
          }
          umma_commit(bar_empty + 8 * stage);  // frees the stage when these MMAs have read it
          if (++stage == C::kStages) stage = 0, phase ^= 1;
        }
        if (dead) break;
        umma_commit(bar_tfull + 8 * acc);  // accumulator complete
      }
      if (G_PROF) G_PROF[blockIdx.x * 16 + 0] = m_full, G_PROF[blockIdx.x * 16 + 1] = m_tempty, G_PROF[blockIdx.x * 16 + 2] = clock64() - m_t0;
    }
  } else {
    // ------------------------------- epilogue -----------------------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, +32) are the ones this warp may read
    const int col_half = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    int it = 0;
    long long e_wait = 0, e_store = 0;
    const long long e_t0 = clock64();
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      int tm, tn;
      tile_coords(tile, g.tiles_m, g.tiles_n, tm, tn);
      const int axis = tn / g.tiles_n_axis, tj = tn - axis * g.tiles_n_axis;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      bool ok;
      OMNI_TIMED(e_wait, ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, g.status));
      tc_fence_after();
      if (!ok) break;
      const int row = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      constexpr int OUTC = (is_swiglu(EPI)) ? BN / 2 : BN;  // output columns of this tile
      const int col_tile = (EPI == EPI_F32 && g.dual) ? axis * g.N + tj * OUTC : tj * OUTC;
      const int col_lim = (EPI == EPI_F32 && g.dual) ? (axis + 1) * g.N : g.N;  // exclusive bound of valid columns
      OMNI_TIMED(e_store, (store_tile<BN, EPI, OUTC / 64>(taddr, row, col_tile, col_lim, col_half * (OUTC / 2), g)));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
    if (G_PROF && warp == 2 && lane == 0)
      G_PROF[blockIdx.x * 16 + 5] = e_wait, G_PROF[blockIdx.x * 16 + 6] = e_store, G_PROF[blockIdx.x * 16 + 7] = clock64() - e_t0;
  }

  // ------------------------------- teardown -------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // copies issued before the abort may still be landing in this CTA's shared memory: give them
    // time before the memory is handed to another CTA
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernel: two CTAs of a cluster (two SMs) work on one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA fetches its own 128 rows of A and its own half of the B tile
// (128 of the 256 rows; for EPI_SWIGLU rank 0 holds the Wg rows and rank 1 the Wu rows), so a CTA
// moves 32 KB per 64-wide K block instead of 48 KB and six stages fit in shared memory.
// The accumulator of a CTA (its 128 rows x 256 columns) sits in its own TMEM.
//   rank 0 (leader)  its MMA lane issues every MMA of the pair; the "full" barrier of a stage lives
//                    here and counts the bytes of both CTAs' loads
//   both ranks       producer lane loads the local tiles; epilogue warps drain the local accumulator
// Stage-free and accumulator-ready signals reach both CTAs through the multicast form of
// tcgen05.commit; accumulator-drained signals go to the leader with a remote mbarrier arrive.
// ---------------------------------------------------------------------------------------------
struct PairCfg {
  static constexpr int BN = 256;
  // A stage holds kSub consecutive 64-wide K slices of both operands, so one barrier round trip
  // (wait, commit) feeds 4 * kSub MMAs: the single issuing thread spends its time issuing.
  static constexpr int kSub = 2;
  static constexpr int kSliceA = BM * BK * 2;        // 16 KB: this CTA's 128 rows of A, one K slice
  static constexpr int kSliceB = (BN / 2) * BK * 2;  // 16 KB: this CTA's half of B, one K slice
  static constexpr int kStageA = kSub * kSliceA;
  static constexpr int kStageB = kSub * kSliceB;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = 6 / kSub;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kStaging = kEpiWarps * 4096;  // per epilogue warp: 32 rows x 128 bytes for the TMA stores
  static constexpr int kSmem = kStages * kStage + 1024 + kStaging + 1024;
};

// MAJOR: bit 0 = the B operand is given transposed ([K, N], N contiguous), bit 1 = the A operand is
// ([K, M], M contiguous).  Such an operand is loaded as boxes of 64 K rows x 64 M/N elements and fed to
// the tensor cores as an MN-major tile, so the gradient GEMMs of the backward (dy Wd, dy^T act, ...)
// read their operands where they lie instead of transposed copies.  Per slice the two 64-element
// groups of this CTA's 128 rows / columns lie 8 KB apart.
template <int EPI, bool ROUTER, int MAJOR = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
                     const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_r0,
                     const __grid_constant__ CUtensorMap tm_r1, const __grid_constant__ CUtensorMap tm_out,
                     const __grid_constant__ CUtensorMap tm_lg, const GemmArgs g) {
  // ROUTER: the first g.router_tiles tile columns multiply x by the router sub-keys instead of the MLP
  // weights: rank 0 holds 128 rows of the x-axis keys, rank 1 the same rows of the y-axis keys, and the
  // epilogue stores fp32 logits.  It rides along with the gate/up GEMM because it reads the same A.
  using C = PairCfg;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t sA = base;
  const uint32_t sB = base + C::kStages * C::kStageA;
  uint8_t* bar_ptr = base_ptr + C::kStages * C::kStage;
  const uint32_t bars = base + C::kStages * C::kStage;
  const uint32_t bar_full = bars;
  const uint32_t bar_empty = bars + 8 * C::kStages;
  const uint32_t bar_tfull = bars + 16 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ptr + 16 * C::kStages + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 16 * C::kStages + 40);

  const int warp = threadIdx.x >> 5, lane = lane_id();
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int rt = ROUTER ? g.router_tiles : 0;
  const int num_tiles = g.tiles_m * (g.tiles_n + rt);  // tiles_m counts 256-row pair tiles here
  const int kblocks = ceil_div(g.K, BK * C::kSub);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * kEpiWarps);  // epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b0);
    prefetch_tmap(&tm_b1);
    if (g.tma_out) prefetch_tmap(&tm_out);
    if (g.tma_logits) prefetch_tmap(&tm_lg);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // the next kernel on the stream may set itself up while this one computes
  pdl_wait();               // the kernel before this one has completed: its outputs may be read now

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      long long p_wait = 0;
      bool dead = false;
      const long long p_t0 = clock64();
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t full_leader0 = mapa_shared(bar_full, 0);
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        int tm, tn_all;
        tile_coords(tile, g.tiles_m, g.tiles_n + rt, tm, tn_all);
        const bool router_tile = ROUTER && tn_all < rt;
        const int tn = router_tile ? tn_all : tn_all - rt;
        const int row_a = tm * (2 * BM) + static_cast<int>(rank) * BM;
        const CUtensorMap* mb = router_tile ? (rank == 1 ? &tm_r1 : &tm_r0)
                                            : ((is_swiglu(EPI) && rank == 1) ? &tm_b1 : &tm_b0);
        const int row_b = (is_swiglu(EPI) || router_tile) ? tn * (BN / 2) : tn * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < kblocks; ++kb) {
          bool ok;
          OMNI_TIMED(p_wait, ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, g.status));
          if (!ok) { dead = true; break; }
          if (G_KNOBS & 1) {
            if (leader) mbar_arrive(bar_full + 8 * stage);
          } else {
            if (leader) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * C::kStage);
            const uint32_t full_leader = full_leader0 + 8 * stage;
#pragma unroll
            for (int sub = 0; sub < C::kSub; ++sub) {
              const int kcol = (kb * C::kSub + sub) * BK;  // past K the box is zero-filled
              const uint32_t dst_a = sA + stage * C::kStageA + sub * C::kSliceA;
              const uint32_t dst_b = sB + stage * C::kStageB + sub * C::kSliceB;
              if (MAJOR & 2) {
                tma_load_2d_pair(dst_a, &tm_a, row_a, kcol, full_leader);
                tma_load_2d_pair(dst_a + C::kSliceA / 2, &tm_a, row_a + 64, kcol, full_leader);
              } else {
                tma_load_2d_pair(dst_a, &tm_a, kcol, row_a, full_leader);
              }
              if (MAJOR & 1) {
                // a transposed B may be two matrices stacked along K ((Wg ; Wu) of the MLP backward): rows
                // [0, k_split) come from the first map, the rest from the second (k_split is a multiple of 64)
                const bool second = !ROUTER && g.router_n > 0 && kcol >= g.router_n;
                const CUtensorMap* mbk = second ? &tm_b1 : mb;
                const int kb_row = second ? kcol - g.router_n : kcol;
                tma_load_2d_pair(dst_b, mbk, row_b, kb_row, full_leader);
                tma_load_2d_pair(dst_b + C::kSliceB / 2, mbk, row_b + 64, kb_row, full_leader);
              } else {
                tma_load_2d_pair(dst_b, mb, kcol, row_b, full_leader);
              }
            }
          }
          if (++stage == C::kStages) stage = 0, phase ^= 1;
        }
        if (dead) break;
      }
      if (G_PROF) G_PROF[blockIdx.x * 16 + 3] = p_wait, G_PROF[blockIdx.x * 16 + 4] = clock64() - p_t0;
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) ---------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN, (MAJOR >> 1) & 1, MAJOR & 1);
      // start-address step of one 16-wide K step, in 16-byte units: 32 bytes along a K-major row, 16 rows of an MN-major tile
      constexpr uint64_t kStepA = (MAJOR & 2) ? (16 * 128) >> 4 : 2, kStepB = (MAJOR & 1) ? (16 * 128) >> 4 : 2;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      long long m_full = 0, m_tempty = 0;
      bool dead = false;
      const uint64_t adesc0 = (MAJOR & 2) ? make_smem_desc_mn(sA, C::kSliceA / 2) : make_smem_desc(sA);
      const uint64_t bdesc0 = (MAJOR & 1) ? make_smem_desc_mn(sB, C::kSliceB / 2) : make_smem_desc(sB);
      const long long m_t0 = clock64();
      for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        OMNI_TIMED(m_tempty, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, g.status));
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          bool ok;
          OMNI_TIMED(m_full, ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status));
          if (!ok) { dead = true; break; }
          tc_fence_after();
          // descriptors of consecutive stages differ only in the start-address field (16-byte units)
          const uint64_t adesc = adesc0 + static_cast<uint64_t>(stage * (C::kStageA >> 4));
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(stage * (C::kStageB >> 4));
          if (!(G_KNOBS & 2)) {
#pragma unroll
            for (int sub = 0; sub < C::kSub; ++sub) {
              const uint64_t ad = adesc + static_cast<uint64_t>(sub * (C::kSliceA >> 4));
              const uint64_t bd = bdesc + static_cast<uint64_t>(sub * (C::kSliceB >> 4));
#pragma unroll
              for (int ks = 0; ks < BK / UMMA_K; ++ks)
                umma_bf16_pair(d_tmem, ad + kStepA * ks, bd + kStepB * ks, idesc, (kb | sub | ks) != 0);
            }
          }
          umma_commit_pair(bar_empty + 8 * stage, 3);  // both CTAs may refill this stage
          if (++stage == C::kStages) stage = 0, phase ^= 1;
        }
        if (dead) break;
        umma_commit_pair(bar_tfull + 8 * acc, 3);  // both CTAs may drain their accumulator
      }
      if (G_PROF) G_PROF[blockIdx.x * 16 + 0] = m_full, G_PROF[blockIdx.x * 16 + 1] = m_tempty, G_PROF[blockIdx.x * 16 + 2] = clock64() - m_t0;
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -----------------------------------
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    int it = 0;
    long long e_wait = 0, e_store = 0;
    const long long e_t0 = clock64();
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      int tm, tn_all;
      tile_coords(tile, g.tiles_m, g.tiles_n + rt, tm, tn_all);
      const bool router_tile = ROUTER && tn_all < rt;
      const int tn = router_tile ? tn_all : tn_all - rt;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      bool ok;
      OMNI_TIMED(e_wait, ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, g.status));
      tc_fence_after();
      if (!ok) break;
      const int row = tm * (2 * BM) + static_cast<int>(rank) * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      constexpr int OUTC = (is_swiglu(EPI)) ? BN / 2 : BN;
      if (router_tile) {
        // accumulator columns [0, 128) are x-axis sub-keys tn*128.., [128, 256) the y-axis ones;
        // the warps of column half h store axis h
        GemmArgs gr = g;
        gr.out = g.logits, gr.ldo = 2 * g.router_n;
        const int col_tile = col_half * g.router_n + tn * (BN / 2);
        if (g.tma_logits)
          store_logits_tma<4>(taddr + col_half * (BN / 2), row - lane, col_tile, &tm_lg,
                              bars + 1024 + static_cast<uint32_t>(warp - 2) * 4096);
        else
          store_tile<BN, EPI_F32, 4>(taddr + col_half * (BN / 2), row, col_tile, (col_half + 1) * g.router_n, 0, gr);
      } else if (g.tma_out) {
        const uint32_t stg = bars + 1024 + static_cast<uint32_t>(warp - 2) * 4096;
        OMNI_TIMED(e_store, (store_tile_tma<BN, EPI, OUTC / 64>(taddr, row - lane, tn * OUTC, g.N, col_half * (OUTC / 2), g, &tm_out, stg)));
      } else {
        OMNI_TIMED(e_store, (store_tile<BN, EPI, OUTC / 64>(taddr, row, tn * OUTC, g.N, col_half * (OUTC / 2), g)));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));
    }
    if ((g.tma_out || g.tma_logits) && lane == 0) bulk_wait_all();  // the boxes still on their way are written before the CTA leaves
    if (G_PROF && warp == 2 && lane == 0)
      G_PROF[blockIdx.x * 16 + 5] = e_wait, G_PROF[blockIdx.x * 16 + 6] = e_store, G_PROF[blockIdx.x * 16 + 7] = clock64() - e_t0;
  }

  // ------------------------------- teardown -------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or read its tiles
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread.  A thread that
// has made no runtime call on this device yet (the autograd engine's backward thread, when a GEMM is the
// first thing it runs) has none: a runtime query of one of this file's kernels binds the device's primary
// context, after which the encode is retried once.
void bind_primary_context();

template <typename... Args>
CUresult encode_tiled(EncodeFn enc, Args... args) {
  CUresult r = enc(args...);
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    bind_primary_context();
    r = enc(args...);
  }
  return r;
}

// Map of a row-major bf16 matrix [rows, cols] with boxes of box_rows x 64 columns, 128-byte swizzle.
int make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols, int box_rows, int64_t ld = 0) {
  EncodeFn enc = get_encode();
  if (!enc) return fail(-2, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld > 0 ? ld : cols) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_tiled(enc, m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-2, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return 0;
}

// Map of a row-major bf16 output [rows, cols] with row stride ld, boxes of 32 rows x 64 columns in
// the 128-byte swizzle: what store_tile_tma sends.
int make_out_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols, int64_t ld) {
  EncodeFn enc = get_encode();
  if (!enc) return fail(-2, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_tiled(enc, m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-2, "cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(r));
  return 0;
}

// Map of the fp32 router logits [rows, cols] (row stride = cols): boxes of 32 rows x 32 columns = 128-byte rows.
int make_logits_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols) {
  EncodeFn enc = get_encode();
  if (!enc) return fail(-2, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_tiled(enc, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-2, "cuTensorMapEncodeTiled (logits) failed with CUresult %d", static_cast<int>(r));
  return 0;
}

// The bf16 outputs of the pair kernels go through TMA stores when the output qualifies (16-byte aligned
// base and row stride).  OMNI_MOE_B200_TMA_STORE=0 keeps the direct stores; the variable is read at every call.
bool tma_store_enabled() {
  const char* e = getenv("OMNI_MOE_B200_TMA_STORE");
  return !(e && e[0] == '0');
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = v > 0 ? v : 148;
  }
  return cached[dev];
}

template <int BN, int EPI>
int launch(const CUtensorMap& a, const CUtensorMap& b0, const CUtensorMap& b1, const GemmArgs& g, cudaStream_t st) {
  using C = Cfg<BN>;
  static OncePerDevice once;
  if (once.first() &&
      cudaFuncSetAttribute(gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
    return fail(-2, "cannot raise the shared-memory limit to %d bytes", C::kSmem);
  const int tiles = g.tiles_m * g.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_kernel<BN, EPI><<<grid, kThreads, C::kSmem, st>>>(a, b0, b1, g);
  return check_launch("gemm_kernel");
}

template <int EPI, bool ROUTER, int MAJOR = 0>
int launch_pair(const CUtensorMap& a, const CUtensorMap& b0, const CUtensorMap& b1, const CUtensorMap& r0,
                const CUtensorMap& r1, GemmArgs g, cudaStream_t st) {
  // output map: only when the bf16 output qualifies for TMA stores; otherwise any valid map fills the slot
  CUtensorMap mo = a;
  g.tma_out = 0;
  if (g.out != nullptr && g.N > 0 && tma_store_enabled() && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && (g.ldo & 7) == 0) {
    if (int e = make_out_map(&mo, g.out, g.M, g.N, g.ldo)) return e;
    g.tma_out = 1;
  }
  // router logits: whole 128-column tiles per axis only (a narrower axis would spill into its neighbour's columns)
  CUtensorMap ml = a;
  g.tma_logits = 0;
  if (ROUTER && g.logits != nullptr && g.router_tiles > 0 && g.router_n % 128 == 0 && tma_store_enabled() &&
      (reinterpret_cast<uintptr_t>(g.logits) & 15) == 0) {
    if (int e = make_logits_map(&ml, g.logits, g.M, 2 * static_cast<int64_t>(g.router_n))) return e;
    g.tma_logits = 1;
  }
  using C = PairCfg;
  static OncePerDevice once;
  if (once.first() &&
      cudaFuncSetAttribute(gemm_pair_kernel<EPI, ROUTER, MAJOR>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
    return fail(-2, "cannot raise the shared-memory limit to %d bytes", C::kSmem);
  const int tiles = g.tiles_m * (g.tiles_n + (ROUTER ? g.router_tiles : 0));
  const int max_pairs = sm_count() / 2;
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (G_GRID_LIMIT > 0 && G_GRID_LIMIT < pairs) pairs = G_GRID_LIMIT;
  launch_after_predecessor(gemm_pair_kernel<EPI, ROUTER, MAJOR>, dim3(2 * pairs), dim3(kThreads), C::kSmem, st, a, b0, b1, r0, r1, mo, ml, g);
  return check_launch("gemm_pair_kernel");
}

void bind_primary_context() {
  cudaFuncAttributes attr;
  (void)cudaFuncGetAttributes(&attr, gemm_kernel<64, EPI_F32>);
  (void)cudaGetLastError();
}

// OMNI_MOE_B200_GEMM=1cta selects the single-CTA kernels for the MLP GEMMs (default: CTA pairs).
bool use_pairs() {
  static const bool v = [] {
    const char* e = getenv("OMNI_MOE_B200_GEMM");
    return !(e && e[0] == '1');
  }();
  return v;
}

#ifdef OMNI_TUNING
long long* g_prof = nullptr;  // set by omni_debug_gemm_profile
int g_knobs = 0, g_grid_limit = 0;
#define OMNI_SET_TUNING(g) ((g).prof = g_prof, (g).knobs = g_knobs, (g).grid_limit = g_grid_limit)
#else
#define OMNI_SET_TUNING(g) ((void)0)
#endif

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" int omni_router_gate(const void* x, const void* gate_x, const void* gate_y, int64_t num_tokens, int hidden,
                                int sqrt_n, float* logits, int32_t* status, void* stream) {
  return omni::router_gate_if(x, gate_x, gate_y, num_tokens, hidden, sqrt_n, logits, nullptr, status, stream);
}

int omni::router_gate_if(const void* x, const void* gate_x, const void* gate_y, int64_t num_tokens, int hidden, int sqrt_n,
                         float* logits, const int* enable, int32_t* status, void* stream) {
  OMNI_REQUIRE(enable == nullptr || sqrt_n < 128, "a conditional launch covers sqrt_n < 128 only");
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(sqrt_n >= 1, "sqrt_n must be >= 1");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && gate_x && gate_y && logits && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(gate_x) && aligned16(gate_y) && aligned16(logits), "pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_pairs() && sqrt_n >= 128 && num_tokens >= 2 * BM * 16) {
    // Wide router grids on many tokens: the CTA-pair kernel with router tiles only (rank 0 holds 128
    // x-axis keys, rank 1 the same 128 y-axis keys of a tile column) runs at GEMM efficiency.
    CUtensorMap ma, mx, my;
    if (int e = make_map(&ma, x, num_tokens, hidden, BM)) return e;
    if (int e = make_map(&mx, gate_x, sqrt_n, hidden, 128)) return e;
    if (int e = make_map(&my, gate_y, sqrt_n, hidden, 128)) return e;
    GemmArgs g{};
    g.M = static_cast<int>(num_tokens), g.N = 0, g.K = hidden, g.dual = 0;
    g.tiles_m = ceil_div(g.M, 2 * BM);
    g.tiles_n = g.tiles_n_axis = 0;
    g.router_tiles = ceil_div(sqrt_n, 128), g.router_n = sqrt_n, g.logits = logits;
    g.out = nullptr, g.ldo = 0, g.status = status;
  OMNI_SET_TUNING(g);
    return launch_pair<EPI_SWIGLU, true>(ma, mx, my, mx, my, g, st);
  }
  const int bn = sqrt_n <= 64 ? 64 : (sqrt_n <= 128 ? 128 : 256);
  CUtensorMap ma, mx, my;
  if (int e = make_map(&ma, x, num_tokens, hidden, BM)) return e;
  if (int e = make_map(&mx, gate_x, sqrt_n, hidden, bn)) return e;
  if (int e = make_map(&my, gate_y, sqrt_n, hidden, bn)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(num_tokens), g.N = sqrt_n, g.K = hidden, g.dual = 1;
  g.tiles_m = ceil_div(g.M, BM);
  g.tiles_n_axis = ceil_div(sqrt_n, bn);
  g.tiles_n = 2 * g.tiles_n_axis;
  g.out = logits, g.ldo = 2 * static_cast<int64_t>(sqrt_n), g.status = status, g.enable = enable;
  OMNI_SET_TUNING(g);
  if (bn == 64) return launch<64, EPI_F32>(ma, mx, my, g, st);
  if (bn == 128) return launch<128, EPI_F32>(ma, mx, my, g, st);
  return launch<256, EPI_F32>(ma, mx, my, g, st);
}

extern "C" int omni_mlp_gate_up(const void* x, const void* gate_w, const void* up_w, int64_t num_tokens, int hidden,
                                int intermediate, void* act, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8, got %d", intermediate);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && gate_w && up_w && act && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(gate_w) && aligned16(up_w) && aligned16(act), "pointers must be 16-byte aligned");
  CUtensorMap ma, mg, mu;
  if (int e = make_map(&ma, x, num_tokens, hidden, BM)) return e;
  if (int e = make_map(&mg, gate_w, intermediate, hidden, 128)) return e;
  if (int e = make_map(&mu, up_w, intermediate, hidden, 128)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(num_tokens), g.N = intermediate, g.K = hidden, g.dual = 0;
  g.tiles_m = ceil_div(g.M, BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(intermediate, 128);
  g.out = act, g.ldo = intermediate, g.status = status;
  OMNI_SET_TUNING(g);
  if (use_pairs()) {
    g.tiles_m = ceil_div(g.M, 2 * BM);
    return launch_pair<EPI_SWIGLU, false>(ma, mg, mu, mg, mu, g, static_cast<cudaStream_t>(stream));
  }
  return launch<256, EPI_SWIGLU>(ma, mg, mu, g, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_mlp_gate_up_limit(const void* x, const void* gate_w, const void* up_w, int64_t num_tokens, int hidden,
                                      int intermediate, float limit, void* act, void* gate_up, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - 2 * BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8, got %d", intermediate);
  OMNI_REQUIRE(limit >= 0.f, "limit must be >= 0 (0 = no clamp), got %g", static_cast<double>(limit));  // also refuses NaN
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && gate_w && up_w && act && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(gate_w) && aligned16(up_w) && aligned16(act) && aligned16(gate_up), "pointers must be 16-byte aligned");
  CUtensorMap ma, mg, mu;
  if (int e = make_map(&ma, x, num_tokens, hidden, BM)) return e;
  if (int e = make_map(&mg, gate_w, intermediate, hidden, 128)) return e;
  if (int e = make_map(&mu, up_w, intermediate, hidden, 128)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(num_tokens), g.N = intermediate, g.K = hidden, g.dual = 0;
  g.tiles_m = ceil_div(g.M, 2 * BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(intermediate, 128);
  g.out = act, g.ldo = intermediate, g.gu_out = gate_up, g.ldgu = 2 * static_cast<int64_t>(intermediate);
  g.limit = limit;
  g.status = status;
  OMNI_SET_TUNING(g);
  if (limit > 0.f) return launch_pair<EPI_SWIGLU_CLAMP, false>(ma, mg, mu, mg, mu, g, static_cast<cudaStream_t>(stream));
  return launch_pair<EPI_SWIGLU, false>(ma, mg, mu, mg, mu, g, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_mlp_gate_up_save(const void* x, const void* gate_w, const void* up_w, int64_t num_tokens, int hidden,
                                     int intermediate, void* act, void* gate_up, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens == 0 || gate_up, "NULL argument");
  return omni_mlp_gate_up_limit(x, gate_w, up_w, num_tokens, hidden, intermediate, 0.f, act, gate_up, status, stream);
}

extern "C" int omni_mlp_gate_up_router(const void* x, const void* gate_w, const void* up_w, const void* gate_x,
                                       const void* gate_y, int64_t num_tokens, int hidden, int intermediate,
                                       int sqrt_n, void* act, float* logits, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - 2 * BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8, got %d", intermediate);
  OMNI_REQUIRE(sqrt_n >= 1, "sqrt_n must be >= 1");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && gate_w && up_w && gate_x && gate_y && act && logits && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(gate_w) && aligned16(up_w) && aligned16(gate_x) && aligned16(gate_y) &&
               aligned16(act) && aligned16(logits), "pointers must be 16-byte aligned");
  CUtensorMap ma, mg, mu, mx, my;
  if (int e = make_map(&ma, x, num_tokens, hidden, BM)) return e;
  if (int e = make_map(&mg, gate_w, intermediate, hidden, 128)) return e;
  if (int e = make_map(&mu, up_w, intermediate, hidden, 128)) return e;
  if (int e = make_map(&mx, gate_x, sqrt_n, hidden, 128)) return e;
  if (int e = make_map(&my, gate_y, sqrt_n, hidden, 128)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(num_tokens), g.N = intermediate, g.K = hidden, g.dual = 0;
  g.tiles_m = ceil_div(g.M, 2 * BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(intermediate, 128);
  g.router_tiles = ceil_div(sqrt_n, 128), g.router_n = sqrt_n, g.logits = logits;
  g.out = act, g.ldo = intermediate, g.status = status;
  OMNI_SET_TUNING(g);
  return launch_pair<EPI_SWIGLU, true>(ma, mg, mu, mx, my, g, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_mlp_down(const void* act, const void* down_w, int64_t num_tokens, int hidden, int intermediate,
                             const float* residual, void* y, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8, got %d", intermediate);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(act && down_w && y && status, "NULL argument");
  OMNI_REQUIRE(aligned16(act) && aligned16(down_w) && aligned16(y) && aligned16(residual), "pointers must be 16-byte aligned");
  const int bn = 128;  // rows per B box: a whole tile of the single-CTA kernel, half a tile of the pair kernel
  CUtensorMap ma, mb;
  if (int e = make_map(&ma, act, num_tokens, intermediate, BM)) return e;
  if (int e = make_map(&mb, down_w, hidden, intermediate, bn)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(num_tokens), g.N = hidden, g.K = intermediate, g.dual = 0;
  g.tiles_m = ceil_div(g.M, BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(hidden, bn);
  g.out = y, g.ldo = hidden, g.residual = residual, g.ldr = hidden, g.status = status;
  OMNI_SET_TUNING(g);
  if (use_pairs()) {
    g.tiles_m = ceil_div(g.M, 2 * BM);
    g.tiles_n = g.tiles_n_axis = ceil_div(hidden, 256);
    return launch_pair<EPI_RES, false>(ma, mb, mb, mb, mb, g, static_cast<cudaStream_t>(stream));
  }
  return launch<128, EPI_RES>(ma, mb, mb, g, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_gemm_bf16_nt(const void* a, const void* b, int64_t m, int64_t n, int64_t k, void* out, int64_t ldo,
                                 int32_t* status, void* stream) {
  OMNI_REQUIRE(m >= 0 && m < (int64_t(1) << 31) - 2 * BM, "m out of range");
  OMNI_REQUIRE(n >= 0 && n < (int64_t(1) << 31) - 256, "n out of range");
  OMNI_REQUIRE(k >= 8 && k % 8 == 0 && k < (int64_t(1) << 31) - 256, "k must be a positive multiple of 8, got %lld", static_cast<long long>(k));
  OMNI_REQUIRE(ldo >= n, "ldo %lld < n", static_cast<long long>(ldo));
  if (m == 0 || n == 0) return 0;
  OMNI_REQUIRE(a && b && out && status, "NULL argument");
  OMNI_REQUIRE(aligned16(a) && aligned16(b) && aligned16(out), "pointers must be 16-byte aligned");
  CUtensorMap ma, mb;
  if (int e = make_map(&ma, a, m, k, BM)) return e;
  if (int e = make_map(&mb, b, n, k, 128)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(m), g.N = static_cast<int>(n), g.K = static_cast<int>(k), g.dual = 0;
  g.out = out, g.ldo = ldo, g.residual = nullptr, g.ldr = 0, g.status = status;
  OMNI_SET_TUNING(g);
  if (use_pairs()) {
    g.tiles_m = ceil_div(g.M, 2 * BM);
    g.tiles_n = g.tiles_n_axis = ceil_div(g.N, 256);
    return launch_pair<EPI_RES, false>(ma, mb, mb, mb, mb, g, static_cast<cudaStream_t>(stream));
  }
  g.tiles_m = ceil_div(g.M, BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(g.N, 128);
  return launch<128, EPI_RES>(ma, mb, mb, g, static_cast<cudaStream_t>(stream));
}

namespace {
int gemm_bf16_impl(const void* a, int a_transposed, int64_t lda, const void* b, const void* b1, int64_t k_split, int b_transposed,
                   int64_t ldb, int64_t m, int64_t n, int64_t k, void* out, int64_t ldo, int32_t* status, void* stream) {
  OMNI_REQUIRE(m >= 0 && m < (int64_t(1) << 31) - 2 * BM, "m out of range");
  OMNI_REQUIRE(n >= 0 && n < (int64_t(1) << 31) - 256, "n out of range");
  OMNI_REQUIRE(k >= 1 && k < (int64_t(1) << 31) - 256, "k out of range");
  OMNI_REQUIRE(ldo >= n, "ldo %lld < n", static_cast<long long>(ldo));
  // rows of either operand must be whole 16-byte pieces: the row stride, and the row length where it is the K extent
  OMNI_REQUIRE(lda >= (a_transposed ? m : k) && lda % 8 == 0, "lda must be a multiple of 8 and cover a row, got %lld", static_cast<long long>(lda));
  OMNI_REQUIRE(ldb >= (b_transposed ? n : k) && ldb % 8 == 0, "ldb must be a multiple of 8 and cover a row, got %lld", static_cast<long long>(ldb));
  OMNI_REQUIRE((a_transposed && b_transposed) || k % 8 == 0, "k must be a multiple of 8 unless both operands are transposed, got %lld",
               static_cast<long long>(k));
  if (m == 0 || n == 0) return 0;
  OMNI_REQUIRE(a && b && out && status, "NULL argument");
  OMNI_REQUIRE(aligned16(a) && aligned16(b) && aligned16(out), "pointers must be 16-byte aligned");
  OMNI_REQUIRE(use_pairs(), "omni_gemm_bf16 runs on the CTA-pair kernels only (OMNI_MOE_B200_GEMM=1cta is set)");
  CUtensorMap ma, mb;
  // transposed operand: the matrix in memory is [k, m] (or [k, n]); boxes of 64 K rows x 64 elements
  if (int e = a_transposed ? make_map(&ma, a, k, m, 64, lda) : make_map(&ma, a, m, k, BM, lda)) return e;
  CUtensorMap mb1;
  if (b1 != nullptr) {
    // first matrix: K rows [0, k_split); second: the remaining k - k_split rows
    if (int e = make_map(&mb, b, k_split, n, 64, ldb)) return e;
    if (int e = make_map(&mb1, b1, k - k_split, n, 64, ldb)) return e;
  } else {
    if (int e = b_transposed ? make_map(&mb, b, k, n, 64, ldb) : make_map(&mb, b, n, k, 128, ldb)) return e;
    mb1 = mb;
  }
  GemmArgs g{};
  g.router_n = b1 != nullptr ? static_cast<int>(k_split) : 0;
  g.M = static_cast<int>(m), g.N = static_cast<int>(n), g.K = static_cast<int>(k), g.dual = 0;
  g.out = out, g.ldo = ldo, g.residual = nullptr, g.ldr = 0, g.status = status;
  OMNI_SET_TUNING(g);
  g.tiles_m = ceil_div(g.M, 2 * BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(g.N, 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch ((a_transposed ? 2 : 0) | (b_transposed ? 1 : 0)) {
    case 0: return launch_pair<EPI_RES, false, 0>(ma, mb, mb1, mb, mb, g, st);
    case 1: return launch_pair<EPI_RES, false, 1>(ma, mb, mb1, mb, mb, g, st);
    case 2: return launch_pair<EPI_RES, false, 2>(ma, mb, mb1, mb, mb, g, st);
    default: return launch_pair<EPI_RES, false, 3>(ma, mb, mb1, mb, mb, g, st);
  }
}
}  // namespace

extern "C" int omni_gemm_bf16(const void* a, int a_transposed, int64_t lda, const void* b, int b_transposed, int64_t ldb, int64_t m,
                              int64_t n, int64_t k, void* out, int64_t ldo, int32_t* status, void* stream) {
  return gemm_bf16_impl(a, a_transposed, lda, b, nullptr, 0, b_transposed, ldb, m, n, k, out, ldo, status, stream);
}

extern "C" int omni_gemm_bf16_stacked_b(const void* a, int a_transposed, int64_t lda, const void* b0, const void* b1, int64_t k_split,
                                        int64_t ldb, int64_t m, int64_t n, int64_t k, void* out, int64_t ldo, int32_t* status,
                                        void* stream) {
  OMNI_REQUIRE(b0 && b1, "NULL argument");
  OMNI_REQUIRE(k_split > 0 && k_split < k && k_split % 64 == 0, "k_split must be a multiple of 64 inside (0, k), got %lld",
               static_cast<long long>(k_split));
  OMNI_REQUIRE(aligned16(b1), "pointers must be 16-byte aligned");
  return gemm_bf16_impl(a, a_transposed, lda, b0, b1, k_split, 1, ldb, m, n, k, out, ldo, status, stream);
}

extern "C" int omni_mlp_fwd(const void* x, const void* gate_w, const void* up_w, const void* down_w, int64_t num_tokens,
                            int hidden, int intermediate, void* act, const float* residual, void* y, int32_t* status,
                            void* stream) {
  if (int e = omni_mlp_gate_up(x, gate_w, up_w, num_tokens, hidden, intermediate, act, status, stream)) return e;
  return omni_mlp_down(act, down_w, num_tokens, hidden, intermediate, residual, y, status, stream);
}

#ifdef OMNI_TUNING
// Tuning builds only, not part of the public header: while `buf` (device memory, 8 int64 per CTA) is set,
// the GEMM kernels record cycle counters there: {MMA wait-for-operands, MMA wait-for-accumulator,
// MMA total, producer wait-for-stage, producer total, epilogue wait, epilogue store, epilogue total}.
extern "C" OMNI_API void omni_debug_gemm_profile(long long* buf) { g_prof = buf; }
extern "C" OMNI_API void omni_debug_gemm_knobs(int knobs, int grid_limit) { g_knobs = knobs, g_grid_limit = grid_limit; }
#endif
