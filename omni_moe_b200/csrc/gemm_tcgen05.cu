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
// One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer (one lane): fills a ring of shared-memory stages
//   warp 1      allocates TMEM; one lane issues tcgen05.mma and commits to the stage / accumulator barriers
//   warps 2-5   epilogue: each owns the 32 TMEM lanes (= tile rows) its warp id selects
// Two accumulators alternate, so the epilogue of tile i overlaps the MMAs of tile i+1.
//
// Every mbarrier wait is bounded.  A wait that runs out sets OMNI_ST_WAIT_TIMEOUT in the status
// word and raises a CTA-wide abort flag that turns all later waits into no-ops, so the kernel still
// drains, frees its TMEM and returns; the results of such a launch are garbage and the host sees the flag.
// No load in this file uses cluster multicast.
#include <cuda.h>

#include "common.cuh"

namespace omni {
namespace {

constexpr int BM = 128;       // tile rows (UMMA M)
constexpr int BK = 64;        // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;    // K per tcgen05.mma for 16-bit types
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr uint32_t kSpinLimit = 1u << 22;

enum { EPI_F32 = 0, EPI_SWIGLU = 1, EPI_RES = 2 };

struct GemmArgs {
  int M, N, K;          // N: logical output columns (EPI_SWIGLU: activation columns; EPI_F32 dual: per-axis columns)
  int dual;             // EPI_F32: 1 = two B matrices of N rows each, outputs side by side (ldc >= 2N)
  int tiles_m, tiles_n; // tiles_n counts tiles over all axes
  int tiles_n_axis;     // tiles per axis (EPI_F32 dual), else tiles_n
  void* out;
  int64_t ldo;
  const float* residual;  // EPI_RES
  int64_t ldr;
  int* status;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (*abort_flag) return false;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 128) {
      __nanosleep(64);
      if ((i & 1023) == 0 && *abort_flag) return false;
    }
  }
  *abort_flag = 1;
  atomicOr(status, OMNI_ST_WAIT_TIMEOUT);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 columns of fp32: thread i of the warp gets row (lane base + i), columns [c, c+32)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is
// not used for swizzled K-major layouts, descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (ignored)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // version
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 A and B, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
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

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                           const __grid_constant__ CUtensorMap tm_b0,
                                                           const __grid_constant__ CUtensorMap tm_b1,
                                                           const GemmArgs g) {
  using C = Cfg<BN>;
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
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int tm = tile % g.tiles_m, tn = tile / g.tiles_m;
        const int axis = tn / g.tiles_n_axis, tj = tn - axis * g.tiles_n_axis;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, g.status);
          if (*abort_flag) break;
          const uint32_t full = bar_full + 8 * stage;
          mbar_arrive_expect_tx(full, C::kStage);
          tma_load_2d(sA + stage * C::kStageA, &tm_a, kb * BK, tm * BM, full);
          const uint32_t dstB = sB + stage * C::kStageB;
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(dstB, &tm_b0, kb * BK, tj * (BN / 2), full);
            tma_load_2d(dstB + (BN / 2) * BK * 2, &tm_b1, kb * BK, tj * (BN / 2), full);
          } else {
            tma_load_2d(dstB, axis == 0 ? &tm_b0 : &tm_b1, kb * BK, tj * BN, full);
          }
          if (++stage == C::kStages) stage = 0, phase ^= 1;
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, g.status);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status);
          if (*abort_flag) break;
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(sA + stage * C::kStageA);
          const uint64_t bdesc = make_smem_desc(sB + stage * C::kStageB);
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            // advancing K by 16 bf16 = 32 bytes = 2 units of the start-address field
            umma_bf16(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, (kb | ks) != 0);
          }
          umma_commit(bar_empty + 8 * stage);  // frees the stage when these MMAs have read it
          if (++stage == C::kStages) stage = 0, phase ^= 1;
        }
        if (*abort_flag) break;
        umma_commit(bar_tfull + 8 * acc);  // accumulator complete
      }
    }
  } else {
    // ------------------------------- epilogue -----------------------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, +32) are the ones this warp may read
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int tm = tile % g.tiles_m, tn = tile / g.tiles_m;
      const int axis = tn / g.tiles_n_axis, tj = tn - axis * g.tiles_n_axis;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, g.status);
      tc_fence_after();
      if (!ok) break;
      const int row = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      constexpr int OUTC = (EPI == EPI_SWIGLU) ? BN / 2 : BN;  // output columns of this tile
      const int col_tile = (EPI == EPI_F32 && g.dual) ? axis * g.N + tj * OUTC : tj * OUTC;
      const int col_lim = (EPI == EPI_F32 && g.dual) ? (axis + 1) * g.N : g.N;  // exclusive bound of valid columns
#pragma unroll 1
      for (int c = 0; c < OUTC; c += 32) {
        float v[32];
        tmem_ld32(taddr + c, v);
        if (EPI == EPI_SWIGLU) {
          float u[32];
          tmem_ld32(taddr + BN / 2 + c, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = silu(v[i]) * u[i];
        }
        const int col0 = col_tile + c;
        if (row < g.M && col0 < col_lim) {
          const bool full = col0 + 32 <= col_lim;
          if (EPI == EPI_F32) {
            float* o = reinterpret_cast<float*>(g.out) + static_cast<int64_t>(row) * g.ldo + col0;
            if (full && (g.ldo & 3) == 0 && (col0 & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
              for (int i = 0; i < 32 && col0 + i < col_lim; ++i) o[i] = v[i];
            }
          } else {
            if (EPI == EPI_RES && g.residual) {
              const float* r = g.residual + static_cast<int64_t>(row) * g.ldr + col0;
              if (full && (g.ldr & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                  const float4 rv = __ldg(reinterpret_cast<const float4*>(r + i));
                  v[i] += rv.x, v[i + 1] += rv.y, v[i + 2] += rv.z, v[i + 3] += rv.w;
                }
              } else {
                for (int i = 0; i < 32 && col0 + i < col_lim; ++i) v[i] += r[i];
              }
            }
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + static_cast<int64_t>(row) * g.ldo + col0;
            if (full && (g.ldo & 7) == 0) {
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
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

// Map of a row-major bf16 matrix [rows, cols] with boxes of box_rows x 64 columns, 128-byte swizzle.
int make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
  EncodeFn enc = get_encode();
  if (!enc) return fail(-2, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-2, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return 0;
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

template <int BN, int EPI>
int launch(const CUtensorMap& a, const CUtensorMap& b0, const CUtensorMap& b1, const GemmArgs& g, cudaStream_t st) {
  using C = Cfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
      return fail(-2, "cannot raise the shared-memory limit to %d bytes", C::kSmem);
    attr_set = true;
  }
  const int tiles = g.tiles_m * g.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_kernel<BN, EPI><<<grid, kThreads, C::kSmem, st>>>(a, b0, b1, g);
  return check_launch("gemm_kernel");
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" int omni_router_gate(const void* x, const void* gate_x, const void* gate_y, int64_t num_tokens, int hidden,
                                int sqrt_n, float* logits, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(sqrt_n >= 1, "sqrt_n must be >= 1");
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(x && gate_x && gate_y && logits && status, "NULL argument");
  OMNI_REQUIRE(aligned16(x) && aligned16(gate_x) && aligned16(gate_y) && aligned16(logits), "pointers must be 16-byte aligned");
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
  g.out = logits, g.ldo = 2 * static_cast<int64_t>(sqrt_n), g.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
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
  return launch<256, EPI_SWIGLU>(ma, mg, mu, g, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_mlp_down(const void* act, const void* down_w, int64_t num_tokens, int hidden, int intermediate,
                             const float* residual, void* y, int32_t* status, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && num_tokens < (int64_t(1) << 31) - BM, "num_tokens out of range");
  OMNI_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8, got %d", hidden);
  OMNI_REQUIRE(intermediate >= 8 && intermediate % 8 == 0, "intermediate must be a positive multiple of 8, got %d", intermediate);
  if (num_tokens == 0) return 0;
  OMNI_REQUIRE(act && down_w && y && status, "NULL argument");
  OMNI_REQUIRE(aligned16(act) && aligned16(down_w) && aligned16(y) && aligned16(residual), "pointers must be 16-byte aligned");
  const int bn = 128;
  CUtensorMap ma, mb;
  if (int e = make_map(&ma, act, num_tokens, intermediate, BM)) return e;
  if (int e = make_map(&mb, down_w, hidden, intermediate, bn)) return e;
  GemmArgs g{};
  g.M = static_cast<int>(num_tokens), g.N = hidden, g.K = intermediate, g.dual = 0;
  g.tiles_m = ceil_div(g.M, BM);
  g.tiles_n = g.tiles_n_axis = ceil_div(hidden, bn);
  g.out = y, g.ldo = hidden, g.residual = residual, g.ldr = hidden, g.status = status;
  return launch<128, EPI_RES>(ma, mb, mb, g, static_cast<cudaStream_t>(stream));
}

extern "C" int omni_mlp_fwd(const void* x, const void* gate_w, const void* up_w, const void* down_w, int64_t num_tokens,
                            int hidden, int intermediate, void* act, const float* residual, void* y, int32_t* status,
                            void* stream) {
  if (int e = omni_mlp_gate_up(x, gate_w, up_w, num_tokens, hidden, intermediate, act, status, stream)) return e;
  return omni_mlp_down(act, down_w, num_tokens, hidden, intermediate, residual, y, status, stream);
}
