// Dispatch planning for expert tables that are row-partitioned over several GPUs.
//
// A rank routes its own tokens and must send every (token, expert, weight) pair to the rank that owns the expert's
// row.  Its tokens are cut into `chunks` equal ranges that are exchanged one after another, so the pairs are grouped
// by key = chunk * world + owner, in ascending pair order inside a key (the order of the pair list a rank receives is
// then already grouped by token).  Two kernels bracket the library's radix pass over those keys:
//   partition_keys_kernel     key of every pair + how many pairs each key has (the split sizes of the exchange);
//   partition_records_kernel  the 12-byte records (token id among the chunk's all-gathered rows, expert row inside
//                             the owner's slice, weight bits) in sorted order.
// An expert id outside [0, world * rows_per_rank) goes to rank 0 / the last rank with a local row outside the slice,
// where the expert kernels report it (OMNI_ST_BAD_EXPERT_INDEX) and skip the pair.
#include "common.cuh"

namespace omni {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxBins = 2048;  // chunks * world; also what one radix pass of the scheduler covers

__device__ __forceinline__ int owner_of(int e, int64_t rows_per_rank, int world) {
  if (e < 0) return 0;
  const int64_t o = e / rows_per_rank;
  return o >= world ? world - 1 : static_cast<int>(o);
}

__global__ void __launch_bounds__(kThreads) partition_keys_kernel(const int* __restrict__ indices, int64_t P, int k,
                                                                  int64_t rows_per_rank, int world, int64_t tokens_per_chunk,
                                                                  int bins, int* __restrict__ keys, int* __restrict__ counts) {
  __shared__ int hist[kMaxBins];
  for (int b = threadIdx.x; b < bins; b += kThreads) hist[b] = 0;
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; p < P; p += stride) {
    const int e = indices[p];
    const int64_t chunk = (p / k) / tokens_per_chunk;
    const int key = static_cast<int>(chunk) * world + owner_of(e, rows_per_rank, world);
    keys[p] = key;
    atomicAdd(&hist[key], 1);
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kThreads)
    if (hist[b]) atomicAdd(&counts[b], hist[b]);
}

__global__ void __launch_bounds__(kThreads) partition_records_kernel(const int* __restrict__ indices, const float* __restrict__ weights,
                                                                     const int* __restrict__ order, int64_t P, int k,
                                                                     int64_t rows_per_rank, int world, int64_t tokens_per_chunk,
                                                                     int64_t token_base, int* __restrict__ records) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= P) return;
  const int64_t p = order[i];
  int tok = -1, local_e = -1, w_bits = 0;
  if (p >= 0 && p < P) {
    const int e = indices[p];
    const int64_t t = p / k;
    tok = static_cast<int>(t - (t / tokens_per_chunk) * tokens_per_chunk + token_base);
    local_e = static_cast<int>(e - owner_of(e, rows_per_rank, world) * rows_per_rank);
    w_bits = __float_as_int(weights[p]);
  }
  records[3 * i] = tok;
  records[3 * i + 1] = local_e;
  records[3 * i + 2] = w_bits;
}

}  // namespace
}  // namespace omni

using namespace omni;

extern "C" int omni_partition_keys(const int32_t* indices, int64_t num_tokens, int k, int64_t rows_per_rank, int world,
                                   int chunks, int32_t* keys, int32_t* counts, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && rows_per_rank >= 1 && world >= 1 && chunks >= 1, "bad sizes");
  OMNI_REQUIRE(static_cast<int64_t>(world) * chunks <= kMaxBins, "chunks * world must be at most %d", kMaxBins);
  OMNI_REQUIRE(num_tokens % chunks == 0, "the token count %lld is not a multiple of chunks = %d",
               static_cast<long long>(num_tokens), chunks);
  OMNI_REQUIRE(num_tokens * k < (int64_t(1) << 31), "too many pairs");
  OMNI_REQUIRE(counts, "NULL argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int bins = world * chunks;
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * bins, st) != cudaSuccess) return fail(-2, "cannot clear the counts");
  const int64_t P = num_tokens * k;
  if (P == 0) return 0;
  OMNI_REQUIRE(indices && keys, "NULL argument");
  int64_t blocks = ceil_div64(P, kThreads * 8);  // eight pairs per thread: fewer flushes of the block histograms
  if (blocks < 1) blocks = 1;
  partition_keys_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(indices, P, k, rows_per_rank, world,
                                                                           num_tokens / chunks, bins, keys, counts);
  return check_launch("partition_keys_kernel");
}

extern "C" int omni_partition_records(const int32_t* indices, const float* weights, const int32_t* order, int64_t num_tokens,
                                      int k, int64_t rows_per_rank, int world, int chunks, int64_t token_base,
                                      int32_t* records, void* stream) {
  OMNI_REQUIRE(num_tokens >= 0 && k >= 1 && rows_per_rank >= 1 && world >= 1 && chunks >= 1, "bad sizes");
  OMNI_REQUIRE(num_tokens % chunks == 0, "the token count %lld is not a multiple of chunks = %d",
               static_cast<long long>(num_tokens), chunks);
  OMNI_REQUIRE(num_tokens * k < (int64_t(1) << 31), "too many pairs");
  const int64_t P = num_tokens * k;
  if (P == 0) return 0;
  OMNI_REQUIRE(indices && weights && order && records, "NULL argument");
  partition_records_kernel<<<static_cast<unsigned>(ceil_div64(P, kThreads)), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      indices, weights, order, P, k, rows_per_rank, world, num_tokens / chunks, token_base, records);
  return check_launch("partition_records_kernel");
}
