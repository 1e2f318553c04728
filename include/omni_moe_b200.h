/*
 * C ABI of libomni_moe_b200.so: the OmniMoE layer-forward hot path on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream (passed as void*, a
 * cudaStream_t), enqueues its kernels on that stream and returns at once:
 *   0   the work was enqueued
 *   <0  an argument was rejected (omni_last_error() gives the reason); nothing was enqueued
 * No entry point allocates, frees, synchronises or throws.  Scratch memory is supplied by the
 * caller (omni_*_workspace_bytes says how much).  Faults that can only be seen on the device
 * (an expert index out of range, a wait inside a kernel that gave up) are written to the int32
 * status word the caller passes; it stays 0 when all is well and the caller reads it when it
 * chooses to synchronise.
 *
 * Each function names the interface of the reference project (HKUSTDial/omni-moe, paths relative
 * to that project) whose work it takes over.
 */
#ifndef OMNI_MOE_B200_H
#define OMNI_MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define OMNI_API __attribute__((visibility("default")))
#else
#define OMNI_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types of tensor arguments */
enum { OMNI_F32 = 0, OMNI_BF16 = 1, OMNI_F16 = 2 };

/* bits of the device status word */
enum {
  OMNI_ST_BAD_EXPERT_INDEX = 1,  /* an expert index was < 0 or >= num_experts; the pair was skipped */
  OMNI_ST_WAIT_TIMEOUT = 2,      /* a bounded wait inside a kernel ran out; results are invalid */
  OMNI_ST_BAD_TOKEN_INDEX = 4    /* a scheduled pair pointed outside the token range */
};

/* Library ABI version (major * 100 + minor). */
OMNI_API int omni_version(void);

/* Message of the last call on this host thread that returned < 0 ("" if none). */
OMNI_API const char *omni_last_error(void);

/*
 * Product-key top-k over the sqrt(N) x sqrt(N) grid of log_probs_x[i] + log_probs_y[j].
 * Replaces triton_omni_router_func (omni_moe/ops/triton/interface.py:32-51), i.e.
 * OmniRouterFunc.forward / _omni_router_forward and its Triton kernel
 * (omni_moe/ops/triton/omni_router.py:13-95,167-232), and the torch.exp that follows it in
 * the module (omni_moe/modules/omni_moe.py:86).
 *
 *   log_probs_x/y  [T, sqrt_n] row-major, element type in_dtype
 *   scores         [T, k] float32, sorted descending              (may not be NULL)
 *   indices        [T, k] int32 (idx_is_i64 == 0) or int64: ix * sqrt_n + iy
 *   weights        [T, k] float32 = exp(scores), or NULL
 * Sums are formed in fp32.  Ties: higher score wins, then the lower index.
 * Limits: 1 <= sqrt_n <= 1024, 1 <= k <= 128, k <= sqrt_n * sqrt_n.
 */
OMNI_API int omni_router_topk(const void *log_probs_x, const void *log_probs_y, int in_dtype,
                     int64_t num_tokens, int sqrt_n, int k,
                     float *scores, void *indices, int idx_is_i64, float *weights,
                     void *stream);

/*
 * The same selection, starting from raw router-gate outputs: applies the eval-mode BatchNorm
 * (as a per-column scale and shift), the per-axis log-softmax and the top-k in one kernel.
 * Replaces, in OmniMoE.forward, router_norm_x/y, F.log_softmax, triton_omni_router_func and
 * torch.exp (omni_moe/modules/omni_moe.py:70-86).
 *
 *   logits     [T, 2*sqrt_n] float32 with row stride ld_logits: columns [0, sqrt_n) are the
 *              x axis, [sqrt_n, 2*sqrt_n) the y axis
 *   bn_scale, bn_shift  [2*sqrt_n] float32: normalised = logit * scale + shift (NULL = identity)
 *   log_probs_out  [T, 2*sqrt_n] float32 or NULL: the log-probabilities the selection used
 */
OMNI_API int omni_router_logits_topk(const float *logits, int64_t ld_logits,
                            const float *bn_scale, const float *bn_shift,
                            int64_t num_tokens, int sqrt_n, int k,
                            float *scores, void *indices, int idx_is_i64, float *weights,
                            float *log_probs_out, void *stream);

/*
 * Router gate GEMMs: logits[:, 0:sqrt_n] = x . gate_x^T, logits[:, sqrt_n:] = x . gate_y^T,
 * bf16 operands, fp32 accumulation and output (tcgen05 tensor cores, operands by TMA).
 * Replaces the two nn.Linear router gates (omni_moe/modules/omni_moe.py:47-52,70-71).
 *
 *   x        [T, H] bf16 row-major       gate_x, gate_y  [sqrt_n, H] bf16 row-major
 *   logits   [T, 2*sqrt_n] float32 row-major
 * Limits: H % 8 == 0, pointers 16-byte aligned.  status: device int32, see top of file.
 */
OMNI_API int omni_router_gate(const void *x, const void *gate_x, const void *gate_y,
                     int64_t num_tokens, int hidden, int sqrt_n,
                     float *logits, int32_t *status, void *stream);

/*
 * Expert-centric scheduling: stable sort of the T*k (token, expert) pairs by expert, with the
 * CSR description of the expert segments.  Replaces get_scheduling_info, tail path
 * (omni_moe/ops/triton/omni_scheduler.py:48-101): ~12 torch launches and one blocking .item().
 *
 *   indices          [T, k] int32 or int64 expert ids
 *   weights          [T, k] routing weights, element size weight_elem_bytes (2 or 4), or NULL
 *   sorted_pair_ids  [P] int32  the permutation: pairs ordered by (expert, pair id)   P = T*k
 *   sorted_experts   [P] int32  expert id at each sorted position
 *   token_ids        [P] int32  sorted_pair_ids / k, or NULL
 *   sorted_weights   [P] weights in sorted order (same element size), or NULL
 *   expert_ids       [min(P, N)] int32  distinct experts, ascending (first U entries valid), or NULL
 *   offsets          [min(P, N) + 1] int32  segment starts, offsets[U] = P, or NULL
 *   meta             [4] int32 device: {U, max pairs per expert, status word, reserved}; U and the
 *                    maximum are only computed when one of token_ids / sorted_weights / offsets is given
 *   workspace        omni_schedule_workspace_bytes(P, N) bytes, 256-byte aligned
 */
OMNI_API size_t omni_schedule_workspace_bytes(int64_t num_pairs, int64_t num_experts);
OMNI_API int omni_schedule(const void *indices, int idx_is_i64, const void *weights, int weight_elem_bytes,
                  int64_t num_tokens, int k, int64_t num_experts,
                  int32_t *sorted_pair_ids, int32_t *sorted_experts, int32_t *token_ids,
                  void *sorted_weights, int32_t *expert_ids, int32_t *offsets, int32_t *meta,
                  void *workspace, size_t workspace_bytes, void *stream);

/*
 * omni_schedule for callers that cannot hand over scratch memory.  (No counterpart in the reference
 * project: this entry point exists for the embedding side.)
 *
 * Some hosts of this library may not allocate device memory themselves at the point where they
 * schedule: a plugin that only receives the tensors its framework passes in, code running inside a
 * memory-planned region where every buffer was fixed ahead of time, or a service whose allocator is
 * owned by another component.  For them the radix-sort scratch is a fixed 6.5 MiB array inside the
 * library image (every GPU that loads the library holds it until the process exits); this function
 * never calls cudaMalloc, cudaFree or any allocating routine.  The caller still passes all inputs
 * and outputs, with the meaning they have in omni_schedule.
 *
 * Limit: num_tokens * k <= omni_schedule_static_max_pairs() (262144); larger problems are refused
 * with a message and nothing is enqueued.
 * The first call on each device looks up the device address of the built-in array (with that
 * device current); make that first call before any stream capture begins.
 * All calls on a device share the one array, which keeps the previous call's contents: the counters
 * that must start at zero are cleared at the start of each call, but two calls whose kernels overlap
 * on the GPU (different streams without an ordering between them) race on it.  Keep calls on one
 * stream, or order them with events.
 */
OMNI_API int64_t omni_schedule_static_max_pairs(void);
OMNI_API int omni_schedule_static(const void *indices, int idx_is_i64, const void *weights, int weight_elem_bytes,
                         int64_t num_tokens, int k, int64_t num_experts,
                         int32_t *sorted_pair_ids, int32_t *sorted_experts, int32_t *token_ids,
                         void *sorted_weights, int32_t *expert_ids, int32_t *offsets, int32_t *meta,
                         void *stream);

/*
 * Routed experts, y[t] = sum_j w[t,j] * silu(x[t] . Up[e[t,j]]) * Down[e[t,j]], in two kernels:
 * omni_expert_coef walks the pairs in expert order (each Up row is fetched once per run of
 * pairs on that expert) and writes c[t,j] = w[t,j] * silu(x[t] . Up[e]) in fp32;
 * omni_expert_combine forms y[t] = sum_j c[t,j] * Down[e[t,j]] per token, without atomics, so
 * the result does not depend on execution order.
 * Replace omni_expert_forward and its two Triton kernels
 * (omni_moe/ops/triton/omni_expert.py:13-168,920-992) behind triton_omni_expert_func
 * (omni_moe/ops/triton/interface.py:54-72).
 *
 *   x [T, H], up/down [N, H] bf16 row-major; weights [T, k] float32; indices [T, k] int32
 *   sorted_pair_ids, sorted_experts: from omni_schedule
 *   coef [T, k] float32
 *   y [T, H] of out_dtype (OMNI_F32 or OMNI_BF16); residual [T, H] of the same type added in, or NULL;
 *   residual may be y itself (the sum is then added in place)
 * Limits: H % 8 == 0, pointers 16-byte aligned.
 */
OMNI_API int omni_expert_coef(const void *x, const void *up, const float *weights,
                     const int32_t *sorted_pair_ids, const int32_t *sorted_experts,
                     int64_t num_tokens, int k, int hidden, int64_t num_experts,
                     float *coef, int32_t *status, void *stream);
/*
 * omni_expert_coef for skewed routing.  Experts that own long runs of the sorted pair list ("hot" experts: at least
 * min_run pairs, up to 64 of them, taken in sorted order) are handled as a dense product: their Up rows are copied
 * side by side and one tcgen05 GEMM gives x . Up[e] for every token, so their pairs read 4 bytes instead of
 * gathering a token row each.  All other pairs go the way of omni_expert_coef.  The reference treats every pair
 * alike (omni_moe/ops/triton/omni_expert.py:13-168); results agree with omni_expert_coef to fp32 summation order.
 * The set of hot experts depends on the sorted list only, so the result is reproducible.
 *
 *   min_run    pairs an expert must own to be treated densely; <= 0 picks max(512, T / 32)
 *   workspace  device scratch of omni_expert_coef_hot_workspace(T, H) bytes, 16-byte aligned
 * Other arguments and limits as omni_expert_coef.
 */
OMNI_API int64_t omni_expert_coef_hot_workspace(int64_t num_tokens, int hidden);
OMNI_API int omni_expert_coef_hot(const void *x, const void *up, const float *weights,
                         const int32_t *sorted_pair_ids, const int32_t *sorted_experts,
                         int64_t num_tokens, int k, int hidden, int64_t num_experts, int64_t min_run,
                         float *coef, void *workspace, int64_t workspace_bytes,
                         int32_t *status, void *stream);
OMNI_API int omni_expert_combine(const void *down, const float *coef, const int32_t *indices,
                        int64_t num_tokens, int k, int hidden, int64_t num_experts,
                        const void *residual, void *y, int out_dtype,
                        int32_t *status, void *stream);

/*
 * The raw dot products of omni_expert_coef, dots[t, j] = x[t] . Up[e[t, j]] (no activation, no routing weight), for
 * a GPU that holds a COLUMN slice of the expert tables (x [T, Hs] and up [N, Hs] are then the same Hs columns of the
 * token rows and of the Up table): the partial products of all slices are added (an all-reduce of [T, k] floats)
 * before w * silu(.) is applied, and omni_expert_combine over the matching Down columns gives the same columns of y.
 * The reference has no multi-GPU path (the tables being cut are omni_moe/modules/omni_moe.py:57-58).
 * Arguments and limits as omni_expert_coef (hidden = Hs).
 */
OMNI_API int omni_expert_dots(const void *x, const void *up, const int32_t *sorted_pair_ids,
                     const int32_t *sorted_experts, int64_t num_tokens, int k, int hidden,
                     int64_t num_experts, float *dots, int32_t *status, void *stream);

/*
 * Dispatch planning for expert tables that are row-partitioned over `world` GPUs (rank r owns rows
 * [r * rows_per_rank, (r + 1) * rows_per_rank)); the reference has no multi-GPU path, the tables being cut are
 * up_embed / down_embed (omni_moe/modules/omni_moe.py:57-58).  A rank's tokens are cut into `chunks` equal ranges
 * that are exchanged one after another.
 *
 * omni_partition_keys: keys[p] = chunk(p) * world + owner(indices[p]) for every pair p of the [T, k] routing table
 *   and counts[key] = number of pairs with that key (cleared by the call): the split sizes of the exchange.
 * omni_partition_records: records[i] = (token id of pair order[i] among its chunk's all-gathered rows
 *   = token_base + token's offset inside its chunk, expert row inside the owner's slice, bits of the weight),
 *   12 bytes each, for order = the stable sort of the pairs by key (omni_schedule over keys, num_experts =
 *   chunks * world).
 * An expert id outside the table is sent to the first or last rank with a row outside its slice; the expert kernels
 * there report OMNI_ST_BAD_EXPERT_INDEX and skip the pair.
 * Limits: num_tokens % chunks == 0, chunks * world <= 2048, num_tokens * k < 2^31.
 */
OMNI_API int omni_partition_keys(const int32_t *indices, int64_t num_tokens, int k, int64_t rows_per_rank,
                        int world, int chunks, int32_t *keys, int32_t *counts, void *stream);
OMNI_API int omni_partition_records(const int32_t *indices, const float *weights, const int32_t *order,
                           int64_t num_tokens, int k, int64_t rows_per_rank, int world, int chunks,
                           int64_t token_base, int32_t *records, void *stream);

/*
 * The two routed-expert kernels for a GPU that holds only a slice of the expert tables (rows
 * [lo, hi) of Up / Down) and works on a list of (token, local expert, weight) pairs that other GPUs
 * dispatched to it, rather than on a [T, k] routing table.  The reference has no multi-GPU path;
 * these do, per GPU, the work of omni_expert_forward (omni_moe/ops/triton/omni_expert.py:920-992).
 *
 * omni_expert_coef_pairs: c[p] = pair_weights[p] * silu(x[pair_tokens[p]] . Up[e[p]]), pairs walked in
 *   expert order (sorted_pair_ids / sorted_experts from omni_schedule over the pairs' local expert ids).
 * omni_expert_combine_segments: y[t] = sum over the pairs p in [token_offsets[t], token_offsets[t+1])
 *   of coef[p] * Down[pair_experts[p]]  (+ residual); the pair list must be grouped by token.
 *   Tokens without pairs get zeros (or the residual).
 */
OMNI_API int omni_expert_coef_pairs(const void *x, const void *up, const int32_t *pair_tokens,
                           const float *pair_weights, const int32_t *sorted_pair_ids,
                           const int32_t *sorted_experts, int64_t num_pairs, int64_t num_tokens,
                           int hidden, int64_t num_experts, float *coef, int32_t *status, void *stream);
OMNI_API int omni_expert_combine_segments(const void *down, const float *coef, const int32_t *pair_experts,
                                 const int32_t *token_offsets, int64_t num_tokens, int hidden,
                                 int64_t num_experts, const void *residual, void *y, int out_dtype,
                                 int32_t *status, void *stream);

/*
 * The same routed-expert sum in one token-centric kernel, for tables that stay resident in L2
 * (2 * num_experts * hidden * 2 bytes well below the 126 MB L2): a warp holds its token's x row in
 * registers and streams the k Up and Down rows of the token; no scheduling pass and no coefficient
 * array are needed.  Replaces the same reference code as omni_expert_coef + omni_expert_combine
 * (omni_moe/ops/triton/omni_expert.py:13-168,920-992).
 *   coef  [T, k] float32 or NULL: if given, also receives w * silu(x . up) per pair
 * Limits: hidden % 8 == 0 and hidden <= 2048.
 */
OMNI_API int omni_expert_fused(const void *x, const void *up, const void *down, const float *weights,
                      const int32_t *indices, int64_t num_tokens, int k, int hidden, int64_t num_experts,
                      const void *residual, void *y, int out_dtype, float *coef,
                      int32_t *status, void *stream);

/*
 * omni_expert_fused with float32 operands and a float32 result: for callers whose tensors are float32 and who expect
 * float32 arithmetic, as triton_omni_expert_func gives them (omni_moe/ops/triton/interface.py:54-72 computes in the
 * dtype of its inputs; docs/omni_expert.md:24-43 lists float32).  x [T, H], up / down [N, H], weights [T, k],
 * residual / y [T, H] all float32 (residual may be NULL or y itself), indices int32.  hidden % 4 == 0, k <= 128.
 * CUDA cores only (one warp per token); bad indices are skipped and reported in *status.
 */
OMNI_API int omni_expert_fused_f32(const float *x, const float *up, const float *down, const float *weights,
                          const int32_t *indices, int64_t num_tokens, int k, int hidden, int64_t num_experts,
                          const float *residual, float *y, int32_t *status, void *stream);

/*
 * Self-test of the bounded device-side wait (no counterpart in the reference, whose Triton kernels have no
 * device-side waits).  Every mbarrier poll of the GEMM kernels is limited: a wait that is never satisfied gives up
 * after a number of probes, raises its block's abort flag, ORs OMNI_ST_WAIT_TIMEOUT into the status word and
 * returns, so a defect shows as a status bit instead of a hung GPU.  This entry runs that code on a barrier of
 * its own that nobody arrives on, with `probe_limit` probes (1 .. 2^20), on `stream`:
 *   out4[0] |= OMNI_ST_WAIT_TIMEOUT      out4[1] = 0 (the wait returned false)
 *   out4[2] = 0 (a second wait of the block returned false at once)      out4[3] = 1 (the abort flag)
 * out4: 4 int32 of device memory, cleared by the call.  The context stays usable afterwards.
 */
OMNI_API int omni_selftest_wait_timeout(int32_t *out4, int probe_limit, void *stream);

/*
 * Router selection and routed experts in one kernel, for the same regime as omni_expert_fused
 * (tables resident in L2): the BatchNorm fold, the log-softmax and the product-key top-k are applied
 * to the token's router logits (as omni_router_logits_topk does, same results) and the k Up / Down
 * rows are gathered.  Replaces, in OmniMoE.forward, router_norm_x/y,
 * F.log_softmax, triton_omni_router_func, torch.exp and triton_omni_expert_func
 * (omni_moe/modules/omni_moe.py:70-95).
 *   logits [T, 2*sqrt_n] fp32 (row stride ld_logits); x, up, down bf16; y [T, H] bf16;
 *   residual [T, H] bf16 or NULL, may be y itself
 *   scores, indices (int32), weights [T, k]: the routing that was used, each may be NULL
 *   status: device word that receives OMNI_ST_WAIT_TIMEOUT if the bounded wait of the first kernel below gives
 *           up (a defect: the warps it waits for never block); may be NULL
 * Two kernels.  For hidden = 256, 512 or 1024: one block per SM owns a range of tokens and its 16 warps take
 * "select a token" and "gather a selected token" tasks from counters in shared memory, so that the selection
 * arithmetic of some warps overlaps the row gathers of others; the k dot products x . Up[e] run on the tensor
 * cores (mma.sync.m16n8k16: the 16 selected Up rows are the A operand, loaded straight from the table in
 * fragment order; x, kept in shared memory, is the B operand).  The routing is bit-identical to
 * omni_router_logits_topk; the output differs from omni_expert_fused in the last bits (another summation order)
 * and is identical run to run.  Otherwise (hidden % 8 == 0, hidden <= 2048): one warp per token on the CUDA
 * cores, bit-identical to omni_router_logits_topk + omni_expert_fused; OMNI_MOE_B200_ROUTED=legacy selects that
 * kernel for every shape.  Limits of both: sqrt_n <= 256, k <= 32.
 */
OMNI_API int omni_route_expert_fused(const float *logits, int64_t ld_logits,
                            const float *bn_scale, const float *bn_shift,
                            const void *x, const void *up, const void *down,
                            int64_t num_tokens, int sqrt_n, int k, int hidden, int64_t num_experts,
                            const void *residual, void *y,
                            float *scores, int32_t *indices, float *weights, int32_t *status,
                            void *stream);

/*
 * Shared SwiGLU MLP, y = (silu(x Wg^T) * (x Wu^T)) Wd^T (+ residual), as two tcgen05 GEMMs: the
 * first computes the gate and up projections of a tile side by side and applies silu(g)*u in
 * its epilogue (the [T, I] gate and up activations never reach memory), the second applies the
 * down projection and, if given, adds the fp32 residual before rounding to bf16.
 * Replaces triton_omni_mlp_func (omni_moe/ops/triton/interface.py:7-29): three cuBLAS GEMMs and
 * the Triton SwiGLU kernel (omni_moe/ops/triton/omni_mlp.py:103-177,252-303); with residual,
 * also the final add of the module (omni_moe/modules/omni_moe.py:102).
 *
 *   x [T, H], gate_w/up_w [I, H], down_w [H, I]  bf16 row-major
 *   act [T, I] bf16 scratch (caller-owned)     residual [T, H] float32 or NULL     y [T, H] bf16
 * Limits: H % 8 == 0, I % 8 == 0, pointers 16-byte aligned.
 */
OMNI_API int omni_mlp_fwd(const void *x, const void *gate_w, const void *up_w, const void *down_w,
                 int64_t num_tokens, int hidden, int intermediate,
                 void *act, const float *residual, void *y,
                 int32_t *status, void *stream);

/*
 * omni_mlp_gate_up and omni_router_gate in one launch: both multiply the same x, so the router
 * sub-keys are appended to the gate/up GEMM as extra tile columns (fp32 logits out) and x is
 * streamed once.  Replaces gate_proj / up_proj / the SwiGLU kernel and the two router gates
 * (omni_moe/modules/omni_moe.py:70-71,96; omni_moe/ops/triton/interface.py:23-29).
 */
OMNI_API int omni_mlp_gate_up_router(const void *x, const void *gate_w, const void *up_w,
                            const void *gate_x, const void *gate_y,
                            int64_t num_tokens, int hidden, int intermediate, int sqrt_n,
                            void *act, float *logits, int32_t *status, void *stream);

/* The two halves of omni_mlp_fwd, for callers that schedule them on different streams. */
OMNI_API int omni_mlp_gate_up(const void *x, const void *gate_w, const void *up_w,
                     int64_t num_tokens, int hidden, int intermediate,
                     void *act, int32_t *status, void *stream);
OMNI_API int omni_mlp_down(const void *act, const void *down_w,
                  int64_t num_tokens, int hidden, int intermediate,
                  const float *residual, void *y, int32_t *status, void *stream);

/*
 * ---- backward of the three operators --------------------------------------------------------
 *
 * Backward of the router op, scores[t,j] = lpx[t, ix] + lpy[t, iy] with indices[t,j] = ix*sqrt_n + iy:
 * every score gradient is added to one column of each axis.  Replaces _omni_router_backward and its
 * Triton kernel (omni_moe/ops/triton/omni_router.py:104-164,235-274), without atomics: the sums
 * come out the same on every run.
 *   dscores [T, k] float32; indices [T, k] int32 or int64; dlog_probs_x / _y [T, sqrt_n] float32,
 *   fully written (columns no expert touches get 0).  sqrt_n <= 1024.
 */
OMNI_API int omni_router_bwd(const float *dscores, const void *indices, int idx_is_i64, int64_t num_tokens,
                    int sqrt_n, int k, float *dlog_probs_x, float *dlog_probs_y, int32_t *status,
                    void *stream);

/*
 * Backward of the routed-expert op, replacing omni_expert_backward and its Triton kernels
 * (omni_moe/ops/triton/omni_expert.py:380-917,1067-1277).  Per pair p = (t, j), e = indices[t,j],
 * g = weights[t,j]:  S = x[t].Up[e],  h = silu(S),  dA = dy[t].Down[e],
 *   dg[t,j] = dA*h,   cdown[t,j] = g*h,   ds[t,j] = dA*g*silu'(S)
 *   dx[t]   = sum_j ds[t,j] * Up[e]          -> omni_expert_combine(up, ds, indices, ...)
 *   dUp[e]  = sum_{p on e} ds[p] * x[t_p],   dDown[e] = sum_{p on e} cdown[p] * dy[t_p]
 *
 * omni_expert_bwd_dots: token-centric; writes ds, cdown, dg ([T, k] float32 each) and, if dx != NULL, the
 *   input gradient dx [T, H] of dx_dtype as well (the Up rows are in registers for the dot products);
 *   fusing dx is available when omni_expert_bwd_dots_fuses_dx(hidden) != 0 (hidden <= 1024), otherwise
 *   pass NULL and form dx with omni_expert_combine.
 * omni_expert_bwd_rows: expert-centric over the schedule of the same indices (omni_schedule with
 *   expert_ids / offsets / meta requested): one gradient row per touched expert, pairs summed in
 *   ascending pair order in fp32, no atomics.  compact = 0: row e of d_up / d_down ([N, H], rows of
 *   untouched experts are NOT written: zero the tables first); compact = 1: row s of [U, H] for
 *   segment s, expert expert_ids[s] (the reference returns dense zero-filled tables,
 *   omni_expert.py:1097-1098; compact rows avoid 2*N*H bytes of zeros for large tables).
 *   num_segments: device pointer to U (meta[0] of omni_schedule); max_segments: host bound on U
 *   (min(T*k, N)) that sizes the launch.  out_dtype: OMNI_F32 or OMNI_BF16.
 *   scratch: omni_expert_bwd_rows_scratch_bytes(T*k, H) bytes of device memory (256-byte aligned), or
 *   NULL.  With it, experts that received more pairs than one block of sorted positions (256, or 512
 *   when the partial rows of 256-blocks would exceed 256 MiB) are summed in two levels (partial rows
 *   per block, then one pass over the partials, both in a fixed order), so skewed routing does not
 *   serialise on one warp; without it every segment is summed by a single warp.
 *   max_segment_len: device pointer to the longest segment (meta[1] of omni_schedule) or NULL; lets the
 *   two-level kernels return at once when no expert is that busy.
 * Limits: H % 8 == 0, 16-byte aligned pointers.
 */
OMNI_API int omni_expert_bwd_dots(const void *x, const void *up, const void *down, const void *dy,
                         const float *weights, const int32_t *indices, int64_t num_tokens, int k,
                         int hidden, int64_t num_experts, float *ds, float *cdown, float *dg,
                         void *dx, int dx_dtype, int32_t *status, void *stream);
OMNI_API int omni_expert_bwd_dots_fuses_dx(int hidden);
OMNI_API int omni_expert_bwd_rows(const void *x, const void *dy, const float *ds, const float *cdown,
                         const int32_t *sorted_pair_ids, const int32_t *expert_ids,
                         const int32_t *offsets, const int32_t *num_segments,
                         const int32_t *max_segment_len, int64_t max_segments,
                         int64_t num_tokens, int k, int hidden, int compact, void *d_up, void *d_down,
                         int out_dtype, void *scratch, size_t scratch_bytes, int32_t *status, void *stream);
OMNI_API size_t omni_expert_bwd_rows_scratch_bytes(int64_t num_pairs, int hidden);

/*
 * Building blocks of the MLP backward (the reference differentiates its MLP through three
 * nn.functional.linear calls and TritonSwiGLUFunc.backward, omni_moe/ops/triton/interface.py:7-29,
 * omni_moe/ops/triton/omni_mlp.py:181-249,306-375).
 *
 * omni_gemm_bf16_nt: out[m, n] = sum_k a[m, k] * b[n, k]; a [m, k], b [n, k] bf16 row-major (both
 *   with the contraction dimension contiguous), fp32 accumulation on the tcgen05 tensor cores, out
 *   bf16 with row stride ldo >= n.  k % 8 == 0; pointers 16-byte aligned.
 * omni_transpose_bf16: out[c, r] = in[r, c] for an in [rows, cols] with row stride ld_in; out is
 *   [cols, out_cols] with row stride ldo, out_cols >= rows, and its columns rows..out_cols-1 are
 *   zero-filled (padding that keeps rows 16-byte aligned when `rows`, a token count, is not a
 *   multiple of 8).  cols, ld_in, out_cols, ldo even.
 * omni_swiglu_bwd: gate_up [T, 2I] = (gate | up) pre-activations, dact [T, I] ->
 *   dgate_up [T, 2I] = (dact*up*silu'(gate) | dact*silu(gate)) and, if dgate_up_t / act_t are given,
 *   the transposed copies the weight-gradient GEMMs contract over: dgate_up_t [2I, ld_t] and
 *   act_t [I, ld_t] with act = silu(gate)*up, columns T..ld_t-1 zero-filled.
 *   All bf16, arithmetic in fp32.  I % 8 == 0, ld_t even.
 */
/*
 * omni_mlp_gate_up_save: omni_mlp_gate_up that also writes the pre-activations for the backward:
 *   gate_up [T, 2I] bf16 = (x Wg^T | x Wu^T), rounded from the fp32 accumulators (the reference's
 *   TritonSwiGLUFunc saves gate and up the same way, omni_moe/ops/triton/omni_mlp.py:359-375).
 */
OMNI_API int omni_mlp_gate_up_save(const void *x, const void *gate_w, const void *up_w, int64_t num_tokens,
                          int hidden, int intermediate, void *act, void *gate_up, int32_t *status,
                          void *stream);
/*
 * omni_mlp_gate_up_limit / omni_swiglu_bwd_limit: the same two steps with the clamp of the reference's
 *   activation (compute_silu_mul, omni_moe/ops/triton/omni_mlp.py:54-61; PrecisionConfig.limit, :27):
 *   with limit > 0 gate and up are limited to [-limit, limit] before silu(gate) * up; limit == 0 is no
 *   clamp.  gate_up may be NULL (nothing saved); when given it receives the UNCLAMPED pre-activations,
 *   from which omni_swiglu_bwd_limit derives both the clamped values and where no gradient passes
 *   (outside [-limit, limit]; the boundary passes, as torch.clamp's gradient does).
 *   omni_swiglu_bwd_limit also takes act (may be NULL): [T, I] bf16 that receives the recomputed
 *   activation silu(gate) * up untransposed, for callers whose weight-gradient GEMMs read their
 *   operands transposed in place (omni_gemm_bf16) and so need no transposed copies.
 */
OMNI_API int omni_mlp_gate_up_limit(const void *x, const void *gate_w, const void *up_w, int64_t num_tokens,
                           int hidden, int intermediate, float limit, void *act, void *gate_up,
                           int32_t *status, void *stream);
OMNI_API int omni_swiglu_bwd_limit(const void *gate_up, const void *dact, int64_t num_tokens, int intermediate,
                          float limit, void *dgate_up, void *dgate_up_t, void *act_t, int64_t ld_t,
                          void *act, void *stream);
OMNI_API int omni_gemm_bf16_nt(const void *a, const void *b, int64_t m, int64_t n, int64_t k, void *out,
                      int64_t ldo, int32_t *status, void *stream);
/*
 * omni_gemm_bf16: out[m, n] = sum_k A[m, k] * B[n, k] with either operand optionally given transposed,
 *   so that the gradient GEMMs of the backward (dy Wd, dy^T act, (dgate|dup)^T x, ...) read their
 *   operands where they lie:
 *     a_transposed == 0: a is [m, k] row-major with row stride lda;  == 1: a is [k, m] with row stride lda
 *     b_transposed == 0: b is [n, k] row-major with row stride ldb;  == 1: b is [k, n] with row stride ldb
 *   (a_transposed = 0, b_transposed = 0 is omni_gemm_bf16_nt).  bf16 operands, fp32 accumulation on the
 *   tcgen05 tensor cores (a transposed operand is fed as an MN-major shared-memory tile), out bf16
 *   with row stride ldo >= n.  lda, ldb multiples of 8; k % 8 == 0 unless both operands are
 *   transposed (then any k: rows past k are zero-filled by the loads); pointers 16-byte aligned.
 */
OMNI_API int omni_gemm_bf16(const void *a, int a_transposed, int64_t lda, const void *b, int b_transposed,
                   int64_t ldb, int64_t m, int64_t n, int64_t k, void *out, int64_t ldo, int32_t *status,
                   void *stream);
/*
 * omni_gemm_bf16_stacked_b: omni_gemm_bf16 with a transposed B given as two matrices stacked along K:
 *   B^T = (b0 ; b1), b0 [k_split, n] and b1 [k - k_split, n], both with row stride ldb; k_split a
 *   multiple of 64.  out = A (b0 ; b1): the input gradient of two linear layers that share their
 *   input, dx = (dgate | dup) (Wg ; Wu), without concatenating the weights.
 */
OMNI_API int omni_gemm_bf16_stacked_b(const void *a, int a_transposed, int64_t lda, const void *b0, const void *b1,
                             int64_t k_split, int64_t ldb, int64_t m, int64_t n, int64_t k, void *out,
                             int64_t ldo, int32_t *status, void *stream);
OMNI_API int omni_transpose_bf16(const void *in, int64_t rows, int64_t cols, int64_t ld_in, void *out,
                        int64_t out_cols, int64_t ldo, void *stream);
OMNI_API int omni_swiglu_bwd(const void *gate_up, const void *dact, int64_t num_tokens, int intermediate,
                    void *dgate_up, void *dgate_up_t, void *act_t, int64_t ld_t, void *stream);

/*
 * Training-mode BatchNorm of the router logits: batch statistics of logits [T, 2*sqrt_n] (the output
 * of omni_router_gate) over all T tokens, folded into the bn_scale / bn_shift [2*sqrt_n] that
 * omni_router_logits_topk and omni_route_expert_fused take, and the running statistics updated as
 * nn.BatchNorm1d(affine=False) does in training (momentum average with the unbiased variance;
 * num_batches_tracked incremented).  Replaces router_norm_x / router_norm_y in training mode
 * (omni_moe/modules/omni_moe.py:53-54,70-71).  Nothing is allocated and nothing is read back, so a
 * training-mode forward can be captured in a CUDA graph.
 *   eps_*, momentum_*: of the two norm layers; momentum < 0 stands for momentum=None (cumulative
 *   average, 1 / num_batches_tracked)
 *   running_* [sqrt_n] of running_dtype (OMNI_F32 or OMNI_BF16), or NULL (track_running_stats off)
 *   num_batches_tracked_*: int64 device scalars or NULL
 *   scratch: omni_router_bn_train_scratch_bytes(T, sqrt_n) bytes
 */
OMNI_API size_t omni_router_bn_train_scratch_bytes(int64_t num_tokens, int sqrt_n);
OMNI_API int omni_router_bn_train(const float *logits, int64_t ld_logits, int64_t num_tokens, int sqrt_n,
                         float eps_x, float eps_y, float momentum_x, float momentum_y,
                         void *running_mean_x, void *running_var_x, void *running_mean_y,
                         void *running_var_y, int running_dtype, int64_t *num_batches_tracked_x,
                         int64_t *num_batches_tracked_y, float *bn_scale, float *bn_shift,
                         void *scratch, size_t scratch_bytes, void *stream);

/*
 * Backward of the router front as one call: from the gradient of the selected scores back to the
 * gradient of the gate logits, through the gather, the per-axis log-softmax and the BatchNorm
 * (torch autograd does this in the reference through F.log_softmax and nn.BatchNorm1d,
 * omni_moe/modules/omni_moe.py:70-86, and OmniRouterFunc.backward, omni_router.py:235-305).
 *   dscores [T, k] float32, indices [T, k] int32 (as selected in the forward)
 *   log_probs [T, 2*sqrt_n] float32 (the forward's log_probs_out), logits [T, ld_logits] float32
 *   bn_scale / bn_shift [2*sqrt_n]: the fold the forward used (batch statistics in training)
 *   training != 0: the statistics were batch statistics, so the gradient also flows through them
 *   dlogits [T, 2*sqrt_n] bf16 (the operand of the two gate-weight GEMMs that follow)
 *   scratch: omni_router_norm_bwd_scratch_bytes(T, sqrt_n) bytes (training only)
 * Limit: sqrt_n <= 256.  No atomics: the sums are reproducible.
 */
OMNI_API size_t omni_router_norm_bwd_scratch_bytes(int64_t num_tokens, int sqrt_n);
OMNI_API int omni_router_norm_bwd(const float *dscores, const int32_t *indices, const float *log_probs,
                         const float *logits, int64_t ld_logits, const float *bn_scale,
                         const float *bn_shift, int64_t num_tokens, int sqrt_n, int k, int training,
                         void *dlogits, void *scratch, size_t scratch_bytes, int32_t *status,
                         void *stream);

#ifdef __cplusplus
}
#endif
#endif /* OMNI_MOE_B200_H */
