/*
 * fastmoe_b200 — C ABI of the B200 (sm_100a) MoE dispatch/combine hot path.
 *
 * Every entry point takes plain device pointers, 64-bit sizes and an opaque
 * CUDA stream handle (a cudaStream_t passed as void*; NULL = the legacy default
 * stream). Nothing here depends on PyTorch. The library is loaded with dlopen /
 * ctypes / cgo / JNI alike.
 *
 * Return value of every function that returns int:
 *    0   success
 *   <0   argument error (FMOE_ERR_*), nothing was launched
 *   >0   a cudaError_t raised by a launch or a copy
 * fmoe_last_error() gives a human-readable message for the calling thread.
 *
 * None of the device entry points allocates, frees or synchronises unless its
 * comment says so: they only enqueue work on `stream`, so they may be captured
 * in a CUDA graph. Scratch memory is always passed in by the caller
 * (`fmoe_*_bytes` tells how much).
 *
 * Reference interface citations are paths inside polkadot21/fastmoe.
 */
#ifndef FASTMOE_B200_H
#define FASTMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define FMOE_OK 0
#define FMOE_ERR_ARG (-1)         /* null pointer, negative size, bad enum       */
#define FMOE_ERR_UNSUPPORTED (-2) /* valid request this build does not serve      */
#define FMOE_ERR_WORKSPACE (-3)   /* workspace missing, misaligned or too small   */
#define FMOE_ERR_DEVICE (-4)      /* wrong GPU architecture / no device           */

/* element types of the payload ([rows, D] matrices) and of the gate weights */
#define FMOE_F32 0
#define FMOE_BF16 1
#define FMOE_F16 2
/* integer types of the index vector */
#define FMOE_I64 0
#define FMOE_I32 1

/* bits of the device status word (int32, caller-allocated, optional).
 * Kernels OR bits into it and skip the offending row; they never trap.      */
#define FMOE_STATUS_BAD_INDEX 1   /* a target index outside [0, T)            */
#define FMOE_STATUS_BAD_EXPERT 2  /* an expert id outside [0, E)              */
#define FMOE_STATUS_NULL_PTR 4    /* a null entry in the pointer table        */
#define FMOE_STATUS_WAIT_TIMEOUT 8 /* a bounded device-side wait gave up      */

/* ---- library ------------------------------------------------------------ */

/* ABI version, bumped on any signature change. */
int fmoe_abi_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char* fmoe_last_error(void);
/* Name of a status code returned by this library. */
const char* fmoe_status_name(int status);

/* Launch-shape knobs for benchmark sweeps; process-wide, not thread-safe against
 * concurrent launches. Keys: "gather_v" (16-byte vectors per thread: 0 = auto,
 * 1, 2, 4), "gather_threads" (threads per CTA, 0 = auto, else a multiple of 32
 * up to 256), "gather_ctas_per_sm" (-1 = auto, 0 = one CTA per work item,
 * else a persistent grid of 148 x value CTAs), "bwd_ctas_per_sm", "gemm_sms" (SMs the
 * grouped GEMM's persistent grid occupies, 1..148; fewer leaves room for NCCL kernels).
 * "gemm_tokens_as_n" (which of fmoe_grouped_gemm's two forward kernels runs: 1 = the expert's
 * tokens are the MMA's N dimension, in steps of 16 rows; 0 = they are its M dimension, in
 * blocks of 128 rows; -1 = by the average rows per expert, the default),
 * "peer_ctas_per_sm" (CTAs per SM of fmoe_permute_peer_fwd when it sends one group of experts
 * beside a running grouped GEMM: default 2; 0 = one CTA per work item, as for a pass over all),
 * "gemm_prefetch" (weight k-blocks of 64 the grouped GEMM asks into L2 ahead of its loads:
 * 0 = none, the default, since it measured slower; up to 64),
 * "host_chunks" (column slices of fmoe_combine_host's pipelined form: 1 = one slice, i.e.
 * copy in, compute, copy out in sequence, the default; 0 = four slices for rows of 16 KB
 * and more; up to 64).
 * Test hooks: "gemm_spin_limit" (probes per bounded device-side wait) and
 * "gemm_skip_loads" (1 = the GEMM's producer issues no loads, so its consumers' waits run
 * out and the kernel reports FMOE_STATUS_WAIT_TIMEOUT instead of computing). */
int fmoe_tune(const char* key, int value);

/* ---- combine: scatter form ---------------------------------------------- */
/*
 * out[idx[g], :] += src_e[r, :] * w[g]   for g = expert_offsets[e] + r,
 * r < chunk_sizes[e], src_e = (T*)ptr_table[e] with row stride D.
 *
 * Replaces the Triton kernel `_grouped_weighted_scatter_add_kernel`
 * (src/fastmoe/kernels/ops.py:57-194) and its launcher
 * `_launch_grouped_kernel` (ops.py:277-310). One launch over the flattened
 * (expert,row) space; consecutive rows that share a target are summed in fp32
 * registers before one vector `red.global.add` per 16 bytes. Needs no scratch.
 * `out` is accumulated into (never zeroed), as in the reference (ops.py:389-390).
 * Adds land in `out`'s type, so bf16/f16 results depend on the arrival order.
 *
 * ptr_table      int64[E]  device: addresses of the E expert matrices
 * chunk_sizes    int32[E]  device: rows of each expert matrix
 * expert_offsets int64[E]  device: exclusive prefix sum of chunk_sizes
 * idx            [N] device, idx_type FMOE_I64|FMOE_I32: target row in out
 * w              [N] device, w_dtype: gate weight per row
 * out            [T, D] device, dtype, row stride out_row_stride (elements)
 * status         optional int32* device status word
 */
int fmoe_combine_scatter(const int64_t* ptr_table, const int32_t* chunk_sizes,
                         const int64_t* expert_offsets, const void* idx, int idx_type,
                         const void* w, int w_dtype, void* out, int64_t out_row_stride,
                         int64_t E, int64_t N, int64_t T, int64_t D, int dtype,
                         int32_t* status, void* stream);

/* ---- combine: planned (token-major gather) form ------------------------- */
/*
 * The fast path. A plan is the inverse of `idx`: for every output row t the
 * list of source rows that target it, in ascending global row order (the order
 * in which the reference's CPU loop adds them, ops.py:373-384), already
 * resolved through the pointer table to a source address and an fp32 gate
 * weight. With the plan, one CTA owns an output row tile, pulls its source
 * rows with 16-byte loads, accumulates in fp32 registers in that fixed order
 * and writes each output element exactly once: no atomics, no zero-fill pass,
 * bit-reproducible from run to run.
 *
 * The plan lives in caller-provided scratch of fmoe_combine_plan_bytes(N, T)
 * bytes, 256-byte aligned. It stays valid while idx, w, the pointer table and
 * the expert matrices are unchanged; forward and backward share it.
 */
size_t fmoe_combine_plan_bytes(int64_t N, int64_t T);

/* Builds the plan. Replaces `prepare_grouped_metadata`'s device side
 * (ops.py:200-271) plus the per-row lookups of the Triton kernel
 * (ops.py:129-163). One cooperative launch (count, scan, place, resolve, with grid-wide
 * barriers in between) where the device allows it and the sizes fit, else four small
 * launches; no host synchronisation either way. */
int fmoe_combine_plan(const int64_t* ptr_table, const int32_t* chunk_sizes,
                      const int64_t* expert_offsets, const void* idx, int idx_type,
                      const void* w, int w_dtype, int64_t E, int64_t N, int64_t T,
                      int64_t D, int dtype, void* plan, size_t plan_bytes,
                      int32_t* status, void* stream);

/* out[t,:] (=|+=) sum over the plan's rows of t, in plan order, of row*w.
 * accumulate=0 overwrites every row of out (rows without sources become 0):
 * the `GroupedWeightedScatterAdd.forward` semantics (ops.py:318-331) without
 * the torch.zeros pass. accumulate=1 adds to out: the `out=` semantics
 * (ops.py:389-390). */
int fmoe_combine_gather(const void* plan, void* out, int64_t out_row_stride, int64_t N,
                        int64_t T, int64_t D, int dtype, int accumulate, void* stream);

/*
 * The planned combine (plan + gather in one call) for callers that can neither pass
 * scratch memory nor let the library allocate: plugin hosts whose own pool has
 * claimed all device memory, or serving loops that cannot afford the device-wide
 * stall of a cudaMalloc. No counterpart in the reference (it allocates through
 * torch on every call); arguments as for fmoe_combine_plan and fmoe_combine_gather.
 *
 * The plan is built in an array of FMOE_STATIC_SCRATCH_BYTES (4 MiB) that is part of
 * the library's device image: every GPU that loads the library holds it until the
 * process exits. Problems whose plan is larger (fmoe_combine_plan_bytes(N, T) >
 * FMOE_STATIC_SCRATCH_BYTES; N=131072 rows into T=16384 outputs still fits) are
 * refused with FMOE_ERR_WORKSPACE. The call allocates and frees nothing.
 *
 * The first call on each device looks up the array's device address (that device
 * must be current, as for every call): make that first call before any stream
 * capture begins. All calls share the one array per device and it keeps the last
 * call's contents (what must start at zero is cleared on `stream` each time), so two
 * calls that may overlap on the GPU, e.g. on different streams without an ordering
 * between them, race on it; order them yourself.
 */
#define FMOE_STATIC_SCRATCH_BYTES 4194304
int fmoe_combine_fwd_static(const int64_t* ptr_table, const int32_t* chunk_sizes,
                            const int64_t* expert_offsets, const void* idx, int idx_type,
                            const void* w, int w_dtype, void* out, int64_t out_row_stride,
                            int64_t E, int64_t N, int64_t T, int64_t D, int dtype,
                            int accumulate, int32_t* status, void* stream);

/*
 * Backward of the combine (replaces `GroupedWeightedScatterAdd.backward`,
 * ops.py:334-359, and adds the gate gradient the reference leaves out at
 * ops.py:358-359; the reference's CPU path produces it through autograd):
 *   grad_rows[g, :] = grad_out[idx[g], :] * w[g]           ([N, D], dtype)
 *   grad_w[g]       = sum_c grad_out[idx[g], c] * src_g[c]  (fp32, optional)
 * grad_out is read once per output row; grad_w may be NULL.
 */
int fmoe_combine_bwd(const void* plan, const void* grad_out, int64_t grad_out_row_stride,
                     void* grad_rows, float* grad_w, int64_t N, int64_t T, int64_t D,
                     int dtype, void* stream);

/*
 * The combine straight from the routing index, without a plan: where the rows to be
 * combined are ONE matrix in sorted-slot order and the index builder's inverse map is at
 * hand (inside the MoE layer: MoEFeedForward.unpermute, src/fastmoe/models/tiny_model.py:
 * 396-409, which the reference always calls with one tensor), the plan's counting sort is
 * redundant: token t's sources are rows slot_of[t*K + k], k < K.
 *   out[t, :] (=|+=) sum_k rows[slot_of[t*K+k], :] * w_sorted[slot_of[t*K+k]]    (k ascending, fp32)
 * rows [T*K, D] dtype, row stride D; slot_of int32[T*K]; w_sorted [T*K] w_dtype (the gate
 * weight of each sorted slot). No scratch memory, one launch, same token-major kernel.
 * The backward writes grad_rows[s, :] = grad_out[t, :] * w_sorted[s] and (optional, fp32)
 * grad_w[s] = <grad_out[t, :], rows[s, :]> for s = slot_of[t*K+k].
 */
int fmoe_combine_routed(const void* rows, const int32_t* slot_of, const void* w_sorted, int w_dtype,
                        void* out, int64_t out_row_stride, int64_t T, int64_t K, int64_t D, int dtype,
                        int accumulate, void* stream);
int fmoe_combine_routed_bwd(const void* rows, const int32_t* slot_of, const void* w_sorted, int w_dtype,
                            const void* grad_out, int64_t grad_out_row_stride, void* grad_rows,
                            float* grad_w, int64_t T, int64_t K, int64_t D, int dtype, void* stream);

/* ---- router: top-k + gate softmax ---------------------------------------- */
/*
 * Per token: the K largest of E logits in descending order (ties: lower expert
 * id first), then softmax over those K values in fp32, rounded to w_dtype.
 * Replaces torch.topk + F.softmax in `MoEFeedForward.gate_and_sort`
 * (src/fastmoe/models/tiny_model.py:97-100).
 * logits [T, E] dtype; topk_idx int64 [T, K]; topk_w [T, K] w_dtype.
 */
int fmoe_route_topk(const void* logits, int dtype, int64_t T, int64_t E, int64_t K,
                    int64_t* topk_idx, void* topk_w, int w_dtype, void* stream);

/* ---- index / offset builder ---------------------------------------------- */
/*
 * Stable counting sort of the T*K routed slots by expert id (ties by flat
 * position t*K+k), replacing argsort + gathers + bincount
 * (tiny_model.py:105-153):
 *   reverse_map[i]  int64[N]  token of sorted slot i
 *   sorted_w[i]     [N] w_dtype gate weight of sorted slot i
 *   counts[e]       int64[E]  rows per expert (torch.bincount)
 *   offsets[e]      int64[E]  exclusive prefix sum of counts
 *   rank_counts[r]  int64[world] rows per owning rank (E/world experts each)
 *   slot_of[t*K+k]  int32[N]  sorted position of routed slot (t,k): the
 *                   inverse map that the permute and the combine consume
 * scratch: fmoe_build_index_bytes(T, E, K) bytes, 256-byte aligned.
 */
size_t fmoe_build_index_bytes(int64_t T, int64_t E, int64_t K);
int fmoe_build_index(const int64_t* topk_idx, const void* topk_w, int w_dtype, int64_t T,
                     int64_t E, int64_t K, int64_t world, int64_t* reverse_map,
                     void* sorted_w, int64_t* counts, int64_t* offsets,
                     int64_t* rank_counts, int32_t* slot_of, void* scratch,
                     size_t scratch_bytes, int32_t* status, void* stream);

/* ---- dispatch permute ------------------------------------------------------ */
/*
 * permuted[slot_of[t*K+k], :] = x[t, :]   (tiny_model.py:133, `x_flat[rev]`),
 * token-major: each row of x is read once and written K times.
 */
int fmoe_permute_fwd(const void* x, int64_t x_row_stride, const int32_t* slot_of,
                     void* permuted, int64_t T, int64_t K, int64_t D, int dtype,
                     void* stream);
/* grad_x[t, :] = sum_k grad_permuted[slot_of[t*K+k], :] in fp32, ascending k
 * (the index_put(accumulate) that autograd runs for tiny_model.py:133). */
int fmoe_permute_bwd(const void* grad_permuted, const int32_t* slot_of, void* grad_x,
                     int64_t grad_x_row_stride, int64_t T, int64_t K, int64_t D,
                     int dtype, void* stream);

/*
 * Dispatch permute fused with the expert-parallel exchange: row (t,k) of x is written
 * straight into the receive buffer of the GPU that owns its expert, at its final
 * expert-major position, with plain peer stores over NVLink. It stands for the permute
 * (tiny_model.py:133) plus the payload all-to-all (tiny_model.py:210-216) plus the
 * regrouping on the receiver.
 *   expert = topk_idx[t*K+k], dest GPU = expert / experts_per_rank,
 *   dest row = dst_row0[expert] + (slot_of[t*K+k] - local_offsets[expert])
 *   written to (char*)peer_bases[dest GPU] + dest row * D * sizeof(element)
 * dst_row0, local_offsets int64[E]; peer_bases int64[world] (device array of mapped base
 * addresses, own buffer included); rows at or beyond cap_rows are dropped and flagged with
 * FMOE_STATUS_BAD_INDEX. ret_local (optional) is this GPU's own return buffer [T*K, D], one
 * row per sorted slot, which the experts' GPUs fill later: the row of a dropped copy is
 * zeroed in it, since nobody will send a result for it, so that the combine adds zero for
 * that copy rather than what an earlier call left in the buffer (the reference's fixed-size
 * exchange hands such rows "garbage", tiny_model.py:360-367). The caller orders the
 * consumers after all writers (a barrier).
 */
int fmoe_permute_peer_fwd(const void* x, int64_t x_row_stride, const int64_t* topk_idx,
                          const int32_t* slot_of, const int64_t* local_offsets,
                          const int64_t* dst_row0, const int64_t* peer_bases, int64_t T, int64_t K,
                          int64_t D, int64_t E, int64_t experts_per_rank, int64_t cap_rows,
                          void* ret_local, int64_t local_lo, int64_t local_hi, int dtype,
                          int32_t* status, void* stream);
/* local_lo, local_hi: only the copies for experts whose index on their owning GPU
 * (expert % experts_per_rank) lies in [local_lo, local_hi) are sent; 0 and experts_per_rank
 * send everything. Sending group after group lets the experts of one group compute while the
 * rows of the next are still crossing NVLink: the overlap that the reference builds from token
 * micro-batches on two streams (tiny_model.py:506-630), without thinning the rows per expert. */

/*
 * Barrier between the GPUs that share the exchange buffers, as one tiny kernel on `stream`:
 * work enqueued after it on any rank's stream starts only when every rank's work enqueued
 * before it (peer stores included) is complete and visible. flag_bases int64[world] (device)
 * holds, for every rank, the mapped address of that rank's flag array (int32[world], zeroed
 * once before the first barrier); seq is the number of this barrier, the same on all ranks,
 * starting at 1 and growing by one per call. Takes the place of the dist.barrier / blocking
 * collectives that order the reference's exchanges (tiny_model.py:182, :195, :210). The wait
 * is bounded: a rank that does not arrive within timeout_ms sets FMOE_STATUS_WAIT_TIMEOUT
 * in `status` and the kernel returns, so a missing peer never hangs the GPU.
 */
int fmoe_peer_barrier(const int64_t* flag_bases, int64_t world, int64_t rank, int32_t seq,
                      int64_t timeout_ms, int32_t* status, void* stream);

/*
 * Placement arithmetic of that exchange, on the device: from the all-gathered counts
 * counts_all[s * E + g] (rows that rank s routes to global expert g; E/world experts per
 * rank, contiguous) it writes, for rank `rank`:
 *   dst_row0[g]       int64[E]        row on expert g's owner where THIS rank's rows for g begin
 *   counts_local[e]   int64[E/world]  rows this rank's expert e receives, cut off at cap_rows
 *   offsets_local[e]  int64[E/world]  their first rows (expert-major, sources in rank order)
 *   rows_used         int64[1]        rows of the receive buffer in use (<= cap_rows)
 *   row_ptrs[i]       int64[cap_rows] ret_bases[source rank of row i] + row_bytes * (sorted slot
 *                                     the row came from): where the result of receive row i goes
 *                                     (fmoe_grouped_gemm's c_row_ptrs); 0 beyond rows_used
 *   grad_row_ptrs     optional, the same from grad_ret_bases (the gradients' return trip)
 * It stands for the two count exchanges and the host-side split arithmetic of
 * MoEFeedForward.dispatch_exchange (src/fastmoe/models/tiny_model.py:176-208), without the
 * two device-to-host reads (:187, :198-199). When more than cap_rows rows are routed to this
 * rank, FMOE_STATUS_BAD_INDEX is set. scratch: 2*E int64. E <= 1024. Two small launches.
 */
int fmoe_ep_layout(const int64_t* counts_all, int64_t world, int64_t E, int64_t rank, int64_t cap_rows,
                   int64_t row_bytes, const int64_t* ret_bases, const int64_t* grad_ret_bases,
                   int64_t* dst_row0, int64_t* counts_local, int64_t* offsets_local, int64_t* rows_used,
                   int64_t* row_ptrs, int64_t* grad_row_ptrs, int64_t* scratch, int32_t* status,
                   void* stream);

/* ---- expert FFN: grouped GEMM on tcgen05 ------------------------------------------ */
/* what the epilogue applies to the product before the one rounding to bf16 */
#define FMOE_ACT_NONE 0
#define FMOE_ACT_SWIGLU 1 /* silu(gate half) * (up half): the output has N/2 columns */
#define FMOE_ACT_GELU 2   /* exact GELU, 0.5 x (1 + erf(x / sqrt 2)), as torch.nn.GELU() */
/*
 * For every expert e with rows [offsets[e], offsets[e] + counts[e]) of A:
 *   FMOE_ACT_NONE:    C[rows, :N]   = A[rows, :K] x W[e]^T                  W[e] is [N, K]
 *   FMOE_ACT_GELU:    C[rows, :N]   = gelu(A[rows, :K] x W[e]^T)
 *   FMOE_ACT_SWIGLU:  C[rows, :N/2] = silu(A x Wg[e]^T) * (A x Wu[e]^T)     W[e] = [Wg; Wu], each [N/2, K]
 * A [R, K], W [E, N, K], C bf16 row-major; offsets/counts int64[E] ON THE DEVICE (the index
 * builder's output: the host never learns the counts). fp32 accumulation in tensor
 * memory, one rounding to bf16. K must be a multiple of 64, N of 256, E <= 1024.
 * Replaces the per-expert Python loop of cuBLAS GEMMs in MoEFeedForward.compute_experts
 * (src/fastmoe/models/tiny_model.py:282-294; the reference's experts are
 * Linear-GELU-Linear, tiny_model.py:68-77: one FMOE_ACT_GELU call and one FMOE_ACT_NONE call;
 * SwiGLU is what the expert-parallel benchmark configuration asks for). Rows of A outside
 * every expert's range are not touched in C. An expert whose range runs past row R of A is
 * cut off at R (and FMOE_STATUS_BAD_EXPERT is set): no tile reads or writes beyond A's rows.
 * c_row_map (optional int64[R] on the device, NULL = identity) sends the result of A's row
 * r to row c_row_map[r] of C: the return-trip reordering of the expert-parallel layer
 * (expert-major rows back to source-rank-major) happens in the store, not in a copy.
 * c_row_ptrs (optional int64[R] on the device, NULL = unused; takes precedence over
 * c_row_map) gives the ADDRESS of the output row of A's row r, which may lie in another
 * GPU's memory mapped into this process (plain peer stores; a zero entry falls back to C):
 * the expert outputs then travel to the GPUs that own the tokens inside the epilogue.
 * A bounded device-side wait that gives up sets FMOE_STATUS_WAIT_TIMEOUT in `status`.
 */
int fmoe_grouped_gemm(const void* a, const void* w, void* c, const int64_t* offsets,
                      const int64_t* counts, const int64_t* c_row_map, const int64_t* c_row_ptrs,
                      int64_t E, int64_t R, int64_t N, int64_t K, int activation, int32_t* status,
                      void* stream);

/* The same product for a forward pass that will be differentiated: besides C it stores the
 * product BEFORE the activation into pre ([R, N] bf16, row r of A -> row r of pre, whatever
 * c_row_map / c_row_ptrs do to C; for FMOE_ACT_SWIGLU the gate columns followed by the up
 * columns), so that the backward's activation derivative (fmoe_swiglu_bwd, fmoe_gelu_bwd)
 * needs no second product. What autograd keeps of Linear's output before the activation in
 * MoEFeedForward.compute_experts (src/fastmoe/models/tiny_model.py:282-294). */
int fmoe_grouped_gemm_keep_pre(const void* a, const void* w, void* c, void* pre, const int64_t* offsets,
                               const int64_t* counts, const int64_t* c_row_map, const int64_t* c_row_ptrs,
                               int64_t E, int64_t R, int64_t N, int64_t K, int activation, int32_t* status,
                               void* stream);

/*
 * Data gradient of the plain grouped GEMM: grad_a[rows of e, :K] = grad_c[rows of e, :N] x W[e]
 * (W[e] is [N, K], read as it lies in memory: its N rows are the reduction dimension and
 * its K columns the output columns, so no transposed copy of the weights is needed). Same
 * kernel, same ragged-row handling and limits as fmoe_grouped_gemm; N must be a multiple of
 * 64 and K of 256. row_ptrs (optional int64[R] on the device) gives the address of every
 * output row, as c_row_ptrs does for fmoe_grouped_gemm: the gradients of the dispatched rows
 * then travel back to the GPUs that own the tokens inside the epilogue (grad_a may be NULL).
 * Stands for `g @ w[e]` per expert in the autograd backward of
 * MoEFeedForward.compute_experts (src/fastmoe/models/tiny_model.py:282-294).
 */
int fmoe_grouped_gemm_dgrad(const void* grad_c, const void* w, void* grad_a, const int64_t* offsets,
                            const int64_t* counts, const int64_t* row_ptrs, int64_t E, int64_t R,
                            int64_t N, int64_t K, int32_t* status, void* stream);

/*
 * Weight gradient of the grouped GEMM: grad_w[e] = grad_c[rows of e]^T x a[rows of e], bf16
 * [E, N, K] with fp32 accumulation; experts without rows get zeros. The reduction runs over
 * the expert's rows (ragged; the counts stay on the device). N must be a multiple of 128
 * and K of 256. Stands for `g.t() @ x` per expert in the autograd backward of
 * MoEFeedForward.compute_experts (src/fastmoe/models/tiny_model.py:282-294).
 */
int fmoe_grouped_gemm_wgrad(const void* grad_c, const void* a, void* grad_w, const int64_t* offsets,
                            const int64_t* counts, int64_t E, int64_t R, int64_t N, int64_t K,
                            int32_t* status, void* stream);

/*
 * Derivative of the fused SwiGLU epilogue: from the pre-activations h = [gate | up]
 * ([rows, 2*ff] bf16, recomputed with the plain grouped GEMM) and the gradient of
 * silu(gate) * up ([rows, ff] bf16), writes [d_gate | d_up] ([rows, 2*ff] bf16), the
 * operand of the gate/up GEMM's data and weight gradients. One streaming pass.
 */
int fmoe_swiglu_bwd(const void* h, const void* grad_act, void* grad_h, int64_t rows, int64_t ff,
                    void* stream);
/* The same over a capacity-sized buffer whose row count lives on the device: only the first
 * min(rows, *rows_used) rows are read and written (rows_used may be NULL = all rows). Used
 * by the fused expert-parallel exchange, whose receive buffers are sized for the worst case. */
int fmoe_swiglu_bwd_ragged(const void* h, const void* grad_act, void* grad_h, int64_t rows, int64_t ff,
                           const int64_t* rows_used, void* stream);

/* Derivative of the FMOE_ACT_GELU epilogue: from the pre-activations h ([rows, n] bf16,
 * recomputed with FMOE_ACT_NONE) and the gradient of gelu(h), writes grad_h = grad_act *
 * gelu'(h) ([rows, n] bf16), the operand of the first GEMM's data and weight gradients
 * (the backward of nn.GELU() between the two linears of tiny_model.py:70-74). n % 8 == 0. */
int fmoe_gelu_bwd(const void* h, const void* grad_act, void* grad_h, int64_t rows, int64_t n,
                  void* stream);

/* ---- host-buffer call -------------------------------------------------------- */
/*
 * The whole combine for a caller that holds HOST memory: copies the E expert
 * matrices, idx and w into `arena` (device scratch of at least
 * fmoe_combine_host_arena_bytes(...) bytes, caller-allocated), builds the
 * pointer table and the plan there, runs the gather and copies out[T, D] back
 * to `out_host`. Host buffers should be pinned for full PCIe speed. The call
 * returns after the stream has drained (it synchronises `stream`). With
 * fmoe_tune("host_chunks", n > 1) the rows travel in n slices of columns: a slice
 * is gathered and copied back on a helper stream of the library (one per device,
 * created on first use) while the next slice is still arriving, so the two PCIe
 * directions overlap; the result does not depend on the slicing. Off by default:
 * on the B200 hosts measured, the strided copies in cost more than the overlap
 * returns (T=8192, D=16384, E=256, top-8, bf16: 45.0 ms in one piece, 44.9 ms in
 * two slices, 47.2 ms in four, 52.0 ms in eight).
 * Mirrors `grouped_weighted_scatter_add(expert_tensors, indices, weights,
 * out_shape)` (ops.py:365-394) for host callers.
 */
size_t fmoe_combine_host_arena_bytes(const int64_t* chunk_sizes_host, int64_t E, int64_t N,
                                     int64_t T, int64_t D, int dtype);
int fmoe_combine_host(const void* const* expert_rows_host, const int64_t* chunk_sizes_host,
                      const void* idx_host, int idx_type, const void* w_host, int w_dtype,
                      void* out_host, int64_t E, int64_t N, int64_t T, int64_t D, int dtype,
                      void* arena, size_t arena_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FASTMOE_B200_H */
