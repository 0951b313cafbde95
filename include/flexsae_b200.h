/*
 * flexsae_b200 -- C ABI of the B200 (sm_100a) decoder-loss library.
 *
 * The library implements the two fused sparse-autoencoder decoder losses of flex_sae,
 *
 *   TopK          loss = mean_{b,d}   (bias + sum_k     vals[b,k] * weight[indices[b,k]] - target[b])^2
 *   Hierarchical  loss = mean_{b,k,d} (bias + sum_{i<=k} vals[b,i] * weight[indices[b,i]] - target[b])^2
 *
 * and their gradients with respect to weight, vals and bias.  Every pointer below is a DEVICE
 * pointer unless its name ends in _host; all tensors are dense row-major.  No entry point
 * allocates or frees device memory, synchronises the stream or touches the default stream:
 * work is enqueued on the stream handle passed in (a cudaStream_t cast to void*; NULL is the
 * legacy default stream).  Scratch memory comes from the caller, sized by the *_workspace_bytes
 * functions.  Return value: 0 on success, a negative FLEXSAE_E* code for rejected arguments,
 * or the positive cudaError_t of a failed launch; flexsae_last_error() describes the last
 * failure of the calling thread.
 *
 * Each entry point names the part of the reference it stands in for
 * (paths are relative to the reference's repository root).
 */
#ifndef FLEXSAE_B200_H
#define FLEXSAE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of weight / vals / bias / target */
#define FLEXSAE_F32 0
#define FLEXSAE_BF16 1
#define FLEXSAE_F16 2

/* loss kinds */
#define FLEXSAE_TOPK 0
#define FLEXSAE_HIER 1

/* how dweight is accumulated */
#define FLEXSAE_DW_ATOMIC 0        /* vectorised red.global.add.f32 into an L2-resident slab */
#define FLEXSAE_DW_DETERMINISTIC 1 /* stable sort by decoder row + fixed-order segmented sums */
#define FLEXSAE_DW_ATOMIC_SHARDED 2 /* only for flexsae_bwd_workspace_bytes: what flexsae_loss_bwd_sharded needs */
#define FLEXSAE_DW_ATOMIC_WIDE 3    /* as FLEXSAE_DW_ATOMIC with the widest column pieces (32 lanes per batch row unless
                                       "lanes_bwd" says otherwise): for heavily skewed indices, see flexsae_index_skew */

/* error codes */
#define FLEXSAE_EINVAL (-1)      /* bad shape, dtype code, null pointer or misaligned pointer */
#define FLEXSAE_EWORKSPACE (-2)  /* workspace smaller than *_workspace_bytes() */
#define FLEXSAE_EUNSUPPORTED (-3)/* shape outside what the kernels handle */

/* bits of the optional device status word */
#define FLEXSAE_STATUS_BAD_INDEX 1 /* an index outside [0,F) was met; it was read as row 0 */
#define FLEXSAE_STATUS_PIPELINE_TIMEOUT 2 /* a bounded wait inside a kernel gave up (option "wait_limit_ms"): the results of
                                             that call are invalid; read the word after every step of a sharded run */

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int flexsae_version(void);

/* Text of the last error on this thread ("" if none). No reference counterpart: the reference
 * validates nothing and fails inside Triton. */
const char* flexsae_last_error(void);

/* Tuning knobs, process-wide: "lanes_fwd", "lanes_bwd", "lanes_sharded" (8, 16, 32 lanes share one
 * batch row; 0 = choose so that one column piece of the decoder and its fp32 gradient slabs stay in
 * L2; the batch-sharded backward takes wider pieces, see "lanes_sharded"),
 * "l2_budget_mb" (working set one column piece may occupy; the single-GPU atomic backward uses 4/5 of
 * it while a decoder row receives at most 8 contributions on average, B*K <= 8*F), "segments"
 * (what flexsae_choose_segments answers; 0 = derive from the shape), "pipeline" (1: the atomic
 * backward runs all column pieces in one launch; 0: one launch per piece), "convert_offset_pct",
 * "direct_f32" (1: with an fp32 decoder the reductions go straight into dweight),
 * "ticket_order" (1: the blocks of the single-launch backward take their roles from an atomic
 * ticket, i.e. in the order in which they really start, instead of from blockIdx.x),
 * "slabs" (2..4 fp32 accumulation slabs in rotation) and "convert_lag" (1 .. slabs-1: the slab of a
 * column piece is converted that many pieces after it was accumulated, so that the conversion never
 * waits for the piece's last accumulating blocks and nobody waits for the conversion),
 * "exchange_blocks" and "exchange_offset_pct" (sharded backward: how many blocks per column piece
 * do the cross-GPU exchange and how far into the piece's blocks they are placed), "scatter_rotate"
 * (1: each rank starts its scatter sweeps at a different block of batch rows, so that the ranks do
 * not push to the same owner at the same moment; 0: off; -1, the default: on from 4 ranks up -- it
 * costs 3 % on two GPUs and gains 3 % on four), "flag_fan_out" (1: a finished slot is announced to
 * all ranks by parallel stores; 0 and -1 as before), "sharded_convert_blocks" and
 * "sharded_convert_offset_pct" (sharded backward: number and placement of the converting blocks
 * when they differ from the single-GPU kernel's; 0 / -1 = the same; the placement defaults to 45), "wait_limit_ms" (how long any
 * one wait inside a kernel -- for other blocks of the launch, for another GPU -- may last before it
 * gives up and sets FLEXSAE_STATUS_PIPELINE_TIMEOUT; 5000 by default, measured on the GPU's own
 * nanosecond timer; a rank of a sharded run that enqueues its backward later than that after the
 * others makes them give up, so keep it well above any host-side stall).
 * Stands in for the literal tile constants at the reference's launch sites
 * (torch-ext/flex_sae/hierarchical_kernels.py:220-224,263-267; topk_kernels.py:64-66,181-183).
 * Returns 0, or FLEXSAE_EINVAL for an unknown name or value. */
int flexsae_set_option(const char* name, int64_t value);
int64_t flexsae_get_option(const char* name);

/* The backward of one batch row can be cut into independent K-segments when the forward leaves
 * the running state at each segment boundary; small batches need that to fill the GPU.
 * flexsae_choose_segments answers how many segments to use for a shape (0 on invalid arguments);
 * the same number must be given to the forward, the backward and flexsae_state_bytes, which
 * answers the size of the float32 state buffer the forward writes for the backward:
 * B*D floats (TopK, or Hierarchical with one segment) or 2*segments*B*D floats (Hierarchical
 * with several segments).
 * Stands in for final_recon[B,D] saved by the reference forward
 * (torch-ext/flex_sae/hierarchical_kernels.py:201,285). */
int flexsae_choose_segments(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype);
size_t flexsae_state_bytes(int kind, int64_t B, int64_t K, int64_t D, int segments);

/* Scratch bytes the forward / backward need for this shape (0 on invalid arguments).
 * Stands in for the torch.zeros / torch.empty temporaries the reference's launchers allocate
 * (hierarchical_kernels.py:200-201,241-243; topk_kernels.py:146-166). */
size_t flexsae_fwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D,
                                   int weight_dtype);
size_t flexsae_bwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D,
                                   int weight_dtype, int dw_mode);

/*
 * Forward of either loss.
 *   indices [B,K] int64, weight [F,D], vals [B,K], bias [D], target [B,D]
 *   loss_out   one float32: the loss, already divided by the normaliser
 *   state_out  flexsae_state_bytes() of float32: reconstruction minus target at the end of every
 *              K-segment (and, Hierarchical, the running sum of those residuals over k)
 *   segments   from flexsae_choose_segments (1 is always valid)
 *   inv_norm   1/(B*D) (TopK) or 1/(B*K*D) (Hierarchical); pass the GLOBAL batch size when B is
 *              one shard of a larger batch; <= 0 means "derive from B"
 *   status     optional int32 word, OR-ed with FLEXSAE_STATUS_* bits (may be NULL)
 * kind = FLEXSAE_HIER replaces _hierarchical_sae_forward + hierarchical_sae_forward_kernel
 *   (torch-ext/flex_sae/hierarchical_kernels.py:12-89,190-227);
 * kind = FLEXSAE_TOPK replaces embedding_bag_forward + its kernel and the eager
 *   bias/residual/square/mean tail (torch-ext/flex_sae/topk_kernels.py:15-68,220-222).
 */
int flexsae_loss_fwd(int kind, const int64_t* indices, const void* weight, const void* vals,
                     const void* bias, const void* target, float* loss_out, float* state_out,
                     int segments, void* workspace, size_t workspace_bytes, int64_t B, int64_t K,
                     int64_t F, int64_t D, int weight_dtype, int vals_dtype, int bias_dtype,
                     int target_dtype, double inv_norm, int32_t* status, void* stream);

/*
 * Backward of either loss.
 *   state      what flexsae_loss_fwd wrote for the same inputs and the same `segments`
 *   grad_out   one float32 ON THE DEVICE: the upstream gradient of the scalar loss
 *   dweight    [F,D] in weight_dtype, fully overwritten (untouched rows become 0)
 *   dvals      [B,K] in vals_dtype, dbias [D] in bias_dtype, fully overwritten
 *   dw_mode    FLEXSAE_DW_ATOMIC, FLEXSAE_DW_ATOMIC_WIDE or FLEXSAE_DW_DETERMINISTIC
 * kind = FLEXSAE_HIER replaces _hierarchical_sae_backward + hierarchical_sae_backward_kernel and
 *   the dW.mul_(grad) passes (torch-ext/flex_sae/hierarchical_kernels.py:92-187,230-270,288-299);
 * kind = FLEXSAE_TOPK replaces embedding_bag_backward with its three kernels and the autograd
 *   backward of the eager tail (torch-ext/flex_sae/topk_kernels.py:71-185,200-210,220-222).
 */
int flexsae_loss_bwd(int kind, const int64_t* indices, const void* weight, const void* vals,
                     const float* state, int segments, const float* grad_out, void* dweight,
                     void* dvals, void* dbias, void* workspace, size_t workspace_bytes, int64_t B,
                     int64_t K, int64_t F, int64_t D, int weight_dtype, int vals_dtype,
                     int bias_dtype, double inv_norm, int dw_mode, int32_t* status, void* stream);

/*
 * Backward of one batch shard with the cross-GPU sum of dweight done inside the same kernel, over
 * NVLink peer memory (2..8 GPUs of one node, one process per GPU, decoder replicated).  Every rank
 * calls it with its own rows and the GLOBAL inv_norm; on return (stream order) dweight holds the sum
 * over all ranks, dvals the local rows' gradient, dbias the LOCAL share (sum it with any collective:
 * it is D values).  The reference has no counterpart (it is single-GPU); in a data-parallel run it
 * replaces flexsae_loss_bwd followed by an all-reduce of the dense [F,D] gradient.
 *   x_ptrs / y_ptrs / flag_ptrs   host arrays of `world` DEVICE pointers, entry r = rank r's
 *       inbox, gather buffer and flag array, each mapped into this process (CUDA IPC / symmetric
 *       memory), of the sizes flexsae_shard_buffer_bytes answers; peers only STORE into them;
 *       the flag buffers (two words per rank: one for its scatters, one for its exchanges) must be
 *       zero before the first call
 *   multicast_x / multicast_y   optional: the multicast (NVLink SHARP) addresses that map onto
 *       all ranks' x / y buffers; when given, the reduction is done by the switch
 *       (multimem.ld_reduce) and the reduced rows are broadcast with multimem.st; NULL, NULL =
 *       plain peer stores
 *   dweight_ptrs   optional: host array of `world` device pointers, entry r = rank r's `dweight`
 *       argument of this same call, mapped into this process (so dweight itself lives in symmetric
 *       / IPC memory; dweight_ptrs[rank] == dweight).  The reduced rows are then stored straight
 *       into every rank's dweight and the gather buffer and its copy pass are skipped.  A peer may
 *       start writing into this rank's dweight as soon as this rank has started the call, so
 *       whatever read the previous contents must precede the call in stream order.  Not with the
 *       multicast path.  NULL = through the gather buffer
 *   seq_base   first call: 1; every later call on the same buffers: previous seq_base +
 *       flexsae_shard_slots(F, D, weight_dtype) (an upper bound of the flag values one call uses);
 *       identical on all ranks.  Before it would pass
 *       INT32_MAX, start again: all ranks idle, flag buffers zeroed, seq_base = 1
 * Only FLEXSAE_DW_ATOMIC accumulation.  All ranks must issue the same sequence of calls.  Waits on
 * other GPUs are bounded; if one gives up, FLEXSAE_STATUS_PIPELINE_TIMEOUT is set in `status` and the
 * gradients of that call are invalid.
 */
int flexsae_shard_buffer_bytes(int64_t F, int64_t D, int weight_dtype, int world, size_t* x_bytes,
                               size_t* y_bytes, size_t* flag_bytes);
int flexsae_shard_slots(int64_t F, int64_t D, int weight_dtype);
int flexsae_loss_bwd_sharded(int kind, const int64_t* indices, const void* weight, const void* vals,
                             const float* state, int segments, const float* grad_out, void* dweight,
                             void* dvals, void* dbias, void* workspace, size_t workspace_bytes,
                             int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                             int vals_dtype, int bias_dtype, double inv_norm, int32_t* status,
                             void* stream, int world, int rank, int seq_base, void* const* x_ptrs,
                             void* const* y_ptrs, void* const* flag_ptrs, void* multicast_x,
                             void* multicast_y, void* const* dweight_ptrs);

/*
 * The step in front of the losses: for each of B rows of encoder activations acts[B,F], the K
 * largest entries as indices[B,K] (int64 decoder rows) and vals[B,K] in descending order of value
 * (equal values: lower index first) -- the layout and order the loss entry points take.  The
 * reference has no counterpart: its losses start from indices and vals (its tests and example draw
 * them at random, tests/test_all_kernels.py:20-33, example.py:45-51) and a caller is left to run
 * torch.topk on the encoder output.  One launch, no scratch memory; each row is read from HBM once
 * (a second pass finds it in L2); the selection is exact and deterministic (a lower bound from 1024
 * running maxima, an unordered candidate list, a total-order sort; a whole-row radix select for rows
 * with masses of equal values).  A NaN counts as larger than every number, as in torch.topk; -0.0
 * and +0.0 are equal (ordered by index, reported as +0.0).  relu != 0 clamps the reported values at
 * zero (a NaN stays a NaN).
 * Needs F a multiple of 8 (16-bit activations) or 4 (fp32), acts 16-byte aligned, K <= min(F, 1024).
 */
int flexsae_topk_select(const void* acts, int acts_dtype, int64_t B, int64_t F, int64_t K, int relu,
                        void* vals, int vals_dtype, int64_t* indices, void* stream);

/*
 * Sum of `n` values (n <= capacity) over the 2..8 GPUs of one node through peer memory, in ONE
 * single-block launch: what the batch-sharded losses use for the scalar loss and for dbias instead
 * of a library all-reduce, whose latency dominates at these sizes.  The reference has no
 * counterpart (it is single-GPU).  Values travel and are added as fp32, in rank order, so every
 * rank receives identical bits; `in` and `out` hold `dtype` elements and may be the same memory.
 *   buf_ptrs   host array of `world` device pointers, entry r = rank r's exchange buffer of
 *       flexsae_small_allreduce_bytes(world, capacity) bytes, mapped into this process, zero before
 *       the first call; peers only store into it
 *   seq        1 on the first call on these buffers, then +1 per call (before INT32_MAX start again:
 *       all ranks idle, buffers zeroed, seq = 1); identical on all ranks, which must issue the same
 *       sequence of calls (each rank: in stream order)
 * The wait for the other ranks is bounded; if it gives up, FLEXSAE_STATUS_PIPELINE_TIMEOUT is set in
 * `status` and `out` is invalid.
 */
int flexsae_small_allreduce_bytes(int world, int64_t capacity, size_t* bytes);
int flexsae_small_allreduce(const void* in, void* out, int64_t n, int dtype, int world, int rank, int seq,
                            void* const* buf_ptrs, int64_t capacity, int32_t* status, void* stream);

/*
 * How unevenly indices[B,K] use the decoder rows.  Takes up to 65536 positions at an odd stride,
 * counts them per decoder row and writes result[0] = the largest count, result[1] = the number of
 * positions taken (device int32[2]).  One launch and two memsets, asynchronous on `stream`; the
 * workspace holds F int32.  When one decoder row takes more than about 1/144 of the positions
 * FLEXSAE_DW_ATOMIC_WIDE is the faster backward, otherwise FLEXSAE_DW_ATOMIC.  Measured at F=65536,
 * D=2304, bf16 (ms per fwd+bwd, L2-sized / wide pieces): uniform indices, share 1/8000: 1.55 / 1.78
 * (B=4096, K=128) and 2.45 / 2.78 (B=16384, K=64); Zipf 0.6, share 1/240: 2.49 / 2.68; Zipf 0.8,
 * share 1/81: 3.30 / 2.92; Zipf 1.1 (config 4), share 1/65, its hottest rows being named by every
 * batch row: 3.71 / 2.98.  The reference has no counterpart: its tile sizes are
 * literals (torch-ext/flex_sae/hierarchical_kernels.py:263-267).
 */
size_t flexsae_index_skew_workspace_bytes(int64_t F);
int flexsae_index_skew(const int64_t* indices, int64_t B, int64_t K, int64_t F, void* workspace,
                       size_t workspace_bytes, int32_t* result, void* stream);

/*
 * The integer part of the deterministic dweight mode on its own: the n = B*K positions (b*K + k) of
 * indices[B,K] grouped by decoder row, in ascending position inside each group -- a stable sort,
 * so the result is one fixed permutation (out-of-range indices count as row 0, as in the losses).
 *   order      [n]    position held by each sorted slot
 *   slot_of    [n]    sorted slot of each position (the inverse permutation)
 *   seg_begin  [F+1]  first slot of each decoder row; seg_begin[F] = n
 *   item_begin [F+1]  first "item" of each decoder row, an item being a run of at most 32 slots of
 *                     one row and every row owning at least one (the unit of the ordered sums)
 * Any of the four outputs may be NULL.  All are int32 device arrays.
 * Replaces count_per_embedding_kernel, the cumsum and map_embeddings_and_outputs_kernel of the
 * reference's TopK backward (torch-ext/flex_sae/topk_kernels.py:71-94,146-163): seg_begin is its
 * emb_begin_pos, order its reverse_mapping -- except that the reference places positions with
 * fetch-add, so its order inside a segment changes from run to run.
 */
size_t flexsae_sort_workspace_bytes(int64_t n, int64_t F);
int flexsae_sort_by_decoder_row(const int64_t* indices, int64_t n, int64_t F, void* workspace,
                                size_t workspace_bytes, int32_t* order, int32_t* slot_of,
                                int32_t* seg_begin, int32_t* item_begin, void* stream);

/*
 * flexsae_loss_fwd for callers that must not allocate device memory.  It has no counterpart in
 * the reference (whose launchers allocate with torch on every call).
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a plug-in whose host
 * application owns every device allocation and hands the plug-in only its inputs and outputs, a
 * process whose memory pool was given out in full at start-up, a latency-critical loop in which
 * the implicit synchronisation of an allocation is not acceptable, or a host callback running on
 * a thread where CUDA allocation calls are not permitted.  Such
 * a caller has nowhere to get the forward's scratch buffer from, so this variant keeps that
 * scratch (the per-(column piece, row) partial losses) in a fixed 1 MiB array that is part of the
 * library image.  Inputs and outputs are still the caller's.
 *
 *  - Limit: column pieces x B <= 262144 partial sums, i.e. flexsae_fwd_workspace_bytes(...) <=
 *    1 MiB (the headline shape needs 9 x 4096 = 36864).  Larger shapes are refused with
 *    FLEXSAE_EUNSUPPORTED and a message that states both sizes.
 *  - Cost: each GPU that loads the library holds the 1 MiB until the process exits.
 *  - The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
 *    that device current, result cached per device ordinal).  Make that first call during set-up,
 *    before any stream capture begins.  The device that is current at the call must be the one
 *    the tensors and the stream belong to.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - All calls on one device share the array, and it keeps whatever the last call left there.
 *    Nothing has to be cleared: the kernel writes every partial before the final sum reads it.
 *    Two calls whose kernels overlap on the same GPU (different streams, no ordering between
 *    them) race on the array and give wrong losses; order them.
 * Arguments and result are those of flexsae_loss_fwd without workspace / workspace_bytes.
 */
int flexsae_loss_fwd_static_scratch(int kind, const int64_t* indices, const void* weight,
                                    const void* vals, const void* bias, const void* target,
                                    float* loss_out, float* state_out, int segments, int64_t B,
                                    int64_t K, int64_t F, int64_t D, int weight_dtype,
                                    int vals_dtype, int bias_dtype, int target_dtype,
                                    double inv_norm, int32_t* status, void* stream);

/* Number of kernels the last flexsae_loss_fwd / flexsae_loss_bwd call of this thread enqueued
 * (for launch accounting in benchmarks). No reference counterpart. */
int flexsae_last_launch_count(void);

#ifdef FLEXSAE_TRACE
/* Tuning builds only (compiled with -DFLEXSAE_TRACE; `python -m flexsae_b200.build --trace` makes
 * libflexsae_b200_trace.so): the sharded backward records, per slot and block role, when the first
 * block started and the last one ended on the GPU's nanosecond timer.  This call synchronises the
 * current device, copies the table of 64 slots x 8 fields to `out` (bytes must be 64*8*8) and clears
 * it when `clear` is non-zero.  `python -m flexsae_b200.slot_timeline` prints it.  The default build
 * has neither the hooks nor this symbol.  No reference counterpart. */
int flexsae_debug_trace_read(unsigned long long* out, size_t bytes, int clear);
#endif

#ifdef __cplusplus
}
#endif
#endif /* FLEXSAE_B200_H */
