/*
 * talu_gaf.h - C ABI of libtalu_gaf.so: grouped-affine (gaf4 / gaf8) quantized
 * matmul for NVIDIA B200 (sm_100a).
 *
 * Drop-in for the matmul operator behind talu's linear layers.  The weight
 * layout is talu's own, unchanged (core/src/converter/grouped_affine.zig:565-593):
 *
 *   packed  u32 [N, K/vpw]  value j of a word at bits [j*bits, (j+1)*bits), vpw = 32/bits
 *   scales  u16 [N, K/G]    bf16 (tag 1) or f16 (tag 0) bit patterns
 *   biases  u16 [N, K/G]
 *   w[n,k] = f32(q[n,k]) * f32(scale[n,k/G]) + f32(bias[n,k/G])
 *   y[m,n] = sum_k x[m,k] * w[n,k]
 *
 * Conventions (the ones talu's own C API follows, core/POLICY.md:96-134):
 *   - every function returns an int32 status, 0 = ok; nothing aborts or throws;
 *   - out-parameters are zeroed before any work;
 *   - tgaf_last_error(ctx) gives the text of the last failure on that context;
 *   - a context is bound to one device and one stream; calls on one context
 *     are not re-entrant (same rule as the reference's per-backend argument
 *     pack, core/src/inference/backend/cuda/engine.zig:4435);
 *   - compute entry points only enqueue work on the context's stream and
 *     return; tgaf_synchronize or the *_host variants wait for it;
 *   - there is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef TALU_GAF_H
#define TALU_GAF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TGAF_ABI_VERSION 1

/* status codes */
#define TGAF_OK 0
#define TGAF_ERR_INVALID_ARGUMENT 1 /* the reference's error.InvalidArgument */
#define TGAF_ERR_CUDA 2
#define TGAF_ERR_OUT_OF_MEMORY 3
#define TGAF_ERR_NCCL 4
#define TGAF_ERR_UNSUPPORTED 5
#define TGAF_ERR_TIMEOUT 6
#define TGAF_ERR_DEVICE_FLAG 7 /* a kernel's bounded wait ran out and set its error word */

/* scales dtype tags: core/src/compute/cuda/gaffine_u4_matvec.zig:13-14 */
#define TGAF_SCALES_F16 0u
#define TGAF_SCALES_BF16 1u

/* how tgaf_weight_upload cuts a weight for tensor parallelism */
#define TGAF_SHARD_NONE 0u
#define TGAF_SHARD_COL 1u /* split N (output features): qkv / gate / up; no collective */
#define TGAF_SHARD_ROW 2u /* split K (input features) on group boundaries: o / down; outputs are partial sums */

/* element types for tgaf_allreduce */
#define TGAF_DTYPE_F32 0u
#define TGAF_DTYPE_BF16 1u

typedef struct tgaf_ctx tgaf_ctx;
typedef struct tgaf_weight tgaf_weight;

int32_t tgaf_abi_version(void);
const char *tgaf_status_string(int32_t status);

/* ---- context ------------------------------------------------------------
 * Replaces the device / registry / launch-stream triple a talu CUDA backend
 * owns (core/src/compute/cuda/device.zig:147-193).  `stream` is a cudaStream_t
 * (CUstream) the caller owns, or NULL for a non-blocking stream the context
 * creates.  The default stream is named by its handle cudaStreamLegacy (0x1)
 * or cudaStreamPerThread (0x2), not by NULL. */
int32_t tgaf_ctx_create(int32_t device_ordinal, void *stream, tgaf_ctx **out_ctx);
int32_t tgaf_ctx_destroy(tgaf_ctx *ctx);
int32_t tgaf_ctx_set_stream(tgaf_ctx *ctx, void *stream);
int32_t tgaf_synchronize(tgaf_ctx *ctx);
const char *tgaf_last_error(const tgaf_ctx *ctx);
/* Tuning knobs by name; unknown names are TGAF_ERR_INVALID_ARGUMENT.
 *   "gemv_ctas"        persistent CTAs of the streaming GEMVs (0 = one per SM; at most one per SM, because the
 *                      CTAs of a launch wait on one another)
 *   "pdl"              programmatic dependent launch between consecutive GEMVs (default 1)
 *   "prefetch_units"   depth of the next-weight L2 prefetch per CTA (default 2, 0 = off)
 *   "force_generic"    shape-agnostic kernel only; "no_dp4a": M <= 4 on the bf16 tensor-core GEMV (A/B aids)
 *   "peer_allreduce", "fused_allreduce", "peer_pdl", "ffn_one_launch": see tgaf_allreduce,
 *                      tgaf_linear_bf16_allreduce, tgaf_ffn_swiglu_bf16
 *   "comm_timeout_ms"  wall-clock limit of tgaf_synchronize while a communicator exists (default 30000,
 *                      0 = wait for ever)
 *   "wait_limit"       polls a kernel of tgaf_allreduce makes for a peer's word before it gives up
 *                      (0 = default, several seconds)
 *   "peer_expect_absent_rank"  diagnostic for the give-up path: tgaf_allreduce's kernel also waits for a
 *                      rank that does not exist, so its bounded wait runs out (tgaf_synchronize then
 *                      returns TGAF_ERR_DEVICE_FLAG and the context stays usable) */
int32_t tgaf_ctx_set_option(tgaf_ctx *ctx, const char *name, int64_t value);

/* ---- weights ------------------------------------------------------------
 * tgaf_weight_upload replaces uploadLinearWeightGroupedAffineU4
 * (core/src/inference/backend/cuda/engine.zig:8209-8273): host pointers in the
 * canonical layout (they may be unaligned mmap views - they are read as bytes),
 * copied to device memory the library owns.  N, K are the FULL (unsharded)
 * sizes; with shard_kind != NONE only this rank's slice is kept:
 *   COL: rows    [rank*N/P, (rank+1)*N/P)             requires N % P == 0
 *   ROW: columns [rank*K/P, (rank+1)*K/P)             requires K % (P*lcm(G, vpw)) == 0
 * Shape rules are the reference's (gaffine_u4_matvec.zig:99-113,
 * engine.zig:8229-8233, models/load/transforms.zig:158-185):
 *   bits in {4,8}; K % vpw == 0; G % vpw == 0; K % G == 0; K/G <= 1024 per rank;
 *   scales dtype in {f16, bf16}. */
int32_t tgaf_weight_upload(tgaf_ctx *ctx, const void *packed, const void *scales,
                           const void *biases, uint64_t N, uint64_t K,
                           uint32_t group_size, uint32_t bits, uint32_t scales_dtype,
                           uint32_t shard_kind, uint32_t tp_rank, uint32_t tp_size,
                           tgaf_weight **out_weight);
/* Same, for the three device buffers a caller already holds (the reference's
 * GaffineU4LinearWeight, engine.zig:220-292).  No copy; the caller keeps
 * ownership and must keep them alive.  No sharding. */
int32_t tgaf_weight_wrap_device(tgaf_ctx *ctx, const void *d_packed, const void *d_scales,
                                const void *d_biases, uint64_t N, uint64_t K,
                                uint32_t group_size, uint32_t bits, uint32_t scales_dtype,
                                tgaf_weight **out_weight);
int32_t tgaf_weight_free(tgaf_ctx *ctx, tgaf_weight *w);
/* local (per-rank) sizes of a weight */
int32_t tgaf_weight_dims(const tgaf_weight *w, uint64_t *n_local, uint64_t *k_local,
                         uint32_t *group_size, uint32_t *bits);

/* Names the weight that the NEXT tgaf_linear_* call after the coming one will
 * stream, i.e. call order: hint(B); linear(A); linear(B).  While A's kernel
 * drains, its copy warps ask L2 for the first tiles of B, so HBM keeps streaming
 * across A's write-out, the launch gap and B's prologue.  One-shot: consumed (or
 * dropped) by the first linear call that follows; NULL clears it.  Results never
 * depend on it.  `next` must stay alive until that call has run on the GPU.
 * "prefetch_units" (tgaf_ctx_set_option) bounds how much of B is requested.
 * No counterpart in the reference, whose decoder issues each linear on its own
 * (core/src/inference/backend/cuda/engine.zig:4431-4474). */
int32_t tgaf_hint_next_weight(tgaf_ctx *ctx, const tgaf_weight *next);

/* ---- the matmul operator ------------------------------------------------
 * Replaces the .gaffine_u4 arm of CudaBackend.linearForwardRows
 * (engine.zig:4431-4474) and, on the CPU side, MatmulFn for
 * grouped_affine_u4 / u8 (core/src/compute/cpu/matmul_primitives.zig:101-121,
 * :947-974, :1037-1063).
 *   x: [M, K_local] row-major, y: [M, N_local] row-major, device pointers.
 * bf16 variant: bf16 in, fp32 accumulate, bf16 out (round to nearest even).
 * f32 variant: the reference's f32-in / f32-out contract. */
int32_t tgaf_linear_bf16(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16,
                         uint32_t M, void *y_bf16);
int32_t tgaf_linear_f32(tgaf_ctx *ctx, const tgaf_weight *w, const float *x,
                        uint32_t M, float *y);
/* Linear.forward with its optional bias (core/src/inference/backend/cpu/executor/model.zig:98-139): the matmul,
 * then y[m, n] += bias[n] (addBiasRows).  d_bias: f32 [N_local] on the device, or NULL for none.  The bias is
 * added to this rank's output as it is: for a row-parallel weight add it on one rank only, or after the sum. */
int32_t tgaf_linear_bf16_bias(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16, uint32_t M,
                              const float *d_bias, void *y_bf16);
int32_t tgaf_linear_f32_bias(tgaf_ctx *ctx, const tgaf_weight *w, const float *x, uint32_t M,
                             const float *d_bias, float *y);
/* No counterpart in the reference.  tgaf_linear_bf16 for hosts that must not allocate
 * while they serve: a backend that gives the rest of the device's memory to its KV cache
 * at start-up cannot afford a cudaMalloc in the token loop (it synchronises the device
 * and may fail).  This call allocates nothing - no cudaMalloc / cudaFree, no growth of
 * the context's scratch: the kernel's split-K scratch is a fixed 8 MiB (+ 8192 counters)
 * device array inside the library image, present on every GPU that loads the library
 * until the process exits.  x, y and the weight are the caller's, as in tgaf_linear_bf16.
 *   - A problem that needs more scratch than that (very many output rows at M > 8) is
 *     rejected with TGAF_ERR_UNSUPPORTED and a message; nothing is launched.
 *   - The first call on a device looks the array's device address up; make that call
 *     before any stream capture, and not from two host threads at once.
 *   - All calls on a device share the array: calls that overlap on the GPU (two streams)
 *     race.  The counters are cleared on the stream before each launch. */
int32_t tgaf_linear_bf16_fixed_scratch(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16,
                                       uint32_t M, void *y_bf16);

/* Host-buffer variants: copy x to the device, run, copy y back, wait. */
int32_t tgaf_linear_bf16_host(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16_host,
                              uint32_t M, void *y_bf16_host);
int32_t tgaf_linear_f32_host(tgaf_ctx *ctx, const tgaf_weight *w, const float *x_host,
                             uint32_t M, float *y_host);
/* The same without the wait: the call returns once everything is enqueued.  Several calls may be queued back
 * to back; the copies run on the context's own copy streams around the kernels (a ring of four staging
 * buffers, ordered by events), so x of the next call and y of the previous one travel while a kernel runs.
 * y_host is valid, and x_host may be changed, after tgaf_synchronize.  Use page-locked host memory, or the
 * copies are not asynchronous.  Do not capture these calls into a CUDA graph. */
int32_t tgaf_linear_bf16_host_async(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16_host,
                                    uint32_t M, void *y_bf16_host);
/* `count` such calls in list order with one crossing of the ABI (the list is the layer order, so each launch
 * is also given the following weight as its next-weight hint).  Stops at the first error. */
int32_t tgaf_linear_bf16_host_async_batch(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights,
                                          const void *const *xs_bf16_host, const uint32_t *ms,
                                          void *const *ys_bf16_host);
/* The same list recorded once (it is run once, then captured into a CUDA graph of its copies and kernels) and
 * replayed with one call per step - the form a decoder with fixed page-locked I/O buffers wants: refill the x
 * buffers, tgaf_host_batch_submit, tgaf_synchronize, read the y buffers.  The buffers, the weights and the
 * context must outlive the batch; nothing else may be queued with tgaf_linear_bf16_host_async while a batch is
 * in flight (they share the staging ring). */
typedef struct tgaf_host_batch tgaf_host_batch;
int32_t tgaf_host_batch_create(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights,
                               const void *const *xs_bf16_host, const uint32_t *ms, void *const *ys_bf16_host,
                               tgaf_host_batch **out_batch);
/* The same with reduce[i] = 1 marking row-parallel weights whose y_i is summed over the communicator's ranks
 * before it travels back (every rank records and submits the same list; all ms equal).  reduce == NULL: as above.
 * Either call records the STAGED form when all ms are equal and the list can run as one launch (see launch
 * lists below) or has a sum over the ranks: the x buffers go up into one device block, one launch list runs, the
 * y block comes down; host buffers that lie back to back in memory travel as one copy, so a caller that keeps
 * its activations (and its outputs) in one page-locked block pays two copies per step. */
int32_t tgaf_host_batch_create_reduce(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights,
                                      const void *const *xs_bf16_host, const uint32_t *ms, void *const *ys_bf16_host,
                                      const uint8_t *reduce, tgaf_host_batch **out_batch);
/* 1 when the recorded list is the staged form around ONE kernel launch */
int32_t tgaf_host_batch_uses_one_launch(const tgaf_host_batch *batch);
int32_t tgaf_host_batch_submit(tgaf_ctx *ctx, tgaf_host_batch *batch);
int32_t tgaf_host_batch_destroy(tgaf_ctx *ctx, tgaf_host_batch *batch);

/* ---- launch lists ---------------------------------------------------------
 * The linears of a decoder step as ONE call: `count` operations y_i = x_i * W_i^T, bf16 device buffers, all with
 * the same m.  No counterpart in the reference, whose decoder issues each linear on its own
 * (core/src/inference/backend/cuda/engine.zig:4431-4474); it is the device-buffer sibling of tgaf_host_batch.
 * When every weight is gaf4 with one group size and scales dtype and m <= 8 (m <= 4 for groups of 32 codes, for lists
 * with sums over the ranks or with dependent operations, and for lists with small weights: above four rows every
 * operation must give each CTA four units of 128 rows x 512 codes), or every weight is gaf8_32 / gaf8_64 of one scheme and
 * m <= 4, the whole list runs as ONE kernel
 * launch: the copy warps stream from one weight straight into the next, so launch gap, ring ramp-up / drain and
 * write-out tail are paid once per list instead of once per weight; otherwise the calls run one after the other.
 * Weights of any sizes may share a list (up to four rows the launch is sized for the largest; the unit ranges are dealt
 * so that over the whole list every CTA streams the same number of units to within one).
 *   depends[i] = 1: x_i is written by an earlier operation of the list (as down after gate|up): operation i starts
 *                   on its activations only when operation i - 1 is complete on the whole GPU.  0 (or depends ==
 *                   NULL): the caller promises that x_i is written by no operation of this list.
 *   reduce[i]  = 1: W_i is row-parallel; y_i is summed over the communicator's ranks (inside the launch when the
 *                   peer-memory path is up, see tgaf_linear_bf16_allreduce).  NULL: none.
 * The buffers, the weights and the context must outlive the batch.  tgaf_batch_run only enqueues (it may be
 * captured into a CUDA graph after one eager run). */
typedef struct tgaf_batch tgaf_batch;
int32_t tgaf_batch_create(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights, const void *const *xs_bf16,
                          uint32_t m, void *const *ys_bf16, const uint8_t *depends, const uint8_t *reduce,
                          tgaf_batch **out_batch);
int32_t tgaf_batch_run(tgaf_ctx *ctx, tgaf_batch *batch);
/* 1 when the list runs as one kernel launch, 0 when its calls run one after the other */
int32_t tgaf_batch_uses_one_launch(const tgaf_batch *batch);
int32_t tgaf_batch_destroy(tgaf_ctx *ctx, tgaf_batch *batch);

/* Raw-pointer launch with the argument list of the reference's kernel wrapper
 * compute.cuda.gaffine_u4_matvec.runWithFunction
 * (core/src/compute/cuda/gaffine_u4_matvec.zig:58-97; kernel
 * core/src/compute/cuda/kernels/ops/quant_ops.cu:46-57): f32 activations
 * [batch_rows, in_dim], f32 out [batch_rows, out_dim], all device pointers.
 * Validation = the wrapper's validateArgs (:99-113). */
int32_t tgaf_gaffine_u4_matvec_f32(tgaf_ctx *ctx, const float *input, const uint32_t *packed_weight,
                                   const uint16_t *scales, const uint16_t *biases, float *out,
                                   uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                   uint32_t scales_dtype_tag, uint32_t batch_rows);
/* 8-bit counterpart (the reference has no gaf8 CUDA kernel: it dequantizes gaf8
 * to f32 on the host and calls cuBLAS, engine.zig:8106-8125). */
int32_t tgaf_gaffine_u8_matvec_f32(tgaf_ctx *ctx, const float *input, const uint32_t *packed_weight,
                                   const uint16_t *scales, const uint16_t *biases, float *out,
                                   uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                   uint32_t scales_dtype_tag, uint32_t batch_rows);

/* ---- dequant --------------------------------------------------------------
 * Replaces decodeGroupedAffineU4Row / U8Row (core/src/compute/cpu/quant_decode.zig:64-130)
 * and convertToF32 (core/src/models/load/transforms.zig:651-714): out f32
 * [N_local, K_local], bit-exact fmaf(q, scale, bias). */
int32_t tgaf_dequant_f32(tgaf_ctx *ctx, const tgaf_weight *w, float *d_out);
int32_t tgaf_dequant_f32_host(tgaf_ctx *ctx, const tgaf_weight *w, float *h_out);

/* Embedding rows: out f32 [count, K_local], row i = dequant(weight row token_ids[i]) * multiplier.
 * Replaces talu_embedding_lookup_gaffine_u4_f32 (core/src/compute/cuda/kernels/ops/quant_ops.cu:12-44,
 * one token per launch there) and gatherDecodeGroupedAffineU4Rows / U8Rows
 * (core/src/compute/cpu/quant_decode.zig:133-210).  token_ids is a HOST array, checked before anything
 * is enqueued: an id >= N is TGAF_ERR_INVALID_ARGUMENT (the reference's error.InvalidTokenId). */
int32_t tgaf_embedding_lookup_f32(tgaf_ctx *ctx, const tgaf_weight *w, const uint32_t *token_ids,
                                  uint32_t count, float multiplier, float *d_out);

/* ---- the SwiGLU FFN as one operator ---------------------------------------
 * y[m, d_model] = down( silu(gate(x)) * up(x) ), the body of SwiGLU.forward
 * (core/src/inference/backend/cpu/kernels/ffn.zig:103-400) with the reference's fused gate|up weight
 * in its concat layout (rows [gate..., up...], ffn.zig:228-241); on the reference's CUDA backend this is
 * tryFusedGateUpForward + a silu-mul kernel + the down matvec
 * (core/src/inference/backend/cuda/engine.zig:4476-4553, kernels/ops/quant_ops.cu:221-286).
 * w_gate_up: [2 * d_ff, d_model], w_down: [d_model, d_ff].  bf16 in, bf16 out.
 * For M = 1 on gaf4 weights of one group size BOTH linears run in ONE kernel: the copy warp streams
 * straight on from the first weight into the second, the intermediate stays fp32, and the activation is
 * applied while the second linear quantises its operand; otherwise: linear, silu-mul kernel, linear.
 * Option "ffn_one_launch" = 0 forces the latter. */
int32_t tgaf_ffn_swiglu_bf16(tgaf_ctx *ctx, const tgaf_weight *w_gate_up, const tgaf_weight *w_down,
                             const void *x_bf16, uint32_t m, void *y_bf16);
/* The same with the gate's activation chosen by the caller, as SwiGLU.forward does with use_gelu
 * (ffn.zig:213-266): TGAF_ACT_SILU = silu(g) * u (talu_silu_mul_f32,
 * core/src/compute/cuda/kernels/ops/reduction_ops.cu:46-57), TGAF_ACT_GELU = tanh-form gelu(g) * u
 * (talu_gelu_mul_f32, reduction_ops.cu:59-72). */
#define TGAF_ACT_SILU 1u
#define TGAF_ACT_GELU 2u
int32_t tgaf_ffn_gated_bf16(tgaf_ctx *ctx, const tgaf_weight *w_gate_up, const tgaf_weight *w_down,
                            const void *x_bf16, uint32_t m, uint32_t activation, void *y_bf16);

/* ---- tensor parallel exchange (no counterpart in the reference, which is
 * single-device): sum of the row-parallel partial outputs over all ranks. ----
 * The communicator belongs to the context.  Rank 0 makes the id and the host
 * program hands its bytes to the other ranks by any means it has. */
#define TGAF_COMM_ID_BYTES 128
int32_t tgaf_comm_make_id(uint8_t id[TGAF_COMM_ID_BYTES]);
int32_t tgaf_comm_init(tgaf_ctx *ctx, const uint8_t id[TGAF_COMM_ID_BYTES], uint32_t rank, uint32_t nranks);
/* Waits for the context's stream, then destroys the communicator.  Release every CUDA graph
 * that captured tgaf_allreduce first: NCCL waits for them.  tgaf_ctx_destroy aborts a
 * communicator that is still there instead of waiting. */
int32_t tgaf_comm_destroy(tgaf_ctx *ctx);
/* In place, on the context's stream.  Tiles of up to 131072 values (decode: [M <= 16, 8192]) are
 * summed by one kernel over NVLink peer memory when every rank of the communicator could map every
 * other rank's exchange region (same node, CUDA IPC): each rank pushes its tile, widened to fp32, to
 * all peers, then adds the ranks' tiles in rank order - the result is bit-identical on every rank
 * and from run to run, with one rounding for bf16.  Anything else goes to ncclAllReduce.  All
 * ranks must issue the same sequence of calls.  A peer that does not show up within several
 * seconds makes the kernel give up: tgaf_synchronize then returns TGAF_ERR_DEVICE_FLAG.
 * Option "peer_allreduce" = 0 (tgaf_ctx_set_option, same value on every rank) or the environment
 * variable TGAF_PEER_ALLREDUCE=0 keeps everything on NCCL. */
int32_t tgaf_allreduce(tgaf_ctx *ctx, void *d_buf, uint64_t count, uint32_t dtype);
/* y = sum over ranks of x_local * W_local^T for a row-parallel weight (TGAF_SHARD_ROW): tgaf_linear_bf16
 * followed by tgaf_allreduce on y, as one call.  For M <= 4 on gaf4 weights with the peer-memory path
 * available it is ONE kernel: the GEMV's write-out pushes each finished block of 128 outputs, as fp32, to
 * every rank over NVLink while later blocks are still being computed, then adds the ranks' blocks in rank
 * order and rounds once (bit-identical on all ranks; more accurate than summing rounded bf16 outputs).
 * Everything else runs the two steps one after the other.  Option "fused_allreduce" = 0 forces that. */
int32_t tgaf_linear_bf16_allreduce(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16, uint32_t m, void *y_bf16);
/* tgaf_ffn_swiglu_bf16 with a column-parallel gate|up (each rank holds matching gate and up rows) and a
 * row-parallel down whose partial sums are added over the ranks (inside the kernel when it can). */
int32_t tgaf_ffn_swiglu_bf16_allreduce(tgaf_ctx *ctx, const tgaf_weight *w_gate_up, const tgaf_weight *w_down,
                                       const void *x_bf16, uint32_t m, void *y_bf16);
/* 1 when the peer-memory path of tgaf_allreduce is available on this communicator, else 0 */
int32_t tgaf_comm_uses_peer_memory(const tgaf_ctx *ctx);

/* ---- failure handling on the host ------------------------------------------
 * The reference's model is typed driver errors returned to the caller
 * (core/src/compute/cuda/device.zig:226-237); it has no collectives.  Here a stream can hold a collective
 * that never completes because a rank is missing or has failed.  While a context has a communicator,
 * tgaf_synchronize therefore does not block: it polls the stream and the collective library's asynchronous
 * error state (ncclCommGetAsyncError) under a wall-clock limit (option "comm_timeout_ms"); on an error
 * (TGAF_ERR_NCCL) or at the limit (TGAF_ERR_TIMEOUT) it aborts the communicator (ncclCommAbort), drops the
 * peer mappings and returns; single-GPU calls on the context keep working, tgaf_comm_init makes a new
 * communicator.  tgaf_watchdog_wait is that loop with its three hooks in the caller's hands, for hosts that
 * run their own collectives next to this library (and for tests without a GPU):
 *   work_done(user)   > 0 finished, 0 still running, < 0 failed (-> TGAF_ERR_CUDA)
 *   async_error(user) 0 = none, anything else -> abort_comm(user), TGAF_ERR_NCCL        (may be NULL)
 *   abort_comm(user)  called once before TGAF_ERR_NCCL / TGAF_ERR_TIMEOUT is returned   (may be NULL)
 * timeout_ms = 0 waits for ever. */
typedef struct tgaf_watch_fns {
    int32_t (*work_done)(void *user);
    int32_t (*async_error)(void *user);
    void (*abort_comm)(void *user);
} tgaf_watch_fns;
int32_t tgaf_watchdog_wait(const tgaf_watch_fns *fns, void *user, uint32_t timeout_ms);

#ifdef __cplusplus
}
#endif
#endif /* TALU_GAF_H */
