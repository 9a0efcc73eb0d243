/* C ABI of the B200 (sm_100a) Qwen4 mixture-of-experts layer.
 *
 * libqwen4_moe_b200.so exports two groups of symbols:
 *
 *  1. The entry points of picoforge's MoE operator (picoforge src/qwen4_moe.h:13-27 and
 *     the two private helpers its tests and GPU glue link, src/qwen4_moe_internal.h:15,94),
 *     byte-compatible: same names, same by-value view structs, same status codes, same
 *     "outputs untouched on error" behaviour.  picoforge's forward graph
 *     (src/qwen4_forward.c:174-187, :365) links against them unchanged.
 *
 *  2. Additive `qw4cu_*` entry points that the reference does not have: device-pointer
 *     forward (inputs already in HBM), bit-exact weight decode and grouping probes for
 *     parity tests, and timing / memory plumbing for the benchmark.
 *
 * Plain C11; no CUDA or C++ types cross this boundary.  All strides and capacities are
 * BYTES, all dimensions are element counts, the last axis is contiguous.
 */
#ifndef QWEN4_MOE_B200_H
#define QWEN4_MOE_B200_H
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------
 * Types shared with the engine.  Layouts follow picoforge src/qwen4_types.h:14-46,75-80,
 * src/qwen4_packed.h:6-11 and src/qwen4_moe.h:7-11.  When this header is included after
 * picoforge's own headers, define QWEN4_MOE_B200_NO_TYPES to skip them.
 * ---------------------------------------------------------------------------------- */
#ifndef QWEN4_MOE_B200_NO_TYPES
#define QWEN4_MAX_RANK 4u

typedef enum {
    QW4_OK = 0,
    QW4_INVALID_ARGUMENT = 1,
    QW4_MISSING = 2,
    QW4_TYPE = 3,
    QW4_RANGE = 4,
    QW4_SHAPE = 5,
    QW4_STRIDE = 6,
    QW4_FORMAT = 7,
    QW4_UNSUPPORTED = 8,
    QW4_OVERFLOW = 9,
    QW4_CAPACITY = 10,
    QW4_OOM = 11,
    QW4_OWNER = 12,
    QW4_BUSY = 13,
    QW4_STALE = 14,
    QW4_BAD_STATE = 15,
    QW4_NONFINITE = 16,
    QW4_IO = 17,
    QW4_EOF = 18,
    QW4_CANCELLED = 19,
    QW4_GPU_ERROR = 20
} Qwen4Status;

typedef struct {
    Qwen4Status code;
    int os_errno;
    uint64_t file_offset;
    uint64_t row;                 /* token row of a nonfinite router logit */
    size_t requested_bytes;
    size_t completed_bytes;
    char subject[128];
    char detail[256];
} Qwen4Error;

typedef struct {
    const unsigned char *data;
    size_t bytes;
} Qwen4CpuSpan;

/* Read-only and mutable FP32 views of rank <= 4. */
typedef struct {
    const float *data;
    size_t capacity_bytes;
    size_t rank;
    size_t dim[QWEN4_MAX_RANK];
    size_t stride_bytes[QWEN4_MAX_RANK];
} Qwen4F32;

typedef struct {
    float *data;
    size_t capacity_bytes;
    size_t rank;
    size_t dim[QWEN4_MAX_RANK];
    size_t stride_bytes[QWEN4_MAX_RANK];
} Qwen4F32Mut;

typedef struct {
    uint32_t *data;
    size_t capacity_bytes;
    size_t rows;
    size_t cols;
    size_t row_stride_bytes;
} Qwen4U32Mut;

typedef struct {
    uint32_t hidden_size;
    uint32_t experts;
    uint32_t top_k;
    uint32_t intermediate;
    uint32_t shared_intermediate;
    uint32_t down_physical;       /* stored K of the routed down projection, >= intermediate */
    bool norm_topk_prob;
    uint32_t trunk_type[3];
} Qwen4MoeConfig;

/* One weight tensor [expert][row][packed K], K contiguous.  gguf_type is the GGUF tensor
 * type id: 0 F32, 1 F16, 8 Q8_0, 10 Q2_K, 12 Q4_K, 16 IQ2_XXS, 30 BF16, 39 MXFP4. */
typedef struct {
    uint32_t gguf_type;
    size_t k_storage;
    size_t k_logical;
    size_t n_out;
    size_t n_experts;
    size_t row_bytes;
    size_t expert_bytes;
    size_t tensor_bytes;
} QW4PackedLayout;

typedef struct {
    Qwen4CpuSpan span;
    QW4PackedLayout layout;
} QW4PackedCpuView;

typedef struct Qwen4Moe Qwen4Moe;
typedef struct Qwen4MoeWork Qwen4MoeWork;

typedef struct {
    QW4PackedCpuView router;
    QW4PackedCpuView gate;
    QW4PackedCpuView up;
    QW4PackedCpuView down;
    QW4PackedCpuView shared_gate;
    QW4PackedCpuView shared_up;
    QW4PackedCpuView shared_down;
    QW4PackedCpuView shared_router;
} Qwen4MoeWeights;

typedef struct {
    Qwen4U32Mut ids;
    Qwen4F32Mut weights;
} Qwen4MoeRoutes;

typedef void (*QW4MoeObserver)(void *ctx, size_t stage, size_t expert, size_t token,
                               Qwen4F32 input, Qwen4F32 output);

typedef struct {
    size_t *offsets;              /* [experts + 1] */
    size_t offsets_capacity_bytes;
    size_t *cursors;              /* [experts], scratch; ends equal to offsets[e + 1] */
    size_t cursors_capacity_bytes;
    size_t *pair_to_row;          /* [T * K] */
    size_t *row_to_pair;          /* [T * K] */
    size_t pair_to_row_capacity_bytes;
    size_t row_to_pair_capacity_bytes;
} QW4MoeGrouping;
#endif /* QWEN4_MOE_B200_NO_TYPES */

/* ------------------------------------------------------------------------------------
 * Group 1: the reference operator's entry points.
 * ---------------------------------------------------------------------------------- */

/* Replaces qwen4_moe_create (picoforge src/qwen4_moe.h:13-14, src/qwen4_moe.c:47-74).
 * Validates the eight layouts against the config with the reference's status codes, then
 * UPLOADS every weight tensor into HBM (all experts resident; no SSD pool).  The host
 * bytes are read during this call only: later changes to them are not seen by forward. */
Qwen4Status qwen4_moe_create(const Qwen4MoeConfig *config, const Qwen4MoeWeights *weights,
                             Qwen4Moe **out, Qwen4Error *err);

/* Replaces qwen4_moe_destroy (src/qwen4_moe.h:15, src/qwen4_moe.c:76).  Workspaces keep
 * the device image alive until the last of them is destroyed. */
void qwen4_moe_destroy(Qwen4Moe *moe);

/* Replaces qwen4_moe_work_size (src/qwen4_moe.h:16-17, src/qwen4_moe.c:106-111).
 * Reports the HOST bytes of a workspace (metadata plus pinned staging for routes); the
 * device scratch it also owns is reported by qw4cu_moe_work_device_bytes. */
Qwen4Status qwen4_moe_work_size(const Qwen4Moe *moe, size_t token_cap, size_t *bytes,
                                Qwen4Error *err);

/* Replaces qwen4_moe_work_create (src/qwen4_moe.h:18-19, src/qwen4_moe.c:112-124). */
Qwen4Status qwen4_moe_work_create(const Qwen4Moe *moe, size_t token_cap, size_t byte_budget,
                                  Qwen4MoeWork **out, Qwen4Error *err);

/* Replaces qwen4_moe_work_reset (src/qwen4_moe.h:20, src/qwen4_moe.c:125-130): clears the
 * failure latch set by a forward that returned an error. */
Qwen4Status qwen4_moe_work_reset(Qwen4MoeWork *work, Qwen4Error *err);

/* Replaces qwen4_moe_work_destroy (src/qwen4_moe.h:21, src/qwen4_moe.c:131-133). */
void qwen4_moe_work_destroy(Qwen4MoeWork *work);

/* Replaces qwen4_moe_route (src/qwen4_moe.h:24-25, src/qwen4_moe.c:188-249): softmax over
 * experts, top-k with ties to the lower id, optional renormalisation.  Host views in and
 * out; the arithmetic runs on the GPU in the reference's order (serial exp-sum). */
Qwen4Status qwen4_moe_route(const Qwen4MoeConfig *config, Qwen4F32 logits,
                            Qwen4MoeRoutes routes, Qwen4F32Mut probabilities, Qwen4Error *err);

/* Replaces qwen4_moe_forward (src/qwen4_moe.h:26-27, src/qwen4_moe.c:384-431).  x and y are
 * HOST views; the call copies x to HBM, runs the layer, copies y (and routes) back and is
 * synchronous.  y is written only when the status is QW4_OK. */
Qwen4Status qwen4_moe_forward(const Qwen4Moe *moe, Qwen4F32 x, Qwen4F32Mut y,
                              Qwen4MoeRoutes *optional_routes, Qwen4MoeWork *work,
                              Qwen4Error *err);

/* Replaces qw4_moe_group_pairs (src/qwen4_moe_internal.h:78-95, src/qwen4_moe.c:251-303):
 * stable counting sort of (token, slot) pairs by expert, computed by the dispatch kernels. */
Qwen4Status qw4_moe_group_pairs(const Qwen4MoeConfig *config, Qwen4U32Mut ids,
                                QW4MoeGrouping grouping, Qwen4Error *err);

/* Replaces qw4_moe_observe (src/qwen4_moe_internal.h:9-15, src/qwen4_moe.c:134-136).  While an
 * observer is set, qwen4_moe_forward runs the layer stage by stage in the reference's order (32-token
 * microbatches, one plain kernel per stage, sums in ascending k) instead of the fused kernels, and
 * reports every stage the reference reports, with its stage / expert / token arguments: projections
 * 0-7, 8 SiLU, 9 product, 10 sigmoid, 11 routed sum, 12 y.  A diagnostic path: slow by design. */
void qw4_moe_observe(Qwen4MoeWork *work, QW4MoeObserver observer, void *ctx);

/* ------------------------------------------------------------------------------------
 * Group 2: additions (no counterpart in the reference).
 * ---------------------------------------------------------------------------------- */

/* Number of CUDA devices, or -1 when the runtime cannot be initialised. */
int qw4cu_device_count(void);
/* Selects the device used by every later call on this thread.  Returns 0 on success. */
int qw4cu_set_device(int device);
/* Text of the last CUDA error seen by this library on this thread ("" if none). */
const char *qw4cu_last_error(void);

/* Router arithmetic.  0 "exact": logits summed serially over k without FMA, bit-identical
 * to the reference CPU path (ids always match).  1 "fast": warp-tree sums; ids can differ
 * only where two probabilities are within rounding of each other.  Default 0.  The
 * environment variable QW4CU_ROUTER=exact|fast sets the initial value. */
void qw4cu_set_router_mode(int mode);
int qw4cu_get_router_mode(void);

/* Device bytes held by the resident weight image of one MoE, and by one workspace. */
size_t qw4cu_moe_device_bytes(const Qwen4Moe *moe);
size_t qw4cu_moe_work_device_bytes(const Qwen4MoeWork *work);

/* Forward on device pointers: x_dev [tokens, hidden] and y_dev [tokens, hidden] are dense
 * FP32 in HBM; ids_dev [tokens, k] and weights_dev [tokens, k] may be NULL.  Enqueues on
 * the library's stream (one per device, shared by all workspaces) and returns without waiting; errors found by the kernels are
 * reported by qw4cu_moe_work_sync. */
Qwen4Status qw4cu_moe_forward_device(const Qwen4Moe *moe, const float *x_dev, float *y_dev,
                                     size_t tokens, uint32_t *ids_dev, float *weights_dev,
                                     Qwen4MoeWork *work, Qwen4Error *err);

/* The same forward followed by the hyper-connection add of its caller, inside the kernel that writes y:
 *     residual_dev[t, h, c] += inject_dev[t, h] * y[t, c]        for h < streams
 * with the product and the sum rounded separately (picoforge src/qwen4_base.c:160-176; its forward graph calls
 * qwen4_hc_add right after the layer, src/qwen4_forward.c:365-367, and its GPU path fuses the add into the down
 * epilogue, src/qwen4_moe_internal.h:55-58).  residual_dev [tokens, streams, hidden] and inject_dev
 * [tokens, streams] are dense FP32 in HBM and must not overlap x, y or each other; y_dev is written as usual.
 * tokens <= 2048.  A nonfinite residual is reported like a nonfinite y, by qw4cu_moe_work_sync.  The one-kernel
 * decode path and the tensor-core paths apply the add where they write y; the CUDA-core fallback kernels run it
 * as one more launch. */
Qwen4Status qw4cu_moe_forward_hc_add_device(const Qwen4Moe *moe, const float *x_dev, float *y_dev, size_t tokens,
                                            float *residual_dev, const float *inject_dev, size_t streams,
                                            Qwen4MoeWork *work, Qwen4Error *err);
/* Waits for the workspace's stream, converts the device error word (bit 1 nonfinite, bit 2
 * bounds, bit 4 state) into a status and latches the workspace on failure. */
Qwen4Status qw4cu_moe_work_sync(Qwen4MoeWork *work, Qwen4Error *err);
/* The same for n workspaces on the stream in force (e.g. the layers of a stack enqueued back to back): all status
 * words are fetched, then one wait; the first failing workspace's status is returned, every failing one is latched. */
Qwen4Status qw4cu_moe_work_sync_many(Qwen4MoeWork *const *works, size_t n, Qwen4Error *err);

/* Expert parallelism (no counterpart in the reference, which is a single-device engine).
 * Experts are cut into equal contiguous blocks, one per rank; the router and the shared expert
 * are replicated; tokens are data-parallel, the same number on every rank.  A sharded handle
 * holds experts [first_expert, first_expert + local_experts): weights->gate/up/down carry
 * local_experts experts, the router and the shared expert are complete.
 *
 * One layer step moves one exchange row per TOKEN (qw4cu_ep_row_floats(moe) floats: the token's
 * activations, its k route ids, its k route weights) to every rank with an all-gather, lets every
 * rank run its own experts on the tokens routed to them and form per-token partial sums (its
 * experts' weighted outputs, plus the sigmoid-gated shared expert for its own tokens), and ends
 * with a reduce-scatter (sum) that hands every rank the finished rows of its own tokens.  The sum
 * over a token's experts therefore runs per rank and then over ranks, not in slot order: y agrees
 * with the one-device layer within the layer tolerance, ids and route weights bit for bit.
 *
 * qw4cu_moe_ep_forward_device does the whole step, both exchanges included.  A C host makes the
 * communicator itself: rank 0 calls qw4cu_ep_unique_id and hands the 128 bytes to the other ranks by
 * any means, then every rank calls qw4cu_ep_create with its device current (world 1 needs no NCCL and
 * no id).  NCCL is taken from the process at run time (libnccl.so.2, or the file named by
 * QW4CU_NCCL_LIBRARY).  Transport of the two exchanges (qw4cu_ep_transport: 1 peer memory, 0 NCCL):
 * by default this library's own kernels over NVLink peer memory: the ranks map each other's exchange
 * buffers (CUDA IPC handles, handed round through the communicator when the buffers are made), the
 * all-gather is a push of the rank's rows into every rank's buffer with plain peer stores, the
 * reduce-scatter a pull of the own tokens' partial rows from every rank, added in rank order; ranks meet
 * at epoch words that they raise in each other's memory, every wait is bounded (about eight seconds, then
 * QW4_GPU_ERROR "device state error" at the next qw4cu_moe_work_sync).  NCCL's ncclAllGather /
 * ncclReduceScatter carry the exchanges when a mapping fails on any rank or QW4CU_EP_TRANSPORT=nccl.
 * The workspace must have capacity for (world + 1) * tokens_local tokens.  Every rank must make the same
 * sequence of calls with the same token count, qw4cu_ep_destroy included (with the peer transport it waits
 * for the other ranks, so that no buffer goes away under a peer that still reads it); all calls enqueue on
 * the stream in force and return without waiting (the exchange buffers are made on the first call of a
 * size, a collective step with host synchronisation: make that call outside any stream capture).
 *
 * The two compute pieces are also callable on their own, for a caller with an exchange of its
 * own (or one process that plays several ranks):
 *   begin    routes x [tokens_local, hidden], writes this rank's exchange rows to rows_local_dev
 *            [tokens_local, row floats] (and ids / weights [tokens_local, k] if not NULL) and starts
 *            the shared expert of these tokens on a second stream;
 *   experts  rows_all_dev: the rows of all ranks in rank order [tokens_total, row floats]; own_first:
 *            index of this rank's first token in it; partial_dev [tokens_total, hidden] receives the
 *            partial sums.  y of a token = sum over ranks of its partial rows. */
typedef struct QW4CuEp QW4CuEp;
Qwen4Status qw4cu_moe_create_sharded(const Qwen4MoeConfig *config, const Qwen4MoeWeights *weights,
                                     uint32_t first_expert, uint32_t local_experts, Qwen4Moe **out,
                                     Qwen4Error *err);
int qw4cu_ep_unique_id(unsigned char id[128]);
Qwen4Status qw4cu_ep_create(const unsigned char id[128], int rank, int world, QW4CuEp **out, Qwen4Error *err);
void qw4cu_ep_destroy(QW4CuEp *ep);
int qw4cu_ep_transport(const QW4CuEp *ep);
/* Test aid for the bounded waits of the peer transport: runs the wait kernel as rank 0 of two on a flag row that
 * nothing raises (raise_first = 0) or that the "peer" has already raised (1), with a limit of `polls` polls (capped
 * at 65536, about a tenth of a second).  Returns 1 when the wait ran out and recorded the state error, 0 when it
 * was satisfied, -1 on a CUDA error.  Needs no second GPU and leaves the context usable. */
int qw4cu_ep_wait_probe(uint32_t polls, int raise_first);
size_t qw4cu_ep_row_floats(const Qwen4Moe *moe);
Qwen4Status qw4cu_moe_ep_forward_device(const Qwen4Moe *moe, QW4CuEp *ep, const float *x_dev, float *y_dev, size_t tokens_local,
                                        uint32_t *ids_dev, float *weights_dev, Qwen4MoeWork *work, Qwen4Error *err);
Qwen4Status qw4cu_moe_ep_begin_device(const Qwen4Moe *moe, const float *x_dev, size_t tokens_local, float *rows_local_dev,
                                      uint32_t *ids_dev, float *weights_dev, Qwen4MoeWork *work, Qwen4Error *err);
Qwen4Status qw4cu_moe_ep_experts_device(const Qwen4Moe *moe, const float *rows_all_dev, size_t tokens_total, size_t own_first,
                                        float *partial_dev, Qwen4MoeWork *work, Qwen4Error *err);
/* Profiling aid of qw4cu_moe_ep_forward_device.  qw4cu_ep_trace(1) makes every later step record an event at its
 * ten stage boundaries and end with a synchronisation that adds the stage times up (0 switches it off; both clear
 * the sums).  qw4cu_ep_trace_read copies the summed milliseconds of stages 0-9 (router logits; routing and packing;
 * all-gather; local ids and lists; digits of x; gate/up; digits of the activations; down; shared-expert join and
 * partial sums; reduce-scatter) and returns the number of steps summed. */
void qw4cu_ep_trace(int on);
uint64_t qw4cu_ep_trace_read(double *ms, int n);
/* Router and routes only: x [tokens, hidden] -> ids, weights [tokens, k] (device pointers, either may be NULL). */
Qwen4Status qw4cu_moe_route_device(const Qwen4Moe *moe, const float *x_dev, size_t tokens,
                                   uint32_t *ids_dev, float *weights_dev, Qwen4MoeWork *work,
                                   Qwen4Error *err);
/* Makes every later call on this device enqueue on the caller's CUDA stream (a cudaStream_t
 * passed as void *), so that the library's kernels order with the caller's own work, e.g. the
 * collectives of an expert-parallel step.  NULL restores the library's own stream; the legacy
 * default stream is named by its handle cudaStreamLegacy ((cudaStream_t)1), not by 0. */
int qw4cu_set_stream(void *cuda_stream);

/* Timing on the workspace's stream with CUDA events.  begin/end record events; elapsed
 * waits for the end event and returns milliseconds (negative on error). */
int qw4cu_moe_work_timer_begin(Qwen4MoeWork *work);
int qw4cu_moe_work_timer_end(Qwen4MoeWork *work);
float qw4cu_moe_work_timer_elapsed_ms(Qwen4MoeWork *work);
/* Launch strategy of qw4cu_moe_forward_device.  0 (default): kernels are launched one by
 * one.  1: the second identical call on a workspace (same layer, pointers, token count) is
 * captured into a CUDA graph and later identical calls replay it. */
void qw4cu_set_graph_mode(int on);
int qw4cu_get_graph_mode(void);
/* Which expert kernels run.  -1 (default): batches of up to 64 tokens use the tensor-core
 * grouped kernels (groups of <= 4 rows, int8 MMA on the raw codes) when every expert tensor is
 * Q4_K or IQ2_XXS, everything else the CUDA-core kernels.  0: CUDA-core kernels only.  1:
 * tensor-core grouped kernels for any batch size the formats allow. */
void qw4cu_set_expert_path(int path);
/* One-kernel decode path (no counterpart in the reference): batches of up to four tokens whose
 * expert tensors are all Q4_K or IQ2_XXS run the whole layer as one persistent kernel, one CTA
 * per SM.  The reference's router arithmetic (serial sums, about 9 k cycles of dependent adds)
 * runs in a few CTAs of their own while the others start the experts from tree-summed logits; the
 * exact routes are compared with that speculation before the down projection, and the experts
 * are run again with the exact ids in the rare launch where the expert sets differ, so ids and
 * route weights are always the exact mode's.  -1 (default): used whenever the layer fits it; 0:
 * never (the multi-kernel sequence runs instead).  A layer that fits this path holds, for each of
 * its IQ2_XXS expert tensors, a second resident image made at create (4-bit codes, 4.5 bits per
 * weight: the kernel streams that one; same decoded values); qw4cu_moe_device_bytes counts it.
 * A layer created while mode 0 is in force gets neither the image nor the path, whatever the mode later.
 * qw4cu_decode_phase_clocks copies the SM clock that the first streaming CTA of the workspace's
 * last one-kernel launch read at its phase boundaries into clocks[0..12] (start, x staged, fast
 * logits written, x digitised, barrier 1 passed, expert sets speculated, sources listed, gate/up
 * slices done, activation digits stored, barrier 2 passed and routes received, routes verified,
 * activation digits loaded, end); call it after qw4cu_moe_work_sync.
 * qw4cu_decode_repairs: launches of this workspace, since it was created or reset, that had to
 * run the experts a second time.  qw4cu_set_decode_wrong_speculation(1) makes every later launch
 * speculate a wrong expert for its first token (test aid for that repair path; 0 restores). */
void qw4cu_set_fused_decode(int mode);
/* Tensor-core prefill path (no counterpart in the reference): batches of more than 64 tokens whose
 * expert tensors are all Q4_K run gate/up and down as grouped GEMMs on tcgen05 tensor cores with
 * TMEM accumulators (groups of <= 32 token rows per expert, exact integer codes as fp16 operands,
 * activations split into fp16 hi + lo).  -1 (default): used whenever the layer fits; 0: never. */
void qw4cu_set_prefill_path(int path);
/* Tile kernels: int8 tensor-core MMAs whose weight fragments are built once per group of <= 16 rows of an
 * expert (two-int8-digit activations staged in shared memory per group), for Q4_K, IQ2_XXS and Q2_K tensors.
 * -1 (default): batches of more than 64 rows that the tcgen05 prefill cannot take (IQ2_XXS tensors);
 * 0: never; 1: every batch of more than four rows. */
void qw4cu_set_tile_path(int path);
/* Profiling aid of the tensor-core prefill kernels: device_words is a device array of 64 x 8 bytes (NULL: off).
 * CTA 0 of every later launch stores the SM cycles its roles (0 epilogue, 1 dequantise, 2 TMA, 3 MMA issue,
 * 4 activation loader) spent waiting, at [32 * mode + 4 * role + kind]; kind 3 is the role's whole run. */
void qw4cu_prefill_debug(void *device_words);
int qw4cu_decode_phase_clocks(const Qwen4MoeWork *work, uint64_t clocks[16]);
int qw4cu_decode_repairs(const Qwen4MoeWork *work, uint32_t *count);
/* Profiling aid: the first `words` (<= 1024) 32-bit words of the one-kernel path's counter block: counters,
 * phase clocks, and from word 256 four marks per CTA (cycles since that CTA started). */
int qw4cu_decode_debug_words(const Qwen4MoeWork *work, uint32_t *out, size_t words);
void qw4cu_set_decode_wrong_speculation(int on);
/* Profiling aid: launch only one step of the small-batch sequence on later forwards, so that a
 * kernel can be timed back to back in isolation (the workspace keeps the results of an
 * earlier complete forward).  Steps: 0 router logits, 1 quantise x, 2 route + dispatch, 3 routed
 * gate+up, 4 shared gate+up, 5 quantise act, 6 routed down, 7 quantise shared act, 8 shared
 * down, 9 combine; -1 (default) runs the whole layer. */
void qw4cu_set_only_step(int step);
/* Profiling aid: while on, every layer forward records a CUDA event between its stages
 * (router logits + activation quantisation, route, dispatch, routed gate+up, shared gate+up,
 * routed down, shared down, combine) and graphs are not replayed.  qw4cu_stage_times copies
 * the accumulated milliseconds of the eight stages into ms[8] and the number of forwards into
 * *forwards, then clears both. */
void qw4cu_set_stage_timing(int on);
int qw4cu_stage_times(double *ms, uint64_t *forwards);
/* Kernels launched by this library in this process so far. */
uint64_t qw4cu_launch_count(void);
/* Names of the kernels launched after qw4cu_launch_log_begin (the first 512), comma-separated into out[cap];
 * returns how many were logged.  Not thread-safe: a test and profiling aid. */
void qw4cu_launch_log_begin(void);
size_t qw4cu_launch_log(char *out, size_t cap);

/* Decodes rows [row0, row0 + rows) of one expert of a resident tensor (index 0-7 in
 * Qwen4MoeWeights order) FROM THE DEVICE IMAGE into host floats [rows, k_storage].  Used to
 * prove that the resident (repacked) image decodes to the reference's bits. */
Qwen4Status qw4cu_moe_decode_rows(const Qwen4Moe *moe, uint32_t tensor, size_t expert,
                                  size_t row0, size_t rows, float *out, size_t out_elements,
                                  Qwen4Error *err);
/* The same from the EXPANDED image that the one-kernel decode path streams for an IQ2_XXS expert tensor
 * (tensor 1-6); QW4_UNSUPPORTED when the tensor has none (another format, or a layer that does not fit
 * that path). */
Qwen4Status qw4cu_moe_decode_rows_expanded(const Qwen4Moe *moe, uint32_t tensor, size_t expert,
                                           size_t row0, size_t rows, float *out, size_t out_elements,
                                           Qwen4Error *err);

/* Dispatch lists for ids that are already in device memory, computed WITHOUT allocating
 * anything.  This entry point has no counterpart in the reference.  It is for callers that
 * must not allocate while they run: a decode loop that has given all spare HBM to weights and
 * caches, where cudaMalloc can fail and in any case stalls the device.  The caller passes
 * inputs and outputs, all device pointers: ids_dev [tokens, top_k] dense uint32; offsets_dev
 * [experts + 1], pair_to_row_dev and row_to_pair_dev [tokens * top_k] uint32.  The kernel's own
 * working memory is a fixed array built into the library (about 33 KB of every GPU that loads
 * it, until exit), which limits a call to QW4CU_NOALLOC_MAX_EXPERTS experts and
 * QW4CU_NOALLOC_MAX_PAIRS pairs; more returns QW4_CAPACITY with the limit in the message.  One
 * CTA does the work in `pairs` loop steps, about a millisecond at the pair limit.
 * The first call on each device looks up the array's device address, so make that call before
 * any stream capture begins.  All calls share the array: calls that overlap on the GPU race,
 * so serialise them.
 * Stream: the kernel is enqueued on the stream the library uses at that moment (the one given
 * to qw4cu_set_stream, else the library's own stream once a workspace exists on the device,
 * else the legacy default stream), behind earlier library calls on it, so ids produced by
 * qw4cu_moe_route_device need no synchronisation in between.  The call then waits for that
 * stream and returns when the lists are complete.
 * Ids are taken to be distinct within a token (routing produces them so); an id >= experts
 * returns QW4_RANGE and leaves the outputs unspecified. */
#define QW4CU_NOALLOC_MAX_EXPERTS 4096
#define QW4CU_NOALLOC_MAX_PAIRS (1 << 18)
Qwen4Status qw4cu_group_pairs_device_noalloc(uint32_t experts, uint32_t top_k, size_t tokens,
                                             const uint32_t *ids_dev, uint32_t *offsets_dev,
                                             uint32_t *pair_to_row_dev, uint32_t *row_to_pair_dev,
                                             Qwen4Error *err);

/* ------------------------------------------------------------------------------------
 * One layer's MoE tensors straight from a GGUF v3 file (csrc/gguf_slice.c).
 *
 * picoforge reaches them through its model-wide loader: container parse src/gguf.c:31-106,
 * role table src/qwen4_weights.c:91-99, packed layouts src/qwen4_packed.c:8-32, dimensions
 * src/qwen4_config.c:170-172,200-211; its harness prints the same facts with --describe
 * (tests/test_qwen4_moe.c:376-396).  Tensor order everywhere below: router, gate, up, down,
 * shared gate, shared up, shared down, shared router (the order of Qwen4MoeWeights).
 * Names: blk.<layer>.ffn_gate_inp / ffn_{gate,up,down}_exps / ffn_{gate,up,down}_shexp /
 * ffn_gate_inp_shexp (.weight); keys: qwen4exp.embedding_length, .expert_count,
 * .expert_used_count, .expert_feed_forward_length, .expert_shared_feed_forward_length and the
 * optional ds4.qwen4.down.{logical,physical}_input.  A malformed file yields a status
 * (QW4_IO, QW4_FORMAT, QW4_MISSING, QW4_TYPE, QW4_SHAPE, QW4_UNSUPPORTED), never an abort.
 * ---------------------------------------------------------------------------------- */
typedef struct {
    char name[128];
    uint32_t type, rank;                   /* GGUF tensor type id; 1..3 dimensions */
    uint64_t shape[4];                     /* shape[0] is the contiguous (K) axis */
    uint64_t file_offset, bytes;           /* absolute offset of the payload in the file */
} QW4CuGgufTensor;

typedef struct {
    Qwen4MoeConfig config;                 /* trunk_type = the gate / up / down types of THIS layer */
    QW4CuGgufTensor tensor[8];
    QW4PackedLayout layout[8];
    uint64_t data_offset, file_bytes;
} QW4CuGgufSlice;

/* Header walk only: no payload byte is read and no device is touched. */
Qwen4Status qw4cu_gguf_slice_describe(const char *path, uint32_t layer, QW4CuGgufSlice *out, Qwen4Error *err);
/* describe + qwen4_moe_create on a read-only mapping of the file, released before returning (the resident
 * image is the only copy afterwards).  `slice` may be NULL. */
Qwen4Status qw4cu_moe_create_from_gguf(const char *path, uint32_t layer, Qwen4Moe **out, QW4CuGgufSlice *slice, Qwen4Error *err);

/* ------------------------------------------------------------------------------------
 * Speculative verify over a stack of layers, with the route log (csrc/verify_stack.c).
 *
 * The real caller of the four-token decode batch: picoforge appends one confirmed token plus up to three
 * drafts as one batch of 1..4 rows and then keeps the first n (qwen4_gpu_forward_verify / _keep,
 * src/qwen4_forward_gpu.h:55-63).  The MoE layer is stateless across tokens, so verify is a 1..4-row forward
 * per layer and keep moves the position.  With a log file set, every append writes the reference's record
 * (src/qwen4_forward_gpu.m:896-899): uint32 {position, rows, layers, top_k}, then ids [layer][row][top_k].
 * Layer l reads what layer l - 1 wrote (a stand-in for the engine's layer loop, whose attention and
 * hyper-connection steps lie outside this library).  `layers` are borrowed and must outlive the handle;
 * all must share `config`'s hidden size and top_k.
 * ---------------------------------------------------------------------------------- */
typedef struct QW4CuVerify QW4CuVerify;
Qwen4Status qw4cu_verify_create(Qwen4Moe *const *layers, size_t n_layers, const Qwen4MoeConfig *config, QW4CuVerify **out, Qwen4Error *err);
void qw4cu_verify_destroy(QW4CuVerify *verify);
/* path NULL stops logging; the file is truncated and flushed after every append. */
Qwen4Status qw4cu_verify_route_log(QW4CuVerify *verify, const char *path, Qwen4Error *err);
/* x_host, y_host: dense [count, hidden]; ids_host: [layers][count][top_k] or NULL; count 1..4 (QW4_CAPACITY otherwise).
 * An append while another is pending settles that one first with all its rows kept. */
Qwen4Status qw4cu_verify_append(QW4CuVerify *verify, const float *x_host, size_t count, float *y_host, uint32_t *ids_host, Qwen4Error *err);
/* keep 1..rows of the pending append (QW4_RANGE otherwise; QW4_BAD_STATE when nothing is pending). */
Qwen4Status qw4cu_verify_keep(QW4CuVerify *verify, size_t keep, Qwen4Error *err);
uint64_t qw4cu_verify_position(const QW4CuVerify *verify);
size_t qw4cu_verify_pending(const QW4CuVerify *verify);

/* Raw device memory and transfers for callers that keep activations in HBM. */
void *qw4cu_malloc(size_t bytes);
void qw4cu_free(void *device_pointer);
void *qw4cu_host_alloc(size_t bytes);            /* pinned host memory */
void qw4cu_host_free(void *host_pointer);
int qw4cu_upload(void *device_dst, const void *host_src, size_t bytes);
int qw4cu_download(void *host_dst, const void *device_src, size_t bytes);
/* Writes `bytes` of a scratch buffer larger than L2 so that the next kernel starts cold. */
int qw4cu_flush_l2(void);
/* Free and total bytes of the current device (cudaMemGetInfo); 0 on success. */
int qw4cu_mem_info(size_t *free_bytes, size_t *total_bytes);
int qw4cu_device_synchronize(void);

#ifdef __cplusplus
}
#endif
#endif /* QWEN4_MOE_B200_H */
