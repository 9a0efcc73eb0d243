/* Internal C boundary between the C11 host (moe_host.c) and the CUDA translation units.
 * Plain C types only.  Every function returns 0 on success or a nonzero CUDA error code,
 * whose text is kept for qw4cu_last_error(). */
#ifndef QW4_CUDA_SHIM_H
#define QW4_CUDA_SHIM_H
#include <stddef.h>
#include <stdint.h>

#include "../../include/qwen4_moe_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Mirror of qw4::DevTensor (formats.cuh). */
typedef struct {
    const uint8_t *data;
    uint32_t type;
    uint32_t k_storage, k_logical, n_out, n_experts;
    uint32_t row_bytes;
    uint64_t expert_bytes;
    /* tile kernels, gate / up tensors: tensor maps (CUtensorMap, 128 bytes each) of the sections of the resident image
     * (Q4_K and IQ2_XXS: the packed rows; Q2_K: codes, scale bytes, super-scales), made by qw4sh_tile_prepare; with them
     * the eight row pieces of a section come as one request.  0 sections: the kernel copies row by row. */
    unsigned char tile_maps[3][128];
    int tile_sections;
} QW4ShTensor;

typedef struct {
    uint32_t hidden, experts, top_k, inter, shared_inter, down_physical;
    int norm;
    QW4ShTensor w[8];             /* router, gate, up, down, sgate, sup, sdown, srouter */
    /* one-kernel decode path: tensor maps (CUtensorMap, 128 bytes each) of gate, up, shared gate, shared up, made by
     * qw4sh_fused_prepare once the images are resident; ready = 0 when the layer does not fit that path */
    unsigned char fused_maps[4][128];
    int fused_maps_ready;
    /* the same path: expanded images (4-bit codes) of the IQ2_XXS expert tensors, owned by the layer */
    void *fused_alt[8];
    size_t fused_alt_bytes;
} QW4ShLayer;

/* Device scratch of one workspace, sized for `cap` tokens. */
typedef struct {
    size_t cap;
    float *x, *y;                 /* [cap, hidden] staging for the host-pointer forward */
    float *logits, *probs;        /* [cap, experts] */
    float *shared_logit;          /* [cap] */
    uint32_t *ids;                /* [cap, k] */
    float *weights;               /* [cap, k] */
    uint32_t *offsets;            /* [experts + 1] */
    uint32_t *pair_to_row, *row_to_pair;  /* [cap * k] */
    uint32_t *active;             /* [experts + 1]: active[0] = count, then expert ids */
    float *act;                   /* [cap * k, inter] in pair order */
    float *shared_act;            /* [cap, shared_inter] */
    float *routed;                /* [cap, hidden], only when an observer is set */
    float *out;                   /* [cap * k, hidden] per-pair down outputs (tensor-core path) */
    float *shared_out;            /* [cap, hidden] */
    /* int8 digit images of the three activation matrices (quantize_rows): x [cap rows of
     * hidden], act [cap*k rows of inter], shared_act [cap rows of shared_inter] */
    int8_t *xq, *xneg, *aq, *aneg, *sq, *sneg;   /* [rows, 2, K] digits and negated digits */
    int *xsum, *asum, *ssum;      /* [rows, K / 32, 2] digit sums per 32-column chunk */
    float *xscale, *ascale, *sscale;  /* [rows] */
    void *groups, *shared_groups; /* [cap * k], [cap / 4 + 1] groups of <= 4 rows (16 bytes each) */
    uint32_t *n_groups;           /* [2]: routed, shared */
    uint32_t *status;             /* [4]: error bits, first bad row, spare */
    /* tensor-core prefill: fp16 hi / lo images and 32-column sums (hi, lo) of x [0-3], act [4-7], shared act [8-11] */
    void *half[12];
    void *groups32, *shared_groups32;  /* groups of <= 32 rows (16 bytes each): routed, shared */
    uint32_t *n_groups32;         /* [2]: routed, shared */
    uint32_t *dispatch_scratch;   /* [2 * experts * ceil(cap / 32) + experts]: token bitmaps, word prefixes, counts */
    uint32_t *sync;               /* [256]: counters and phase clocks of the one-kernel decode path */
    void *fused_aq, *fused_asc;   /* one-kernel decode path: activation digits and their per-chunk scales */
    float *logits_fast;           /* one-kernel decode path: tree-summed logits [4, experts + 1 padded to 4] */
    void *stream;                 /* cudaStream_t: the library's one stream on this device */
    void *timer[2];               /* cudaEvent_t */
    void *graph_cache;            /* replay cache of the launch sequence (qw4sh_graph_cache_create) */
    /* hyper-connection add fused into whichever kernel writes y (set per call, NULL otherwise):
     * residual [tokens, streams, hidden] += inject [tokens, streams] * y, multiply and add rounded separately */
    float *hc_residual;
    const float *hc_inject;
    uint32_t hc_streams;
    /* set per call, NULL otherwise: pinned host words [4] into which the one-kernel decode path copies the status
     * words when its last CTA leaves (the host forward then needs no copy of them) */
    uint32_t *status_mirror;
} QW4ShWork;

enum { QW4SH_ERR_NONFINITE = 1u, QW4SH_ERR_BOUNDS = 2u, QW4SH_ERR_STATE = 4u };

int qw4sh_device_count(void);
int qw4sh_set_device(int device);
int qw4sh_current_device(void);           /* -1 when the runtime cannot tell */
const char *qw4sh_last_error(void);
uint64_t qw4sh_launch_count(void);

void *qw4sh_malloc(size_t bytes);
void qw4sh_free(void *p);
void *qw4sh_host_alloc(size_t bytes);
void qw4sh_host_free(void *p);
int qw4sh_memcpy(void *dst, const void *src, size_t bytes, int to_device);
int qw4sh_memcpy2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch,
                         size_t width_bytes, size_t rows, int to_device, void *stream);
int qw4sh_memset_async(void *dst, int value, size_t bytes, void *stream);
/* The one non-blocking stream this library uses on the current device (created on first use,
 * never destroyed): layers run one after another, as the engine calls them. */
int qw4sh_shared_stream(void **stream);
void *qw4sh_graph_cache_create(void);
void qw4sh_graph_cache_destroy(void *cache);
/* 0: launch kernels directly.  1: the second identical forward (same layer, pointers, token
 * count) is captured into a CUDA graph and later ones replay it. */
void qw4sh_set_graph_mode(int on);
int qw4sh_get_graph_mode(void);
/* Per-kernel timing for profiles: when on, layer forwards record an event between stages
 * (and never replay graphs).  stage_times returns accumulated milliseconds for the
 * QW4SH_STAGES stages and the number of forwards accumulated, then clears them. */
enum { QW4SH_STAGES = 8 };
void qw4sh_set_stage_timing(int on);
/* -1 automatic (tensor-core grouped kernels for small batches), 0 CUDA-core kernels only,
 * 1 tensor-core grouped kernels whenever the formats allow. */
void qw4sh_set_expert_path(int path);
/* Profiling: launch only step `step` of the tensor-core decode sequence (-1: all). */
void qw4sh_set_only_step(int step);
/* Builds per-device tables of the tensor-core path (allocates: call outside stream capture). */
int qw4sh_prepare_mma(void);
int qw4sh_stage_times(double *ms, uint64_t *forwards);
int qw4sh_stream_sync(void *stream);
int qw4sh_device_sync(void);
int qw4sh_event_create(void **event);
void qw4sh_event_destroy(void *event);
int qw4sh_event_record(void *event, void *stream);
float qw4sh_event_elapsed_ms(void *begin, void *end);
int qw4sh_flush_l2(void);

/* Uploads one tensor (natural GGUF layout on the host) and regroups it into the resident
 * layout described in formats.cuh.  *device receives a cudaMalloc'ed image. */
int qw4sh_upload_tensor(const void *host, size_t bytes, uint32_t type, size_t k_storage,
                        size_t n_out, size_t n_experts, void **device);

/* out[rows, k_storage] (device) = exact decode of rows [row0, row0+rows) of one expert. */
int qw4sh_decode_rows(const QW4ShTensor *t, size_t expert, size_t row0, size_t rows, float *out,
                      void *stream);

/* Router arithmetic on logits [tokens, experts] with `pitch` floats per row.  status[0]
 * gets QW4SH_ERR_NONFINITE and status[1] the lowest bad row if a logit is not finite. */
int qw4sh_route(uint32_t experts, uint32_t k, int norm, const float *logits, size_t pitch,
                size_t tokens, float *probs, uint32_t *ids, float *weights, uint32_t *status,
                void *stream);

/* Stable per-expert lists of pair = token * k + slot. */
int qw4sh_group(uint32_t experts, uint32_t k, size_t tokens, const uint32_t *ids, uint32_t *offsets,
                uint32_t *pair_to_row, uint32_t *row_to_pair, uint32_t *active, uint32_t *status,
                void *stream);

/* The whole layer on device pointers: x, y dense [tokens, hidden].  router_mode 0 exact,
 * 1 fast.  ids_out / weights_out may be NULL. */
int qw4sh_layer_forward(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y,
                        size_t tokens, uint32_t *ids_out, float *weights_out, int router_mode);

/* One-kernel decode path (decode_fused.cu): up to four tokens, Q4_K / IQ2_XXS experts.
 * supported: 1 when the layer, batch and pointers fit it.  set_fused_decode: -1 automatic
 * (default), 0 never.  fused_decode launches it; phase_clocks copies CTA 0's SM clock at its
 * phase boundaries of the workspace's last launch (after a synchronise). */
int qw4sh_tile_prepare(QW4ShLayer *layer);
int qw4sh_takes_fused(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, const float *y, size_t tokens);
int qw4sh_fused_prepare(QW4ShLayer *layer);
void qw4sh_fused_release(QW4ShLayer *layer);
int qw4sh_fused_decode_rows_expanded(const QW4ShLayer *layer, int tensor, size_t expert, size_t row0, size_t rows, float *out, void *stream);
int qw4sh_fused_supported(const QW4ShLayer *layer, size_t tokens, const float *x, const float *y, int sm_count);
void qw4sh_set_fused_decode(int mode);
int qw4sh_fused_decode(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens,
                       uint32_t *ids_out, float *weights_out, int router_mode, int sm_count);
int qw4sh_fused_phase_clocks(const QW4ShWork *work, uint64_t clocks[16]);
/* Launches of this workspace whose speculated expert sets had to be repaired (since it was cleared). */
int qw4sh_fused_repairs(const QW4ShWork *work, uint32_t *count);
void qw4sh_set_wrong_speculation(int on);
void qw4sh_fused_scratch_sizes(const QW4ShLayer *layer, size_t *aq_bytes, size_t *asc_bytes, size_t *fast_bytes);

/* Tensor-core prefill path (prefill_tc.cu): Q4_K experts, groups of <= 32 token rows, tcgen05
 * MMAs with TMEM accumulators.  supported: 1 when a tensor fits it. */
/* Stable per-expert lists of plain rows (one id per row; 0xffffffff: none), one CTA. */
int qw4sh_group_rows(uint32_t experts, size_t rows, const uint32_t *ids, uint32_t *offsets, uint32_t *pair_to_row,
                     uint32_t *row_to_pair, uint32_t *active, uint32_t *status, void *stream);
/* Expert parallelism (ep_nccl.cu, kernels.cu): exchange rows of hidden + 2 * (k padded to 4) floats per token. */
typedef struct QW4ShEp QW4ShEp;
uint32_t qw4sh_ep_row_floats(uint32_t hidden, uint32_t k);
int qw4sh_ep_unique_id(unsigned char id[128]);
int qw4sh_ep_create(const unsigned char id[128], int rank, int world, QW4ShEp **out);
void qw4sh_ep_destroy(QW4ShEp *ep);
int qw4sh_ep_rank(const QW4ShEp *ep);
int qw4sh_ep_world(const QW4ShEp *ep);
int qw4sh_ep_reserve(QW4ShEp *ep, uint32_t hidden, uint32_t k, size_t tokens_local);
float *qw4sh_ep_msg_local(QW4ShEp *ep);
float *qw4sh_ep_msg_all(QW4ShEp *ep);
float *qw4sh_ep_partial_buffer(QW4ShEp *ep);
int qw4sh_ep_all_gather(QW4ShEp *ep, size_t floats_per_rank, uint32_t *status, void *stream);
int qw4sh_ep_reduce_scatter(QW4ShEp *ep, float *y, size_t floats_per_rank, uint32_t *status, void *stream);
int qw4sh_ep_transport(const QW4ShEp *ep);
int qw4sh_ep_wait_probe(uint32_t polls, int raise_first);   /* 1: this library's kernels over peer memory; 0: NCCL */
int qw4sh_graph_try(const QW4ShWork *work, const void *layer, const void *x, const void *y, const void *ids, const void *weights,
                    size_t tokens, int mode);
int qw4sh_graph_finish(const QW4ShWork *work, int enqueue_failed);
int qw4sh_ep_trace_on(void);
void qw4sh_ep_trace(int on);
int qw4sh_ep_trace_mark(int index, void *stream);
int qw4sh_ep_trace_collect(void);
uint64_t qw4sh_ep_trace_read(double *ms, int n);
int qw4sh_ep_begin(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, size_t tokens, float *msg_local, int router_mode);
int qw4sh_ep_experts(const QW4ShLayer *layer, const QW4ShWork *work, const float *msg_all, size_t total, size_t own_first, size_t own,
                     uint32_t first_expert, uint32_t local_experts, float *partial);
int qw4sh_quantize_rows_pitched(const float *x, uint32_t pitch, uint32_t rows, uint32_t k, int8_t *xq, int8_t *xneg, int *xsum,
                                float *xscale, void *stream);
void qw4sh_launch_log_begin(void);
size_t qw4sh_launch_log(char *out, size_t cap);
/* Tile kernels (experts_tile.cu): int8 tensor-core products for groups of <= 16 rows. */
int qw4sh_tile_supported(const QW4ShTensor *w, int mode);
void qw4sh_set_tile_path(int path);         /* -1 automatic (default), 0 never, 1 every batch of > 4 rows */
int qw4sh_build_tile_groups(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream);
int qw4sh_build_dense_tile_groups(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream);
int qw4sh_expert_tiles(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                       const uint32_t *row_to_pair, uint32_t k_div, const int8_t *digits, const int *sums, const float *scale,
                       float *out, uint32_t *status, int ctas, void *stream);
int qw4sh_prefill_supported(const QW4ShTensor *w, int mode);
void qw4sh_set_prefill_path(int path);      /* -1 automatic (default), 0 never */
/* Profiling aid: device array of 64 x 8 bytes (or NULL); CTA 0 of later prefill launches stores the cycles its
 * five roles spent in their waits: [32 * mode + 4 * role + kind], kind 3 = the role's total. */
void qw4sh_prefill_debug(void *device_words);
int qw4sh_split_rows(const float *x, uint32_t rows, uint32_t k, void *hi, void *lo, void *sum_hi, void *sum_lo, void *stream);
int qw4sh_build_groups32(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream);
int qw4sh_build_dense_groups32(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream);
int qw4sh_prefill_tc(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                     const uint32_t *row_to_pair, uint32_t k_div, const void *in_hi, const void *in_lo, const void *sum_hi,
                     const void *sum_lo, void *out_hi, void *out_lo, void *osum_hi, void *osum_lo, float *out, uint32_t *status,
                     int ctas, void *stream);

/* The layer stage by stage in the reference's order, every stage copied back and shown to `observer`
 * (observed_forward.cu).  The observer has the signature of QW4MoeObserver. */
int qw4sh_observed_forward(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens, const float *x_host,
                           size_t x_host_pitch, size_t token0, QW4MoeObserver observer, void *ctx);
int qw4sh_route_forward(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, size_t tokens, int router_mode);
/* Caller-provided stream (NULL: back to the library's own).  current_stream returns the one in force. */
int qw4sh_set_stream(void *stream);
int qw4sh_current_stream(void **stream);
/* The stream in force without creating one (NULL: the legacy default stream). */
int qw4sh_existing_stream(void **stream);
int qw4sh_mem_info(size_t *free_bytes, size_t *total_bytes);

#ifdef __cplusplus
}
#endif
#endif
