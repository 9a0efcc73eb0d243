/* C11 host side of the B200 Qwen4 MoE operator: handles, argument checking with the
 * reference's status codes, residency of the weights in HBM, host<->device staging.  All
 * arithmetic is in the CUDA translation units behind cuda_shim.h; there is no CPU path.
 *
 * The entry points mirror picoforge src/qwen4_moe.h:13-27 (see include/qwen4_moe_b200.h).
 */
#include "../../include/qwen4_moe_b200.h"
#include "cuda_shim.h"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

_Static_assert(sizeof(float) == 4 && sizeof(uint32_t) == 4, "32-bit elements");
_Static_assert(sizeof(Qwen4F32) == 88 && sizeof(QW4PackedLayout) == 64, "ABI layout");

enum { CHUNK_TOKENS = 2048, PIN_BYTES = 256 * 1024 };

struct Qwen4Moe {
    Qwen4MoeConfig c;
    QW4PackedCpuView host[8];     /* spans kept for the alias checks of forward */
    QW4ShLayer layer;             /* resident image */
    void *image[8];
    size_t device_bytes;
    size_t refs;
    bool alive;
    uint32_t first_expert, local_experts;   /* expert shard held by this handle (all of them unless sharded) */
};

struct Qwen4MoeWork {
    Qwen4Moe *owner;
    size_t cap, chunk, host_bytes, device_bytes;
    bool busy, failed;
    bool status_clean;            /* the device status words are known to be zero (last read back as zero, nothing launched since) */
    size_t shared_tokens;         /* expert-parallel step: tokens of a shared-expert branch started by the pack call */
    QW4ShWork d;
    void *device_block;           /* one allocation carved into d.* */
    uint32_t *status_host;        /* pinned [4] */
    unsigned char *pin;           /* pinned staging: x | y | ids | weights for small batches */
    QW4MoeObserver observer;
    void *observer_ctx;
};

typedef struct { uintptr_t first, end; } Span;

/* ---- errors --------------------------------------------------------------------------- */
/* Fills *err (when given) and hands the code back, so that `return raise(...)` reads as one step. */
static Qwen4Status raise(Qwen4Error *err, Qwen4Status code, const char *format, ...) {
    if (!err) return code;
    memset(err, 0, sizeof *err);
    err->code = code;
    if (code == QW4_OK) return code;
    strncpy(err->subject, "qwen4_moe", sizeof err->subject - 1);
    va_list args;
    va_start(args, format);
    vsnprintf(err->detail, sizeof err->detail, format, args);
    va_end(args);
    return code;
}
#define report(err, code, text) raise((err), (code), "%s", (text))
static Qwen4Status cuda_failure(Qwen4Error *err, const char *what) {
    return raise(err, QW4_GPU_ERROR, "%s: %s", what, qw4sh_last_error());
}
#define TRY(call) do { Qwen4Status st_ = (call); if (st_ != QW4_OK) return st_; } while (0)

static int router_mode = -1;
static int current_router_mode(void) {
    if (router_mode < 0) {
        const char *env = getenv("QW4CU_ROUTER");
        router_mode = env && strcmp(env, "fast") == 0 ? 1 : 0;
    }
    return router_mode;
}
void qw4cu_set_router_mode(int mode) { router_mode = mode ? 1 : 0; }
int qw4cu_get_router_mode(void) { return current_router_mode(); }

/* ---- argument views ---------------------------------------------------------------------
 * Every caller-owned array an entry point touches is described once as a Region (rows of
 * `cols` elements, `pitch` bytes apart) and validated by region_span, which also yields the
 * address range used for the overlap checks.  The status code of each defect and the order in
 * which defects are reported are the boundary contract (picoforge src/qwen4_moe.c:134-186):
 * shape, element stride, row-size overflow, row pitch, extent overflow, capacity, null,
 * alignment, address overflow. */
typedef struct {
    const char *name;
    const void *base;
    size_t capacity;              /* bytes the caller declares addressable */
    size_t rows, cols, pitch;     /* pitch in bytes */
    size_t elem;                  /* bytes per element; also the required alignment of base */
} Region;

static Qwen4Status region_span(const Region *r, Span *span, Qwen4Error *err) {
    *span = (Span){0, 0};
    if (r->cols > SIZE_MAX / r->elem) return raise(err, QW4_OVERFLOW, "%s: a row does not fit size_t", r->name);
    const size_t row = r->cols * r->elem;
    if (r->pitch < row || r->pitch % r->elem) return raise(err, QW4_STRIDE, "%s: row pitch %zu cannot hold %zu-byte rows", r->name, r->pitch, row);
    if (r->rows == 0 || row == 0) return QW4_OK;              /* nothing to address */
    if (r->rows - 1 > (SIZE_MAX - row) / r->pitch) return raise(err, QW4_OVERFLOW, "%s: extent does not fit size_t", r->name);
    const size_t extent = (r->rows - 1) * r->pitch + row;
    if (extent == 0) return QW4_OK;
    if (r->capacity < extent) return raise(err, QW4_CAPACITY, "%s: %zu bytes declared, %zu needed", r->name, r->capacity, extent);
    if (r->base == NULL) return raise(err, QW4_INVALID_ARGUMENT, "%s: null data for a nonempty view", r->name);
    const uintptr_t at = (uintptr_t)r->base;
    if (at % r->elem) return raise(err, QW4_STRIDE, "%s: data not aligned to %zu bytes", r->name, r->elem);
    if (extent > UINTPTR_MAX - at) return raise(err, QW4_OVERFLOW, "%s: address range wraps", r->name);
    *span = (Span){at, at + extent};
    return QW4_OK;
}
/* A rank-2 token-major FP32 view [rows, cols] (Qwen4F32 and Qwen4F32Mut share the layout). */
static Qwen4Status f32_span(const char *name, const float *data, size_t capacity, size_t rank, const size_t *dim, const size_t *stride,
                            size_t rows, size_t cols, Span *span, Qwen4Error *err) {
    if (rank != 2 || dim[0] != rows || dim[1] != cols) return raise(err, QW4_SHAPE, "%s: want a [%zu, %zu] matrix", name, rows, cols);
    if (stride[1] != sizeof(float)) return raise(err, QW4_STRIDE, "%s: last axis must be dense", name);
    const Region r = {name, data, capacity, rows, cols, stride[0], sizeof(float)};
    return region_span(&r, span, err);
}
#define F32_SPAN(name, view, rows, cols, span, err) \
    f32_span((name), (view).data, (view).capacity_bytes, (view).rank, (view).dim, (view).stride_bytes, (rows), (cols), (span), (err))
static Qwen4Status u32_span(const char *name, Qwen4U32Mut v, Span *span, Qwen4Error *err) {
    const Region r = {name, v.data, v.capacity_bytes, v.rows, v.cols, v.row_stride_bytes, sizeof(uint32_t)};
    return region_span(&r, span, err);
}
static bool spans_meet(Span a, Span b) { return a.first < b.end && b.first < a.end; }
static Qwen4Status all_apart(const Span *spans, size_t n, Qwen4Error *err) {
    for (size_t i = 1; i < n; i++)
        for (size_t j = 0; j < i; j++)
            if (spans_meet(spans[i], spans[j])) return raise(err, QW4_INVALID_ARGUMENT, "arguments %zu and %zu share memory", j, i);
    return QW4_OK;
}
static Qwen4Status check_config(const Qwen4MoeConfig *c, Qwen4Error *err) {
    if (!c) return raise(err, QW4_INVALID_ARGUMENT, "config pointer is null");
    const bool sized = c->hidden_size && c->experts && c->intermediate && c->shared_intermediate;
    const bool routable = c->top_k >= 1 && c->top_k <= c->experts;
    if (!sized || !routable || c->down_physical < c->intermediate) return raise(err, QW4_RANGE, "MoE dimensions out of range");
    return QW4_OK;
}

/* ---- packed layouts (status codes as picoforge src/qwen4_packed.c:8-50) --------------- */
static bool format_of(uint32_t type, size_t *block, size_t *bytes) {
    static const struct { uint32_t id; size_t block, bytes; } table[] = {
        {0, 1, 4}, {1, 1, 2}, {8, 32, 34}, {10, 256, 84}, {12, 256, 144}, {16, 256, 66}, {30, 1, 2}, {39, 32, 17}};
    for (size_t i = 0; i < sizeof table / sizeof *table; i++)
        if (table[i].id == type) { *block = table[i].block; *bytes = table[i].bytes; return true; }
    return false;
}
static bool mul_ok(size_t a, size_t b, size_t *out) {
    if (a && b > SIZE_MAX / a) return false;
    *out = a * b;
    return true;
}
static Qwen4Status check_packed(const QW4PackedCpuView *v, Qwen4Error *err) {
    const QW4PackedLayout *l = &v->layout;
    size_t block, bytes, row, expert, tensor;
    if (!format_of(l->gguf_type, &block, &bytes)) return report(err, QW4_FORMAT, "invalid weight view: format not executable");
    if (!l->k_logical || l->k_logical > l->k_storage || !l->n_out || !l->n_experts)
        return report(err, QW4_SHAPE, "invalid weight view: empty or incompatible dimensions");
    if (l->k_storage % block) return report(err, QW4_FORMAT, "invalid weight view: incomplete physical block");
    if (!mul_ok(l->k_storage / block, bytes, &row) || !mul_ok(row, l->n_out, &expert) || !mul_ok(expert, l->n_experts, &tensor))
        return report(err, QW4_OVERFLOW, "invalid weight view: tensor extent overflow");
    if (l->row_bytes != row || l->expert_bytes != expert || l->tensor_bytes != tensor)
        return report(err, QW4_FORMAT, "invalid weight view: layout bytes differ from physical shape");
    if (v->span.bytes < tensor) return report(err, QW4_CAPACITY, "invalid weight view: span shorter than tensor");
    if (!v->span.data || tensor > UINTPTR_MAX - (uintptr_t)v->span.data)
        return report(err, QW4_INVALID_ARGUMENT, "invalid weight view: bad address");
    if (l->k_storage > UINT32_MAX || l->n_out > UINT32_MAX || l->n_experts > UINT32_MAX || row > UINT32_MAX)
        return report(err, QW4_OVERFLOW, "invalid weight view: dimension exceeds 32 bits");
    return QW4_OK;
}

/* ---- create / destroy ------------------------------------------------------------------ */
static void release(Qwen4Moe *m) {
    if (m && --m->refs == 0) {
        for (int a = 0; a < 8; a++) qw4sh_free(m->image[a]);
        qw4sh_fused_release(&m->layer);
        free(m);
    }
}

static Qwen4Status create_shard(const Qwen4MoeConfig *c, const Qwen4MoeWeights *weights, uint32_t first_expert,
                                uint32_t local_experts, Qwen4Moe **out, Qwen4Error *err) {
    if (out) *out = NULL;
    if (!out || !weights) return report(err, QW4_INVALID_ARGUMENT, "null create argument");
    TRY(check_config(c, err));
    if (!local_experts || first_expert > c->experts || local_experts > c->experts - first_expert)
        return report(err, QW4_RANGE, "expert shard outside the layer");
    const QW4PackedCpuView w[8] = {weights->router, weights->gate, weights->up, weights->down,
        weights->shared_gate, weights->shared_up, weights->shared_down, weights->shared_router};
    const size_t h = c->hidden_size, i = c->intermediate, s = c->shared_intermediate;
    const size_t in[8] = {h, h, h, i, h, h, s, h}, n[8] = {c->experts, i, i, h, s, s, h, 1};
    for (size_t a = 0; a < 8; a++) {
        const QW4PackedLayout *l = &w[a].layout;
        const size_t experts = (a >= 1 && a <= 3) ? local_experts : 1;
        if (l->k_logical != in[a] || l->n_out != n[a] || l->n_experts != experts ||
            l->k_storage != (a == 3 ? c->down_physical : in[a]))
            return report(err, QW4_SHAPE, "MoE weight shape mismatch");
        if ((a == 0 || a == 7) && l->gguf_type != 0) return report(err, QW4_FORMAT, "router must be F32");
        TRY(check_packed(&w[a], err));
    }
    if (qw4sh_device_count() <= 0) return cuda_failure(err, "no CUDA device");
    Qwen4Moe *m = calloc(1, sizeof *m);
    if (!m) return report(err, QW4_OOM, "MoE allocation");
    m->c = *c; memcpy(m->host, w, sizeof w); m->refs = 1; m->alive = true;
    m->first_expert = first_expert; m->local_experts = local_experts;
    m->layer.hidden = c->hidden_size; m->layer.experts = c->experts; m->layer.top_k = c->top_k;
    m->layer.inter = c->intermediate; m->layer.shared_inter = c->shared_intermediate;
    m->layer.down_physical = c->down_physical; m->layer.norm = c->norm_topk_prob ? 1 : 0;
    for (size_t a = 0; a < 8; a++) {
        const QW4PackedLayout *l = &w[a].layout;
        if (qw4sh_upload_tensor(w[a].span.data, l->tensor_bytes, l->gguf_type, l->k_storage, l->n_out, l->n_experts, &m->image[a])) {
            release(m);
            return cuda_failure(err, "weight upload");
        }
        m->device_bytes += l->tensor_bytes;
        m->layer.w[a] = (QW4ShTensor){.data = m->image[a], .type = l->gguf_type, .k_storage = (uint32_t)l->k_storage,
            .k_logical = (uint32_t)l->k_logical, .n_out = (uint32_t)l->n_out, .n_experts = (uint32_t)l->n_experts,
            .row_bytes = (uint32_t)l->row_bytes, .expert_bytes = l->expert_bytes};
    }
    (void)qw4sh_tile_prepare(&m->layer);
    if (qw4sh_fused_prepare(&m->layer)) { release(m); return cuda_failure(err, "decode path images"); }
    m->device_bytes += m->layer.fused_alt_bytes;
    *out = m;
    return report(err, QW4_OK, "");
}

/* For a creator that owned the host bytes only for the duration of create (the GGUF slice reader): the handle
 * stops remembering their addresses. */
void qw4cu_moe_forget_host_weights(Qwen4Moe *m) {
    if (m) for (size_t a = 0; a < 8; a++) m->host[a].span = (Qwen4CpuSpan){NULL, 0};
}

Qwen4Status qwen4_moe_create(const Qwen4MoeConfig *c, const Qwen4MoeWeights *weights, Qwen4Moe **out, Qwen4Error *err) {
    return create_shard(c, weights, 0, c ? c->experts : 0, out, err);
}
Qwen4Status qw4cu_moe_create_sharded(const Qwen4MoeConfig *c, const Qwen4MoeWeights *weights, uint32_t first_expert,
                                     uint32_t local_experts, Qwen4Moe **out, Qwen4Error *err) {
    return create_shard(c, weights, first_expert, local_experts, out, err);
}

void qwen4_moe_destroy(Qwen4Moe *m) {
    if (m && m->alive) { m->alive = false; release(m); }
}
size_t qw4cu_moe_device_bytes(const Qwen4Moe *m) { return m ? m->device_bytes : 0; }

/* ---- workspace ------------------------------------------------------------------------- */
static void *status_start(Qwen4MoeWork *w) {
    w->status_host[0] = 0; w->status_host[1] = UINT32_MAX; w->status_host[2] = 0; w->status_host[3] = 0;
    return w->status_host;
}
/* Clears the device error word, ahead of a batch of launches. */
static int status_clear(Qwen4MoeWork *w) {
    status_start(w);
    return qw4sh_memcpy2d_async(w->d.status, 16, w->status_host, 16, 16, 1, 1, w->d.stream);
}
typedef struct { size_t offset[64], total; } Plan;
static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static size_t pairs_of(const Qwen4Moe *m, size_t chunk) { return chunk * m->c.top_k; }

static Qwen4Status plan_work(const Qwen4Moe *m, size_t cap, size_t *chunk, Plan *plan, Qwen4Error *err) {
    if (!m || !m->alive) return report(err, QW4_BAD_STATE, "inactive MoE");
    const size_t t = cap < CHUNK_TOKENS ? cap : CHUNK_TOKENS, k = m->c.top_k, e = m->c.experts, h = m->c.hidden_size;
    if (k && t > SIZE_MAX / k) return report(err, QW4_OVERFLOW, "pair count overflow");
    const size_t pairs = t * k;
    const size_t i = m->c.intermediate, si = m->c.shared_intermediate;
    /* sizes in 4-byte words */
    const size_t g32 = pairs / 32 + e + 2;                   /* groups of <= 32 rows: at most pairs/32 + experts */
    size_t fused_aq = 0, fused_asc = 0, fused_fast = 0;
    qw4sh_fused_scratch_sizes(&m->layer, &fused_aq, &fused_asc, &fused_fast);
    const size_t count[52] = {t * h, t * h, t * e, t * e, t, pairs, pairs, e + 1, pairs, pairs, e + 1,
        pairs * i, t * si, t * h, 4,
        pairs * h, t * h,                                   /* 15 out, 16 shared_out */
        t * h / 2 + 8, t * h / 2 + 8, t * (h / 32 + 1) * 2, t,                 /* 17 xq, 18 xneg, 19 xsum, 20 xscale */
        pairs * i / 2 + 8, pairs * i / 2 + 8, pairs * (i / 32 + 1) * 2, pairs,  /* 21 aq, 22 aneg, 23 asum, 24 ascale */
        t * si / 2 + 8, t * si / 2 + 8, t * (si / 32 + 1) * 2, t,              /* 25 sq, 26 sneg, 27 ssum, 28 sscale */
        pairs * 4 + t + 16, t + 8, 4, 1024, 0,
        /* 34.. tensor-core prefill: fp16 hi/lo images (2 bytes per value) and 32-column sums of x, act, shared act; groups */
        t * h / 2 + 8, t * h / 2 + 8, t * (h / 32) / 2 + 8, t * (h / 32) / 2 + 8,               /* 34 xh_hi, 35 xh_lo, 36 xs_hi, 37 xs_lo */
        pairs * i / 2 + 8, pairs * i / 2 + 8, pairs * (i / 32 + 1) / 2 + 8, pairs * (i / 32 + 1) / 2 + 8,   /* 38-41 act */
        t * si / 2 + 8, t * si / 2 + 8, t * (si / 32 + 1) / 2 + 8, t * (si / 32 + 1) / 2 + 8,           /* 42-45 shared act */
        g32 * 4 + (t / 32 + 2) * 4, 8,
        2 * e * (t / 32 + 1) + e + 8,
        fused_aq / 4, fused_asc / 4, fused_fast / 4};                                    /* 49-51 one-kernel decode path */                                                      /* 48 dispatch scratch */                                                      /* 46 groups32 (routed, then shared), 47 counts */                                  /* 29 groups, 30 spare, 31 n_groups, 32 sync */
    size_t at = 0;
    for (int j = 0; j < 52; j++) {
        if (count[j] > (SIZE_MAX >> 4)) return report(err, QW4_OVERFLOW, "scratch size overflow");
        plan->offset[j] = at;
        at += align256(count[j] * 4 + 4);
    }
    plan->total = at;
    *chunk = t;
    return QW4_OK;
}

Qwen4Status qwen4_moe_work_size(const Qwen4Moe *m, size_t cap, size_t *bytes, Qwen4Error *err) {
    if (!bytes) return report(err, QW4_INVALID_ARGUMENT, "null size output");
    *bytes = 0;
    Plan plan; size_t chunk;
    TRY(plan_work(m, cap, &chunk, &plan, err));
    *bytes = sizeof(Qwen4MoeWork) + PIN_BYTES + 64;
    return report(err, QW4_OK, "");
}

void qwen4_moe_work_destroy(Qwen4MoeWork *w) {
    if (!w || w->busy) return;
    if (w->d.stream) qw4sh_stream_sync(w->d.stream);
    qw4sh_event_destroy(w->d.timer[0]); qw4sh_event_destroy(w->d.timer[1]);
    qw4sh_graph_cache_destroy(w->d.graph_cache);
    qw4sh_free(w->device_block);
    qw4sh_host_free(w->status_host);
    qw4sh_host_free(w->pin);
    release(w->owner);
    free(w);
}

Qwen4Status qwen4_moe_work_create(const Qwen4Moe *m, size_t cap, size_t budget, Qwen4MoeWork **out, Qwen4Error *err) {
    if (out) *out = NULL;
    if (!out) return report(err, QW4_INVALID_ARGUMENT, "null workspace output");
    Plan plan; size_t chunk;
    TRY(plan_work(m, cap, &chunk, &plan, err));
    const size_t host_bytes = sizeof(Qwen4MoeWork) + PIN_BYTES + 64;
    if (budget < host_bytes) return report(err, QW4_CAPACITY, "workspace budget too small");
    Qwen4MoeWork *w = calloc(1, sizeof *w);
    if (!w) return report(err, QW4_OOM, "workspace metadata");
    w->owner = (Qwen4Moe *)m; w->owner->refs++;
    w->cap = cap; w->chunk = chunk; w->host_bytes = host_bytes; w->device_bytes = plan.total;
    w->device_block = qw4sh_malloc(plan.total);
    w->status_host = qw4sh_host_alloc(64);
    w->pin = qw4sh_host_alloc(PIN_BYTES);
    w->d.graph_cache = qw4sh_graph_cache_create();
    if (!w->device_block || !w->status_host || !w->pin || !w->d.graph_cache || qw4sh_shared_stream(&w->d.stream) ||
        qw4sh_event_create(&w->d.timer[0]) || qw4sh_event_create(&w->d.timer[1])) {
        Qwen4Status st = cuda_failure(err, "workspace allocation");
        qwen4_moe_work_destroy(w);
        return st;
    }
    char *base = w->device_block;
    w->d.cap = chunk;
    w->d.x = (float *)(base + plan.offset[0]); w->d.y = (float *)(base + plan.offset[1]);
    w->d.logits = (float *)(base + plan.offset[2]); w->d.probs = (float *)(base + plan.offset[3]);
    w->d.shared_logit = (float *)(base + plan.offset[4]);
    w->d.ids = (uint32_t *)(base + plan.offset[5]); w->d.weights = (float *)(base + plan.offset[6]);
    w->d.offsets = (uint32_t *)(base + plan.offset[7]);
    w->d.pair_to_row = (uint32_t *)(base + plan.offset[8]); w->d.row_to_pair = (uint32_t *)(base + plan.offset[9]);
    w->d.active = (uint32_t *)(base + plan.offset[10]);
    w->d.act = (float *)(base + plan.offset[11]); w->d.shared_act = (float *)(base + plan.offset[12]);
    w->d.routed = NULL;
    w->d.status = (uint32_t *)(base + plan.offset[14]);
    w->d.out = (float *)(base + plan.offset[15]); w->d.shared_out = (float *)(base + plan.offset[16]);
    w->d.xq = (int8_t *)(base + plan.offset[17]); w->d.xneg = (int8_t *)(base + plan.offset[18]);
    w->d.xsum = (int *)(base + plan.offset[19]); w->d.xscale = (float *)(base + plan.offset[20]);
    w->d.aq = (int8_t *)(base + plan.offset[21]); w->d.aneg = (int8_t *)(base + plan.offset[22]);
    w->d.asum = (int *)(base + plan.offset[23]); w->d.ascale = (float *)(base + plan.offset[24]);
    w->d.sq = (int8_t *)(base + plan.offset[25]); w->d.sneg = (int8_t *)(base + plan.offset[26]);
    w->d.ssum = (int *)(base + plan.offset[27]); w->d.sscale = (float *)(base + plan.offset[28]);
    w->d.groups = base + plan.offset[29]; w->d.shared_groups = base + plan.offset[30];
    w->d.n_groups = (uint32_t *)(base + plan.offset[31]);
    w->d.sync = (uint32_t *)(base + plan.offset[32]);
    for (int j = 0; j < 12; j++) w->d.half[j] = base + plan.offset[34 + j];
    w->d.groups32 = base + plan.offset[46];
    w->d.shared_groups32 = (char *)w->d.groups32 + (pairs_of(m, chunk) / 32 + m->c.experts + 2) * 16;
    w->d.n_groups32 = (uint32_t *)(base + plan.offset[47]);
    w->d.dispatch_scratch = (uint32_t *)(base + plan.offset[48]);
    w->d.fused_aq = base + plan.offset[49]; w->d.fused_asc = base + plan.offset[50];
    w->d.logits_fast = (float *)(base + plan.offset[51]);
    if (qw4sh_prepare_mma()) {
        Qwen4Status st = cuda_failure(err, "tensor-core tables");
        qwen4_moe_work_destroy(w);
        return st;
    }
    if (qw4sh_memset_async(w->device_block, 0, plan.total, w->d.stream) || status_clear(w) || qw4sh_stream_sync(w->d.stream)) {
        Qwen4Status st = cuda_failure(err, "workspace clear");
        qwen4_moe_work_destroy(w);
        return st;
    }
    *out = w;
    return report(err, QW4_OK, "");
}

Qwen4Status qwen4_moe_work_reset(Qwen4MoeWork *w, Qwen4Error *err) {
    if (!w) return report(err, QW4_INVALID_ARGUMENT, "null workspace");
    if (w->busy) return report(err, QW4_BUSY, "workspace executing");
    if (!w->owner->alive) return report(err, QW4_BAD_STATE, "destroyed owner");
    if (qw4sh_memset_async(w->device_block, 0, w->device_bytes, w->d.stream) || status_clear(w) || qw4sh_stream_sync(w->d.stream))
        return cuda_failure(err, "workspace clear");
    w->failed = false;
    return report(err, QW4_OK, "");
}
size_t qw4cu_moe_work_device_bytes(const Qwen4MoeWork *w) { return w ? w->device_bytes : 0; }

void qw4_moe_observe(Qwen4MoeWork *w, QW4MoeObserver fn, void *ctx) {
    if (w && !w->busy) { w->observer = fn; w->observer_ctx = ctx; }
}

/* ---- forward ---------------------------------------------------------------------------- */
static void use_current_stream(Qwen4MoeWork *w) {
    void *stream = NULL;
    if (!qw4sh_current_stream(&stream)) w->d.stream = stream;
}
static Qwen4Status status_result(Qwen4MoeWork *w, Qwen4Error *err) {
    const uint32_t bits = w->status_host[0];
    if (bits & QW4SH_ERR_BOUNDS) return report(err, QW4_GPU_ERROR, "expert id outside the tensor");
    if (bits & QW4SH_ERR_STATE) return report(err, QW4_GPU_ERROR, "device state error");
    if (bits & QW4SH_ERR_NONFINITE) {
        Qwen4Status st = report(err, QW4_NONFINITE, "nonfinite input or arithmetic");
        if (err && w->status_host[1] != UINT32_MAX) err->row = w->status_host[1];
        return st;
    }
    return QW4_OK;
}

Qwen4Status qw4cu_moe_forward_device(const Qwen4Moe *m, const float *x_dev, float *y_dev, size_t tokens,
                                     uint32_t *ids_dev, float *weights_dev, Qwen4MoeWork *w, Qwen4Error *err) {
    if (!m || !w) return report(err, QW4_INVALID_ARGUMENT, "null forward handle");
    if (w->owner != m) return report(err, QW4_OWNER, "workspace belongs to another MoE");
    if (!m->alive || w->failed) return report(err, QW4_BAD_STATE, "inactive MoE/workspace; reset required");
    if (w->busy) return report(err, QW4_BUSY, "workspace executing");
    if (tokens > w->cap) return report(err, QW4_CAPACITY, "batch exceeds token capacity");
    if (tokens && (!x_dev || !y_dev)) return report(err, QW4_INVALID_ARGUMENT, "null device view");
    if (m->local_experts != m->c.experts) return report(err, QW4_BAD_STATE, "sharded handle: use the route/experts/combine calls");
    use_current_stream(w);
    w->status_clean = false;
    const size_t h = m->c.hidden_size, k = m->c.top_k;
    for (size_t start = 0; start < tokens; start += w->chunk) {
        const size_t n = tokens - start < w->chunk ? tokens - start : w->chunk;
        if (qw4sh_layer_forward(&m->layer, &w->d, x_dev + start * h, y_dev + start * h, n,
                                ids_dev ? ids_dev + start * k : NULL, weights_dev ? weights_dev + start * k : NULL,
                                current_router_mode()))
            return cuda_failure(err, "layer launch");
    }
    return report(err, QW4_OK, "");
}

/* The layer followed by the hyper-connection add of its caller (picoforge src/qwen4_forward.c:365-367,
 * src/qwen4_base.c:160-176): residual [tokens, streams, hidden] += inject [tokens, streams] * y, applied by the
 * kernel that writes y (the reference's GPU path fuses it the same way, src/qwen4_moe_internal.h:55-58). */
Qwen4Status qw4cu_moe_forward_hc_add_device(const Qwen4Moe *m, const float *x_dev, float *y_dev, size_t tokens, float *residual_dev,
                                            const float *inject_dev, size_t streams, Qwen4MoeWork *w, Qwen4Error *err) {
    if (!m || !w) return report(err, QW4_INVALID_ARGUMENT, "null forward handle");
    if (tokens && (!residual_dev || !inject_dev)) return report(err, QW4_INVALID_ARGUMENT, "null hyper-connection view");
    if (!streams || streams > 64) return report(err, QW4_SHAPE, "hyper-connection streams out of range");
    if (tokens > w->chunk) return report(err, QW4_CAPACITY, "batch exceeds one launch sequence (2048 rows)");
    w->d.hc_residual = residual_dev; w->d.hc_inject = inject_dev; w->d.hc_streams = (uint32_t)streams;
    const Qwen4Status st = qw4cu_moe_forward_device(m, x_dev, y_dev, tokens, NULL, NULL, w, err);
    w->d.hc_residual = NULL; w->d.hc_inject = NULL; w->d.hc_streams = 0;
    return st;
}

/* ---- expert-parallel pieces -------------------------------------------------------------- */
static Qwen4Status piece_checks(const Qwen4Moe *m, Qwen4MoeWork *w, size_t rows, Qwen4Error *err) {
    if (!m || !w) return report(err, QW4_INVALID_ARGUMENT, "null forward handle");
    if (w->owner != m) return report(err, QW4_OWNER, "workspace belongs to another MoE");
    if (!m->alive || w->failed) return report(err, QW4_BAD_STATE, "inactive MoE/workspace; reset required");
    if (w->busy) return report(err, QW4_BUSY, "workspace executing");
    if (rows > w->chunk || rows > w->cap) return report(err, QW4_CAPACITY, "batch exceeds the workspace (capacity, 2048 rows at most)");
    use_current_stream(w);
    w->status_clean = false;
    return QW4_OK;
}
Qwen4Status qw4cu_moe_route_device(const Qwen4Moe *m, const float *x_dev, size_t tokens, uint32_t *ids_dev, float *weights_dev,
                                   Qwen4MoeWork *w, Qwen4Error *err) {
    TRY(piece_checks(m, w, tokens, err));
    if (tokens && !x_dev) return report(err, QW4_INVALID_ARGUMENT, "null device view");
    if (qw4sh_route_forward(&m->layer, &w->d, x_dev, tokens, current_router_mode())) return cuda_failure(err, "route launch");
    const size_t bytes = tokens * m->c.top_k * 4;
    if (tokens && ids_dev && qw4sh_memcpy2d_async(ids_dev, bytes, w->d.ids, bytes, bytes, 1, 2, w->d.stream)) return cuda_failure(err, "ids copy");
    if (tokens && weights_dev && qw4sh_memcpy2d_async(weights_dev, bytes, w->d.weights, bytes, bytes, 1, 2, w->d.stream)) return cuda_failure(err, "weights copy");
    return report(err, QW4_OK, "");
}
/* ---- expert parallelism ------------------------------------------------------------------ */
struct QW4CuEp { QW4ShEp *shim; };

int qw4cu_ep_unique_id(unsigned char id[128]) { return id ? qw4sh_ep_unique_id(id) : -1; }
Qwen4Status qw4cu_ep_create(const unsigned char id[128], int rank, int world, QW4CuEp **out, Qwen4Error *err) {
    if (out) *out = NULL;
    if (!out || (world > 1 && !id)) return report(err, QW4_INVALID_ARGUMENT, "null communicator argument");
    if (world < 1 || rank < 0 || rank >= world) return report(err, QW4_RANGE, "rank outside the world");
    static const unsigned char none[128] = {0};
    QW4CuEp *ep = calloc(1, sizeof *ep);
    if (!ep) return report(err, QW4_OOM, "communicator");
    if (qw4sh_ep_create(id ? id : none, rank, world, &ep->shim)) { free(ep); return cuda_failure(err, "communicator"); }
    *out = ep;
    return report(err, QW4_OK, "");
}
void qw4cu_ep_trace(int on) { qw4sh_ep_trace(on); }
uint64_t qw4cu_ep_trace_read(double *ms, int n) { return ms ? qw4sh_ep_trace_read(ms, n) : 0; }
void qw4cu_ep_destroy(QW4CuEp *ep) { if (ep) { qw4sh_ep_destroy(ep->shim); free(ep); } }
int qw4cu_ep_transport(const QW4CuEp *ep) { return ep ? qw4sh_ep_transport(ep->shim) : 0; }
int qw4cu_ep_wait_probe(uint32_t polls, int raise_first) {
    const int bits = qw4sh_ep_wait_probe(polls, raise_first);
    return bits < 0 ? -1 : (bits & QW4SH_ERR_STATE) ? 1 : 0;
}
size_t qw4cu_ep_row_floats(const Qwen4Moe *m) { return m ? qw4sh_ep_row_floats((uint32_t)m->c.hidden_size, (uint32_t)m->c.top_k) : 0; }

static Qwen4Status ep_shard(const Qwen4Moe *m, size_t world, size_t rank, Qwen4Error *err) {
    if (!m->local_experts || m->c.experts % m->local_experts || m->c.experts / m->local_experts != world ||
        m->first_expert != rank * m->local_experts)
        return report(err, QW4_BAD_STATE, "the handle must hold this rank's block of experts (equal contiguous blocks, rank-th block)");
    return QW4_OK;
}
Qwen4Status qw4cu_moe_ep_begin_device(const Qwen4Moe *m, const float *x_dev, size_t tokens_local, float *rows_local_dev, uint32_t *ids_dev,
                                      float *weights_dev, Qwen4MoeWork *w, Qwen4Error *err) {
    TRY(piece_checks(m, w, tokens_local, err));
    if (tokens_local && (!x_dev || !rows_local_dev)) return report(err, QW4_INVALID_ARGUMENT, "null device view");
    if (qw4sh_ep_begin(&m->layer, &w->d, x_dev, tokens_local, rows_local_dev, current_router_mode())) return cuda_failure(err, "route and pack");
    const size_t bytes = tokens_local * m->c.top_k * 4;
    if (tokens_local && ids_dev && qw4sh_memcpy2d_async(ids_dev, bytes, w->d.ids, bytes, bytes, 1, 2, w->d.stream)) return cuda_failure(err, "ids copy");
    if (tokens_local && weights_dev && qw4sh_memcpy2d_async(weights_dev, bytes, w->d.weights, bytes, bytes, 1, 2, w->d.stream)) return cuda_failure(err, "weights copy");
    w->shared_tokens = tokens_local;
    return report(err, QW4_OK, "");
}
Qwen4Status qw4cu_moe_ep_experts_device(const Qwen4Moe *m, const float *rows_all_dev, size_t tokens_total, size_t own_first, float *partial_dev,
                                        Qwen4MoeWork *w, Qwen4Error *err) {
    TRY(piece_checks(m, w, tokens_total, err));
    if (tokens_total && (!rows_all_dev || !partial_dev)) return report(err, QW4_INVALID_ARGUMENT, "null device view");
    const size_t own = w->shared_tokens;
    w->shared_tokens = 0;
    if (own_first > tokens_total || own > tokens_total - own_first) return report(err, QW4_RANGE, "own tokens outside the gathered batch");
    if (tokens_total + own > w->cap) return report(err, QW4_CAPACITY, "workspace capacity must cover all ranks' tokens plus this rank's own");
    if (qw4sh_ep_experts(&m->layer, &w->d, rows_all_dev, tokens_total, own_first, own, m->first_expert, m->local_experts, partial_dev))
        return cuda_failure(err, "experts launch");
    return report(err, QW4_OK, "");
}
Qwen4Status qw4cu_moe_ep_forward_device(const Qwen4Moe *m, QW4CuEp *ep, const float *x_dev, float *y_dev, size_t tokens_local, uint32_t *ids_dev,
                                        float *weights_dev, Qwen4MoeWork *w, Qwen4Error *err) {
    if (!ep) return report(err, QW4_INVALID_ARGUMENT, "null communicator");
    if (!m || !w) return report(err, QW4_INVALID_ARGUMENT, "null forward handle");
    const size_t world = (size_t)qw4sh_ep_world(ep->shim), rank = (size_t)qw4sh_ep_rank(ep->shim);
    TRY(ep_shard(m, world, rank, err));
    if (tokens_local && (!x_dev || !y_dev)) return report(err, QW4_INVALID_ARGUMENT, "null device view");
    if (tokens_local > (w->cap) / (world + 1)) return report(err, QW4_CAPACITY, "workspace capacity must cover all ranks' tokens plus this rank's own");
    if (!tokens_local) return report(err, QW4_OK, "");
    const uint32_t h = (uint32_t)m->c.hidden_size, k = (uint32_t)m->c.top_k;
    if (qw4sh_ep_reserve(ep->shim, h, k, tokens_local)) return cuda_failure(err, "exchange buffers");
    TRY(piece_checks(m, w, tokens_local, err));
    /* graph mode: the second identical step on this workspace is captured (collectives included), later ones replay it */
    const int graph = qw4sh_ep_trace_on() ? 0 : qw4sh_graph_try(&w->d, ep, x_dev, y_dev, ids_dev, weights_dev, tokens_local, 1000 + (int)world);
    if (graph < 0) return cuda_failure(err, "graph replay");
    if (graph == 1) return report(err, QW4_OK, "");
    Qwen4Status st = qw4cu_moe_ep_begin_device(m, x_dev, tokens_local, qw4sh_ep_msg_local(ep->shim), ids_dev, weights_dev, w, err);
    if (st == QW4_OK && qw4sh_ep_all_gather(ep->shim, tokens_local * qw4sh_ep_row_floats(h, k), w->d.status, w->d.stream)) st = cuda_failure(err, "all-gather");
    if (st == QW4_OK)
        st = qw4cu_moe_ep_experts_device(m, qw4sh_ep_msg_all(ep->shim), tokens_local * world, rank * tokens_local,
                                         qw4sh_ep_partial_buffer(ep->shim), w, err);
    if (st == QW4_OK && qw4sh_ep_reduce_scatter(ep->shim, y_dev, tokens_local * h, w->d.status, w->d.stream)) st = cuda_failure(err, "reduce-scatter");
    if (graph == 2 && qw4sh_graph_finish(&w->d, st != QW4_OK) && st == QW4_OK) st = cuda_failure(err, "graph capture");
    if (st != QW4_OK) return st;
    if (qw4sh_ep_trace_mark(10, w->d.stream) || qw4sh_ep_trace_collect()) return cuda_failure(err, "stage trace");
    return report(err, QW4_OK, "");
}
int qw4cu_set_stream(void *cuda_stream) { return qw4sh_set_stream(cuda_stream); }

Qwen4Status qw4cu_moe_work_sync(Qwen4MoeWork *w, Qwen4Error *err) {
    if (!w) return report(err, QW4_INVALID_ARGUMENT, "null workspace");
    use_current_stream(w);
    if (qw4sh_memcpy2d_async(w->status_host, 16, w->d.status, 16, 16, 1, 0, w->d.stream) || qw4sh_stream_sync(w->d.stream)) {
        w->failed = true;
        return cuda_failure(err, "stream synchronize");
    }
    Qwen4Status st = status_result(w, err);
    if (st != QW4_OK) { w->failed = true; status_clear(w); qw4sh_stream_sync(w->d.stream); return st; }
    return report(err, QW4_OK, "");
}

/* The same for several workspaces that share the stream in force (layers enqueued back to back): every status
 * word is fetched first, then ONE wait, then each workspace is judged in order; the first failure is returned and
 * its workspace latched (the later ones are judged too, so that none stays unexamined). */
Qwen4Status qw4cu_moe_work_sync_many(Qwen4MoeWork *const *works, size_t n, Qwen4Error *err) {
    if (!works && n) return report(err, QW4_INVALID_ARGUMENT, "null workspace list");
    void *stream = NULL;
    for (size_t i = 0; i < n; i++) {
        if (!works[i]) return report(err, QW4_INVALID_ARGUMENT, "null workspace");
        use_current_stream(works[i]);
        stream = works[i]->d.stream;
        if (qw4sh_memcpy2d_async(works[i]->status_host, 16, works[i]->d.status, 16, 16, 1, 0, stream)) {
            works[i]->failed = true;
            return cuda_failure(err, "status copy");
        }
    }
    if (n && qw4sh_stream_sync(stream)) {
        for (size_t i = 0; i < n; i++) works[i]->failed = true;
        return cuda_failure(err, "stream synchronize");
    }
    Qwen4Status first = QW4_OK;
    Qwen4Error local;
    bool cleared = false;
    for (size_t i = 0; i < n; i++) {
        const Qwen4Status st = status_result(works[i], first == QW4_OK ? err : &local);
        if (st == QW4_OK) continue;
        works[i]->failed = true;
        status_clear(works[i]);
        cleared = true;
        if (first == QW4_OK) first = st;
    }
    if (cleared) qw4sh_stream_sync(stream);
    return first == QW4_OK ? report(err, QW4_OK, "") : first;
}

Qwen4Status qwen4_moe_forward(const Qwen4Moe *m, Qwen4F32 x, Qwen4F32Mut y, Qwen4MoeRoutes *routes,
                              Qwen4MoeWork *w, Qwen4Error *err) {
    if (!m || !w) return report(err, QW4_INVALID_ARGUMENT, "null forward handle");
    if (w->owner != m) return report(err, QW4_OWNER, "workspace belongs to another MoE");
    if (!m->alive || w->failed) return report(err, QW4_BAD_STATE, "inactive MoE/workspace; reset required");
    if (w->busy) return report(err, QW4_BUSY, "workspace executing");
    const size_t t = x.dim[0], h = m->c.hidden_size, k = m->c.top_k;
    if (t > w->cap) return report(err, QW4_CAPACITY, "batch exceeds token capacity");
    if (m->local_experts != m->c.experts) return report(err, QW4_BAD_STATE, "sharded handle: use the route/experts/combine calls");
    use_current_stream(w);
    Span spans[4]; size_t ns = 2;
    TRY(F32_SPAN("x", x, t, h, &spans[0], err));
    TRY(F32_SPAN("y", y, t, h, &spans[1], err));
    if (routes) {
        TRY(F32_SPAN("route weights", routes->weights, t, k, &spans[2], err));
        if (routes->ids.rows != t || routes->ids.cols != k) return raise(err, QW4_SHAPE, "route ids: want a [%zu, %zu] matrix", t, k);
        TRY(u32_span("route ids", routes->ids, &spans[3], err));
        ns = 4;
    }
    TRY(all_apart(spans, ns, err));
    for (size_t a = 0; a < 8; a++) {
        if (!m->host[a].span.data) continue;                        /* created from a file: no host bytes are borrowed */
        const Span weights = {(uintptr_t)m->host[a].span.data, (uintptr_t)m->host[a].span.data + m->host[a].layout.tensor_bytes};
        for (size_t b = 0; b < ns; b++)
            if (spans_meet(spans[b], weights)) return raise(err, QW4_INVALID_ARGUMENT, "argument %zu overlaps weight tensor %zu", b, a);
    }
    /* Nonfinite input is rejected before any state is touched (src/qwen4_moe.c:411-413). */
    for (size_t row = 0; row < t; row++) {
        const float *p = x.data + row * (x.stride_bytes[0] / 4);
        for (size_t col = 0; col < h; col++)
            if (!isfinite(p[col])) return report(err, QW4_NONFINITE, "nonfinite input");
    }
    if (!t) return report(err, QW4_OK, "");
    w->busy = true;
    Qwen4Status st = QW4_OK;
    const bool observe = w->observer != NULL;
    for (size_t start = 0; start < t && st == QW4_OK; start += w->chunk) {
        const size_t n = t - start < w->chunk ? t - start : w->chunk;
        const float *xs = x.data + start * (x.stride_bytes[0] / 4);
        float *ys = y.data + start * (y.stride_bytes[0] / 4);
        const size_t x_bytes = n * h * 4, r_bytes = n * k * 4;
        const bool small = 2 * x_bytes + 2 * r_bytes <= PIN_BYTES;
        float *pin_x = (float *)w->pin, *pin_y = (float *)(w->pin + x_bytes);
        uint32_t *pin_ids = (uint32_t *)(w->pin + 2 * x_bytes);
        float *pin_w = (float *)(w->pin + 2 * x_bytes + r_bytes);
        int rc = w->status_clean ? 0 : status_clear(w);
        w->status_clean = false;
        if (small) {
            for (size_t row = 0; row < n; row++) memcpy(pin_x + row * h, xs + row * (x.stride_bytes[0] / 4), h * 4);
            rc |= qw4sh_memcpy2d_async(w->d.x, h * 4, pin_x, h * 4, h * 4, n, 1, w->d.stream);
        } else rc |= qw4sh_memcpy2d_async(w->d.x, h * 4, xs, x.stride_bytes[0], h * 4, n, 1, w->d.stream);
        /* the one-kernel decode path writes each y element once and reads none: it stores straight into the pinned
         * staging (device-addressable), and the copy of y back drops out of the call */
        const bool direct_y = small && !observe && qw4sh_takes_fused(&m->layer, &w->d, w->d.x, pin_y, n);
        if (!rc && observe)                    /* stage by stage in the reference's order, every stage shown to the observer */
            rc = qw4sh_observed_forward(&m->layer, &w->d, w->d.x, w->d.y, n, xs, x.stride_bytes[0] / 4, start, w->observer, w->observer_ctx);
        else if (!rc) {
            if (direct_y) {                   /* the kernel also hands over the status words itself */
                w->status_host[0] = UINT32_MAX; w->status_host[1] = UINT32_MAX;
                w->d.status_mirror = w->status_host;
            }
            rc = qw4sh_layer_forward(&m->layer, &w->d, w->d.x, direct_y ? pin_y : w->d.y, n, NULL, NULL, current_router_mode());
            w->d.status_mirror = NULL;
        }
        if (!rc && !direct_y) rc = qw4sh_memcpy2d_async(w->status_host, 16, w->d.status, 16, 16, 1, 0, w->d.stream);
        if (!rc && small) {
            if (!direct_y) rc = qw4sh_memcpy2d_async(pin_y, h * 4, w->d.y, h * 4, h * 4, n, 0, w->d.stream);
            if (routes) {
                rc |= qw4sh_memcpy2d_async(pin_ids, k * 4, w->d.ids, k * 4, k * 4, n, 0, w->d.stream);
                rc |= qw4sh_memcpy2d_async(pin_w, k * 4, w->d.weights, k * 4, k * 4, n, 0, w->d.stream);
            }
        }
        if (!rc) rc = qw4sh_stream_sync(w->d.stream);
        if (!rc && direct_y && w->status_host[0] == UINT32_MAX)        /* the launch fell back to the multi-kernel sequence: fetch the words */
            rc = qw4sh_memcpy(w->status_host, w->d.status, 16, 0);
        if (rc) { st = cuda_failure(err, "layer execution"); break; }
        if ((st = status_result(w, err)) != QW4_OK) break;
        w->status_clean = true;
        if (small) {
            for (size_t row = 0; row < n; row++) {
                memcpy(ys + row * (y.stride_bytes[0] / 4), pin_y + row * h, h * 4);
                if (routes) {
                    memcpy(routes->ids.data + (start + row) * (routes->ids.row_stride_bytes / 4), pin_ids + row * k, k * 4);
                    memcpy(routes->weights.data + (start + row) * (routes->weights.stride_bytes[0] / 4), pin_w + row * k, k * 4);
                }
            }
        } else {
            rc = qw4sh_memcpy2d_async(ys, y.stride_bytes[0], w->d.y, h * 4, h * 4, n, 0, w->d.stream);
            if (routes) {
                rc |= qw4sh_memcpy2d_async(routes->ids.data + start * (routes->ids.row_stride_bytes / 4), routes->ids.row_stride_bytes,
                                           w->d.ids, k * 4, k * 4, n, 0, w->d.stream);
                rc |= qw4sh_memcpy2d_async(routes->weights.data + start * (routes->weights.stride_bytes[0] / 4),
                                           routes->weights.stride_bytes[0], w->d.weights, k * 4, k * 4, n, 0, w->d.stream);
            }
            if (!rc) rc = qw4sh_stream_sync(w->d.stream);
            if (rc) { st = cuda_failure(err, "result copy"); break; }
        }
    }
    w->busy = false;
    if (st != QW4_OK) { w->failed = true; return st; }
    return report(err, QW4_OK, "");
}

/* ---- pure routing ---------------------------------------------------------------------- */
/* Scratch of the two stateless entry points below.  They have no workspace argument, so the library keeps one device
 * block and one host block per device between calls and only ever grows them (up to SCRATCH_KEEP; a larger request
 * gets blocks of its own for that call): the reference's seeded route and grouping tests call these thousands of
 * times, and a device allocation per call costs more than the kernels.  One caller at a time per process: the lock
 * is held from scratch_take to scratch_give (the calls are synchronous anyway). */
#define SCRATCH_KEEP ((size_t)256 << 20)
static pthread_mutex_t g_scratch_lock = PTHREAD_MUTEX_INITIALIZER;
static struct { char *dev, *host; size_t dev_bytes, host_bytes; } g_scratch[64];
typedef struct { char *dev, *host; bool own; } Scratch;
static Scratch scratch_take(size_t dev_bytes, size_t host_bytes) {
    Scratch s = {NULL, NULL, false};
    const int device = qw4sh_current_device();
    if (device < 0 || device >= 64 || dev_bytes > SCRATCH_KEEP || host_bytes > SCRATCH_KEEP) {
        s.own = true; s.dev = qw4sh_malloc(dev_bytes); s.host = malloc(host_bytes);
        return s;
    }
    pthread_mutex_lock(&g_scratch_lock);
    if (g_scratch[device].dev_bytes < dev_bytes) {
        qw4sh_free(g_scratch[device].dev);
        g_scratch[device].dev = qw4sh_malloc(dev_bytes);
        g_scratch[device].dev_bytes = g_scratch[device].dev ? dev_bytes : 0;
    }
    if (g_scratch[device].host_bytes < host_bytes) {
        free(g_scratch[device].host);
        g_scratch[device].host = malloc(host_bytes);
        g_scratch[device].host_bytes = g_scratch[device].host ? host_bytes : 0;
    }
    s.dev = g_scratch[device].dev; s.host = g_scratch[device].host;
    return s;
}
static void scratch_give(Scratch s) {
    if (s.own) { qw4sh_free(s.dev); free(s.host); }
    else pthread_mutex_unlock(&g_scratch_lock);
}

Qwen4Status qwen4_moe_route(const Qwen4MoeConfig *c, Qwen4F32 logits, Qwen4MoeRoutes routes, Qwen4F32Mut probabilities,
                            Qwen4Error *err) {
    TRY(check_config(c, err));
    const size_t t = logits.dim[0], e = c->experts, k = c->top_k;
    Span spans[4];
    TRY(F32_SPAN("logits", logits, t, e, &spans[0], err));
    TRY(F32_SPAN("probabilities", probabilities, t, e, &spans[1], err));
    TRY(F32_SPAN("route weights", routes.weights, t, k, &spans[2], err));
    if (routes.ids.rows != t || routes.ids.cols != k) return raise(err, QW4_SHAPE, "route ids: want a [%zu, %zu] matrix", t, k);
    TRY(u32_span("route ids", routes.ids, &spans[3], err));
    TRY(all_apart(spans, 4, err));
    if (!t) return report(err, QW4_OK, "");
    if (t > UINT32_MAX / 2) return report(err, QW4_OVERFLOW, "too many rows");
    const size_t ze = t * e * 4, zk = t * k * 4;
    const Scratch scratch = scratch_take(2 * ze + 2 * zk + 64, ze + 2 * zk + 64);
    char *dev = scratch.dev, *host = scratch.host;
    Qwen4Status st = QW4_OK;
    if (!dev || !host) { st = dev ? report(err, QW4_OOM, "route scratch") : cuda_failure(err, "route scratch"); goto done; }
    float *d_logits = (float *)dev, *d_probs = (float *)(dev + ze), *d_w = (float *)(dev + 2 * ze + zk);
    uint32_t *d_ids = (uint32_t *)(dev + 2 * ze), *d_status = (uint32_t *)(dev + 2 * ze + 2 * zk);
    uint32_t status[4] = {0, UINT32_MAX, 0, 0};
    int rc = qw4sh_memcpy(d_status, status, 16, 1);
    rc |= qw4sh_memcpy2d_async(d_logits, e * 4, logits.data, logits.stride_bytes[0], e * 4, t, 1, NULL);
    if (!rc) rc = qw4sh_route(c->experts, c->top_k, c->norm_topk_prob, d_logits, e, t, d_probs, d_ids, d_w, d_status, NULL);
    if (!rc) rc = qw4sh_stream_sync(NULL);
    if (!rc) rc = qw4sh_memcpy(status, d_status, 16, 0);
    if (rc) { st = cuda_failure(err, "route"); goto done; }
    if (status[0] & QW4SH_ERR_NONFINITE) {
        st = report(err, QW4_NONFINITE, "nonfinite router logit");
        if (err) err->row = status[1];
        goto done;
    }
    float *h_probs = (float *)host, *h_w = (float *)(host + ze + zk);
    uint32_t *h_ids = (uint32_t *)(host + ze);
    if (qw4sh_memcpy(h_probs, d_probs, ze, 0) || qw4sh_memcpy(h_ids, d_ids, zk, 0) || qw4sh_memcpy(h_w, d_w, zk, 0)) {
        st = cuda_failure(err, "route readback"); goto done;
    }
    for (size_t row = 0; row < t; row++) {
        memcpy(probabilities.data + row * (probabilities.stride_bytes[0] / 4), h_probs + row * e, e * 4);
        memcpy(routes.ids.data + row * (routes.ids.row_stride_bytes / 4), h_ids + row * k, k * 4);
        memcpy(routes.weights.data + row * (routes.weights.stride_bytes[0] / 4), h_w + row * k, k * 4);
    }
    st = report(err, QW4_OK, "");
done:
    scratch_give(scratch);
    return st;
}

/* ---- dispatch lists --------------------------------------------------------------------- */
Qwen4Status qw4_moe_group_pairs(const Qwen4MoeConfig *c, Qwen4U32Mut ids, QW4MoeGrouping g, Qwen4Error *err) {
    TRY(check_config(c, err));
    if (ids.cols != c->top_k) return report(err, QW4_SHAPE, "group ID shape mismatch");
    const size_t e = c->experts, k = c->top_k;
    if (ids.rows > SIZE_MAX / k || e == SIZE_MAX) return report(err, QW4_OVERFLOW, "group count overflow");
    const size_t pairs = ids.rows * k;
    Span spans[5];
    TRY(u32_span("ids", ids, &spans[0], err));
    const Region lists[4] = {
        {"offsets", g.offsets, g.offsets_capacity_bytes, 1, e + 1, 0, sizeof(size_t)},
        {"cursors", g.cursors, g.cursors_capacity_bytes, 1, e, 0, sizeof(size_t)},
        {"pair_to_row", g.pair_to_row, g.pair_to_row_capacity_bytes, 1, pairs, 0, sizeof(size_t)},
        {"row_to_pair", g.row_to_pair, g.row_to_pair_capacity_bytes, 1, pairs, 0, sizeof(size_t)}};
    for (size_t a = 0; a < 4; a++) {
        Region r = lists[a];
        if (r.cols > SIZE_MAX / r.elem) return raise(err, QW4_OVERFLOW, "%s: byte count does not fit size_t", r.name);
        r.pitch = r.cols * r.elem;                          /* one dense row */
        TRY(region_span(&r, &spans[a + 1], err));
    }
    TRY(all_apart(spans, 5, err));
    for (size_t t = 0; t < ids.rows; t++) {
        const uint32_t *row = ids.data + t * (ids.row_stride_bytes / 4);
        for (size_t s = 0; s < k; s++) {
            if (row[s] >= e) return report(err, QW4_RANGE, "expert ID out of range");
            for (size_t j = 0; j < s; j++)
                if (row[j] == row[s]) return report(err, QW4_INVALID_ARGUMENT, "duplicate expert ID");
        }
    }
    if (pairs > UINT32_MAX / 2) return report(err, QW4_OVERFLOW, "too many pairs");
    const size_t zp = pairs * 4, ze = (e + 1) * 4;
    const Scratch scratch = scratch_take(3 * zp + 2 * ze + 64 + 16, 3 * zp + ze + 64);
    char *dev = scratch.dev;
    uint32_t *host = (uint32_t *)scratch.host;
    Qwen4Status st = QW4_OK;
    if (!dev || !host) { st = dev ? report(err, QW4_OOM, "group scratch") : cuda_failure(err, "group scratch"); goto done; }
    uint32_t *d_ids = (uint32_t *)dev, *d_p2r = (uint32_t *)(dev + zp), *d_r2p = (uint32_t *)(dev + 2 * zp);
    uint32_t *d_off = (uint32_t *)(dev + 3 * zp), *d_active = (uint32_t *)(dev + 3 * zp + ze);
    uint32_t *d_status = (uint32_t *)(dev + 3 * zp + 2 * ze + 16);
    uint32_t status[4] = {0, 0, 0, 0};
    int rc = qw4sh_memcpy(d_status, status, 16, 1);
    if (pairs) rc |= qw4sh_memcpy2d_async(d_ids, k * 4, ids.data, ids.row_stride_bytes, k * 4, ids.rows, 1, NULL);
    if (!rc) rc = qw4sh_group(c->experts, c->top_k, ids.rows, d_ids, d_off, d_p2r, d_r2p, d_active, d_status, NULL);
    if (!rc) rc = qw4sh_stream_sync(NULL);
    uint32_t *h_off = host, *h_p2r = host + (e + 1), *h_r2p = host + (e + 1) + pairs;
    if (!rc) rc = qw4sh_memcpy(h_off, d_off, ze, 0);
    if (!rc && pairs) rc = qw4sh_memcpy(h_p2r, d_p2r, zp, 0) | qw4sh_memcpy(h_r2p, d_r2p, zp, 0);
    if (rc) { st = cuda_failure(err, "group"); goto done; }
    for (size_t j = 0; j <= e; j++) g.offsets[j] = h_off[j];
    for (size_t j = 0; j < e; j++) g.cursors[j] = h_off[j + 1];
    for (size_t j = 0; j < pairs; j++) { g.pair_to_row[j] = h_p2r[j]; g.row_to_pair[j] = h_r2p[j]; }
    st = report(err, QW4_OK, "");
done:
    scratch_give(scratch);
    return st;
}

/* ---- probes and plumbing ---------------------------------------------------------------- */
static Qwen4Status decode_rows_from(const Qwen4Moe *m, uint32_t tensor, size_t expert, size_t row0, size_t rows, float *out,
                                    size_t out_elements, bool expanded, Qwen4Error *err);
Qwen4Status qw4cu_moe_decode_rows(const Qwen4Moe *m, uint32_t tensor, size_t expert, size_t row0, size_t rows, float *out,
                                  size_t out_elements, Qwen4Error *err) {
    return decode_rows_from(m, tensor, expert, row0, rows, out, out_elements, false, err);
}
Qwen4Status qw4cu_moe_decode_rows_expanded(const Qwen4Moe *m, uint32_t tensor, size_t expert, size_t row0, size_t rows, float *out,
                                           size_t out_elements, Qwen4Error *err) {
    return decode_rows_from(m, tensor, expert, row0, rows, out, out_elements, true, err);
}
static Qwen4Status decode_rows_from(const Qwen4Moe *m, uint32_t tensor, size_t expert, size_t row0, size_t rows, float *out,
                                    size_t out_elements, bool expanded, Qwen4Error *err) {
    if (!m || !m->alive) return report(err, QW4_BAD_STATE, "inactive MoE");
    if (tensor >= 8 || !out) return report(err, QW4_INVALID_ARGUMENT, "bad tensor index or output");
    const QW4ShTensor *t = &m->layer.w[tensor];
    if (expert >= t->n_experts || row0 > t->n_out || rows > t->n_out - row0) return report(err, QW4_RANGE, "row outside tensor");
    if (out_elements / t->k_storage < rows) return report(err, QW4_CAPACITY, "short output");
    if (!rows) return report(err, QW4_OK, "");
    const size_t bytes = rows * (size_t)t->k_storage * 4;
    float *dev = qw4sh_malloc(bytes);
    if (!dev) return cuda_failure(err, "decode scratch");
    int rc = expanded ? qw4sh_fused_decode_rows_expanded(&m->layer, (int)tensor, expert, row0, rows, dev, NULL)
                      : qw4sh_decode_rows(t, expert, row0, rows, dev, NULL);
    if (rc == -3) { qw4sh_free(dev); return report(err, QW4_UNSUPPORTED, "this tensor has no expanded image"); }
    if (!rc) rc = qw4sh_stream_sync(NULL);
    if (!rc) rc = qw4sh_memcpy(out, dev, bytes, 0);
    qw4sh_free(dev);
    if (rc) return cuda_failure(err, "decode");
    for (size_t i = 0; i < rows * (size_t)t->k_storage; i++)
        if (!isfinite(out[i])) return report(err, QW4_NONFINITE, "nonfinite packed value");
    return report(err, QW4_OK, "");
}

int qw4cu_device_count(void) { return qw4sh_device_count(); }
int qw4cu_set_device(int device) { return qw4sh_set_device(device); }
const char *qw4cu_last_error(void) { return qw4sh_last_error(); }
uint64_t qw4cu_launch_count(void) { return qw4sh_launch_count(); }
void qw4cu_launch_log_begin(void) { qw4sh_launch_log_begin(); }
size_t qw4cu_launch_log(char *out, size_t cap) { return qw4sh_launch_log(out, cap); }
void *qw4cu_malloc(size_t bytes) { return qw4sh_malloc(bytes); }
void qw4cu_free(void *p) { qw4sh_free(p); }
void *qw4cu_host_alloc(size_t bytes) { return qw4sh_host_alloc(bytes); }
void qw4cu_host_free(void *p) { qw4sh_host_free(p); }
int qw4cu_upload(void *dst, const void *src, size_t bytes) { return qw4sh_memcpy(dst, src, bytes, 1); }
int qw4cu_download(void *dst, const void *src, size_t bytes) { return qw4sh_memcpy(dst, src, bytes, 0); }
int qw4cu_flush_l2(void) { return qw4sh_flush_l2(); }
int qw4cu_mem_info(size_t *free_bytes, size_t *total_bytes) { return qw4sh_mem_info(free_bytes, total_bytes); }
int qw4cu_device_synchronize(void) { return qw4sh_device_sync(); }
void qw4cu_set_graph_mode(int on) { qw4sh_set_graph_mode(on); }
int qw4cu_get_graph_mode(void) { return qw4sh_get_graph_mode(); }
void qw4cu_set_stage_timing(int on) { qw4sh_set_stage_timing(on); }
void qw4cu_set_expert_path(int path) { qw4sh_set_expert_path(path); }
void qw4cu_set_only_step(int step) { qw4sh_set_only_step(step); }
void qw4cu_set_fused_decode(int mode) { qw4sh_set_fused_decode(mode); }
void qw4cu_set_prefill_path(int path) { qw4sh_set_prefill_path(path); }
void qw4cu_set_tile_path(int path) { qw4sh_set_tile_path(path); }
void qw4cu_prefill_debug(void *device_words) { qw4sh_prefill_debug(device_words); }
int qw4cu_decode_phase_clocks(const Qwen4MoeWork *w, uint64_t clocks[16]) { return w ? qw4sh_fused_phase_clocks(&w->d, clocks) : -1; }
void qw4cu_set_decode_wrong_speculation(int on) { qw4sh_set_wrong_speculation(on); }
int qw4cu_decode_debug_words(const Qwen4MoeWork *w, uint32_t *out, size_t words) { return w && out && words <= 1024 ? qw4sh_memcpy(out, w->d.sync, words * 4, 0) : -1; }
int qw4cu_decode_repairs(const Qwen4MoeWork *w, uint32_t *count) { return w && count ? qw4sh_fused_repairs(&w->d, count) : -1; }
int qw4cu_stage_times(double *ms, uint64_t *forwards) { return qw4sh_stage_times(ms, forwards); }
int qw4cu_moe_work_timer_begin(Qwen4MoeWork *w) { return w ? qw4sh_event_record(w->d.timer[0], w->d.stream) : -1; }
int qw4cu_moe_work_timer_end(Qwen4MoeWork *w) { return w ? qw4sh_event_record(w->d.timer[1], w->d.stream) : -1; }
float qw4cu_moe_work_timer_elapsed_ms(Qwen4MoeWork *w) { return w ? qw4sh_event_elapsed_ms(w->d.timer[0], w->d.timer[1]) : -1.0f; }
