/* The caller of the four-token decode batch: speculative verify over a stack of MoE layers, with the route log.
 *
 * picoforge's GPU forward appends one confirmed token plus up to three drafts as ONE batch of 1..4 rows
 * (qwen4_gpu_forward_verify, src/qwen4_forward_gpu.h:55-63, QWEN4_VERIFY_ROWS = 4) and then keeps the first n
 * rows (qwen4_gpu_forward_keep).  The MoE layer carries no state from token to token, so what verify asks of
 * this layer is exactly a 1..4-row forward per layer, and keep is bookkeeping of the position.  What the layer
 * adds to the caller's records is the route log (src/qwen4_forward_gpu.m:896-899): per append a header of four
 * uint32 {position, rows, layers, top_k}, then the expert ids [layer][row][top_k] as uint32.
 *
 * The stack here stands in for the engine's layer loop: layer l reads what layer l - 1 wrote (the engine puts
 * attention and the hyper-connection mix in between; they are not part of this library).  All layers are
 * enqueued back to back on the library's stream (the one-kernel decode path chains them by programmatic stream
 * serialisation); one host wait per append.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/qwen4_moe_b200.h"
#include "cuda_shim.h"

enum { VERIFY_ROWS = 4 };

struct QW4CuVerify {
    size_t layers, hidden, top_k;
    Qwen4Moe **moe;                     /* borrowed */
    Qwen4MoeWork **work;                /* owned, one per layer: consecutive layers overlap at their edges */
    float *act[2];                      /* device [VERIFY_ROWS, hidden] ping-pong */
    uint32_t *ids_dev;                  /* device [layers][VERIFY_ROWS][top_k] */
    unsigned char *pin;                 /* pinned: x | y | ids */
    uint64_t position;
    size_t pending;                     /* rows of an append that keep has not settled yet */
    FILE *log;
};

static Qwen4Status verify_fail(Qwen4Error *err, Qwen4Status code, const char *detail) {
    if (err) {
        memset(err, 0, sizeof *err);
        err->code = code;
        snprintf(err->subject, sizeof err->subject, "verify");
        snprintf(err->detail, sizeof err->detail, "%s", detail);
    }
    return code;
}

void qw4cu_verify_destroy(QW4CuVerify *v) {
    if (!v) return;
    if (v->log) fclose(v->log);
    for (size_t l = 0; v->work && l < v->layers; l++) qwen4_moe_work_destroy(v->work[l]);
    qw4sh_free(v->act[0]); qw4sh_free(v->act[1]); qw4sh_free(v->ids_dev);
    qw4sh_host_free(v->pin);
    free(v->work); free(v->moe); free(v);
}

Qwen4Status qw4cu_verify_create(Qwen4Moe *const *layers, size_t n_layers, const Qwen4MoeConfig *config, QW4CuVerify **out, Qwen4Error *err) {
    if (out) *out = NULL;
    if (!out || !layers || !config || !n_layers || n_layers > 4096) return verify_fail(err, QW4_INVALID_ARGUMENT, "null or empty layer list");
    QW4CuVerify *v = calloc(1, sizeof *v);
    if (!v) return verify_fail(err, QW4_OOM, "verify handle");
    v->layers = n_layers; v->hidden = config->hidden_size; v->top_k = config->top_k;
    v->moe = calloc(n_layers, sizeof *v->moe);
    v->work = calloc(n_layers, sizeof *v->work);
    if (!v->moe || !v->work) { qw4cu_verify_destroy(v); return verify_fail(err, QW4_OOM, "verify handle"); }
    for (size_t l = 0; l < n_layers; l++) {
        size_t bytes = 0;
        v->moe[l] = layers[l];
        Qwen4Status st = qwen4_moe_work_size(layers[l], VERIFY_ROWS, &bytes, err);
        if (st == QW4_OK) st = qwen4_moe_work_create(layers[l], VERIFY_ROWS, bytes, &v->work[l], err);
        if (st != QW4_OK) { qw4cu_verify_destroy(v); return st; }
    }
    const size_t row = v->hidden * sizeof(float), ids = n_layers * VERIFY_ROWS * v->top_k * sizeof(uint32_t);
    v->act[0] = qw4sh_malloc(VERIFY_ROWS * row);
    v->act[1] = qw4sh_malloc(VERIFY_ROWS * row);
    v->ids_dev = qw4sh_malloc(ids);
    v->pin = qw4sh_host_alloc(2 * VERIFY_ROWS * row + ids);
    if (!v->act[0] || !v->act[1] || !v->ids_dev || !v->pin) { qw4cu_verify_destroy(v); return verify_fail(err, QW4_GPU_ERROR, "verify buffers"); }
    *out = v;
    if (err) memset(err, 0, sizeof *err);
    return QW4_OK;
}

/* path NULL: stop logging.  The file is truncated; records are flushed after every append. */
Qwen4Status qw4cu_verify_route_log(QW4CuVerify *v, const char *path, Qwen4Error *err) {
    if (!v) return verify_fail(err, QW4_INVALID_ARGUMENT, "null verify handle");
    if (v->log) { fclose(v->log); v->log = NULL; }
    if (path && !(v->log = fopen(path, "wb"))) return verify_fail(err, QW4_IO, "route log cannot be opened");
    if (err) memset(err, 0, sizeof *err);
    return QW4_OK;
}

uint64_t qw4cu_verify_position(const QW4CuVerify *v) { return v ? v->position : 0; }
size_t qw4cu_verify_pending(const QW4CuVerify *v) { return v ? v->pending : 0; }

/* x_host, y_host: dense [count, hidden] FP32; ids_host (may be NULL): [layers][count][top_k].  count 1..4.  A verify
 * that is still pending is settled first as if all of its rows had been kept (an ordinary append ends it). */
Qwen4Status qw4cu_verify_append(QW4CuVerify *v, const float *x_host, size_t count, float *y_host, uint32_t *ids_host, Qwen4Error *err) {
    if (!v || !x_host || !y_host) return verify_fail(err, QW4_INVALID_ARGUMENT, "null verify argument");
    if (!count || count > VERIFY_ROWS) return verify_fail(err, QW4_CAPACITY, "a verify append holds 1 to 4 rows");
    if (v->pending) { v->position += v->pending; v->pending = 0; }
    const size_t row = v->hidden * sizeof(float), k = v->top_k, ids_bytes = v->layers * count * k * sizeof(uint32_t);
    float *pin_x = (float *)v->pin, *pin_y = (float *)(v->pin + VERIFY_ROWS * row);
    uint32_t *pin_ids = (uint32_t *)(v->pin + 2 * VERIFY_ROWS * row);
    void *stream = NULL;
    if (qw4sh_current_stream(&stream)) return verify_fail(err, QW4_GPU_ERROR, "no stream");
    memcpy(pin_x, x_host, count * row);
    if (qw4sh_memcpy2d_async(v->act[0], count * row, pin_x, count * row, count * row, 1, 1, stream)) return verify_fail(err, QW4_GPU_ERROR, "input copy");
    for (size_t l = 0; l < v->layers; l++) {
        const Qwen4Status st = qw4cu_moe_forward_device(v->moe[l], v->act[l & 1], v->act[(l + 1) & 1], count, v->ids_dev + l * count * k, NULL,
                                                        v->work[l], err);
        if (st != QW4_OK) return st;
    }
    if (qw4sh_memcpy2d_async(pin_y, count * row, v->act[v->layers & 1], count * row, count * row, 1, 0, stream) ||
        qw4sh_memcpy2d_async(pin_ids, ids_bytes, v->ids_dev, ids_bytes, ids_bytes, 1, 0, stream))
        return verify_fail(err, QW4_GPU_ERROR, "output copy");
    /* every workspace reports its own kernels' error words: all fetched behind the copies, one wait for everything */
    {
        const Qwen4Status st = qw4cu_moe_work_sync_many(v->work, v->layers, err);
        if (st != QW4_OK) return st;
    }
    memcpy(y_host, pin_y, count * row);
    if (ids_host) memcpy(ids_host, pin_ids, ids_bytes);
    if (v->log) {
        const uint32_t head[4] = {(uint32_t)v->position, (uint32_t)count, (uint32_t)v->layers, (uint32_t)k};
        if (fwrite(head, 4, 4, v->log) != 4 || fwrite(pin_ids, 4, v->layers * count * k, v->log) != v->layers * count * k || fflush(v->log))
            return verify_fail(err, QW4_IO, "route log write");
    }
    v->pending = count;
    if (err) memset(err, 0, sizeof *err);
    return QW4_OK;
}

/* Keeps the first `keep` rows (1..rows of the pending append) and drops the rest: the position advances by keep. */
Qwen4Status qw4cu_verify_keep(QW4CuVerify *v, size_t keep, Qwen4Error *err) {
    if (!v) return verify_fail(err, QW4_INVALID_ARGUMENT, "null verify handle");
    if (!v->pending) return verify_fail(err, QW4_BAD_STATE, "no verify is pending");
    if (!keep || keep > v->pending) return verify_fail(err, QW4_RANGE, "keep 1 to the rows of the pending append");
    v->position += keep;
    v->pending = 0;
    if (err) memset(err, 0, sizeof *err);
    return QW4_OK;
}
