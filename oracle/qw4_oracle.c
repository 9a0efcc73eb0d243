/* CPU oracle for the Qwen4 MoE layer.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C11, the arithmetic of picoforge's CPU MoE path so that
 * the CUDA kernels can be checked against it.  It is linked by tests/, by the smoke
 * check and by the CPU-baseline leg of bench.py, and by nothing that ships: the product
 * library never calls into it and has no CPU fallback.
 *
 * Parity is PINNED: tests/test_oracle_vs_reference.py compares every function below with
 * the reference's own objects built from its sources (oracle/Makefile, target `ref`), and
 * tests/golden/ holds vectors generated from those objects for machines without them.
 *
 * Build with -ffp-contract=off: every product and every sum below is a separately
 * rounded binary32 operation, as in the reference (picoforge src/qwen4_packed.c:3,
 * tools/qwen4.mk:6).
 *
 * Each function names the reference lines it follows.
 */
#include <math.h>
#include <pthread.h>
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../picoforge_b200/csrc/iq2xxs_codebook.h"


enum { O_OK = 0, O_INVALID = 1, O_RANGE = 4, O_FORMAT = 7, O_OOM = 11, O_NONFINITE = 16 };

/* ------------------------------------------------------------------------------------
 * Block formats.  Follows picoforge src/gguf.c:13-17 (block table) and
 * src/qwen4_packed.c:51-122 (half_value, packed_value).
 * ---------------------------------------------------------------------------------- */

static bool format_of(uint32_t type, size_t *block, size_t *bytes) {
    switch (type) {
    case 0:  *block = 1;   *bytes = 4;   return true;   /* F32 */
    case 1:  *block = 1;   *bytes = 2;   return true;   /* F16 */
    case 8:  *block = 32;  *bytes = 34;  return true;   /* Q8_0 */
    case 10: *block = 256; *bytes = 84;  return true;   /* Q2_K */
    case 12: *block = 256; *bytes = 144; return true;   /* Q4_K */
    case 16: *block = 256; *bytes = 66;  return true;   /* IQ2_XXS */
    case 30: *block = 1;   *bytes = 2;   return true;   /* BF16 */
    case 39: *block = 32;  *bytes = 17;  return true;   /* MXFP4 */
    default: return false;
    }
}

/* Bytes of one row of k_storage weights, or 0 for an unknown type / incomplete block. */
size_t qw4o_row_bytes(uint32_t type, size_t k_storage) {
    size_t block, bytes;
    if (!format_of(type, &block, &bytes) || k_storage % block) return 0;
    return k_storage / block * bytes;
}

static float bits_to_float(uint32_t bits) {
    float value;
    memcpy(&value, &bits, sizeof value);
    return value;
}

/* binary16 -> binary32, exact, including subnormals, infinities and NaN payloads
 * (src/qwen4_packed.c:54-66). */
static float half_at(const uint8_t *p) {
    uint32_t h = (uint32_t)p[0] | (uint32_t)p[1] << 8;
    uint32_t sign = (h & 0x8000u) << 16, exponent = (h >> 10) & 31u, fraction = h & 1023u;
    if (exponent == 0) {
        if (fraction == 0) return bits_to_float(sign);
        uint32_t e = 113;
        while (!(fraction & 1024u)) { fraction <<= 1; e--; }
        return bits_to_float(sign | e << 23 | (fraction & 1023u) << 13);
    }
    uint32_t e32 = exponent == 31 ? 255u : exponent + 112u;
    return bits_to_float(sign | e32 << 23 | fraction << 13);
}

static void block_q4_k(const uint8_t *b, float *out) {           /* src/qwen4_packed.c:86-93 */
    const float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t *sc = b + 4, *codes = b + 16;
    for (unsigned g = 0; g < 8; g++) {
        unsigned scale, minimum;
        if (g < 4) { scale = sc[g] & 63u; minimum = sc[g + 4] & 63u; }
        else {
            scale = (sc[g + 4] & 15u) | ((sc[g - 4] & 192u) >> 2);
            minimum = (unsigned)(sc[g + 4] >> 4) | ((sc[g] & 192u) >> 2);
        }
        const float dl = d * (float)scale, ml = dmin * (float)minimum;
        const uint8_t *q = codes + (g / 2) * 32;
        const unsigned shift = (g % 2) * 4;
        for (unsigned j = 0; j < 32; j++)
            out[g * 32 + j] = dl * (float)((q[j] >> shift) & 15u) - ml;
    }
}

static void block_q2_k(const uint8_t *b, float *out) {           /* src/qwen4_packed.c:116-121 */
    const float d = half_at(b + 80), dmin = half_at(b + 82);
    for (unsigned lane = 0; lane < 256; lane++) {
        const unsigned s = b[lane / 16];
        const unsigned code = (b[16 + lane / 128 * 32 + lane % 32] >> (2 * (lane % 128 / 32))) & 3u;
        out[lane] = (d * (float)(s & 15u)) * (float)code - dmin * (float)(s >> 4);
    }
}

static void block_iq2_xxs(const uint8_t *b, float *out) {        /* src/qwen4_packed.c:102-115 */
    const float d = half_at(b);
    for (unsigned g = 0; g < 8; g++) {
        const uint8_t *group = b + 2 + 8 * g;
        const uint32_t bits = (uint32_t)group[4] | (uint32_t)group[5] << 8 |
                              (uint32_t)group[6] << 16 | (uint32_t)group[7] << 24;
        const float scale = d * (float)(2 * (bits >> 28) + 1) * 0.125f;
        for (unsigned slot = 0; slot < 4; slot++) {
            unsigned signs = (bits >> (7 * slot)) & 127u, parity = signs;
            parity ^= parity >> 4; parity ^= parity >> 2; parity ^= parity >> 1;
            signs |= (parity & 1u) << 7;
            const unsigned levels = QW4_IQ2XXS_LEVELS[group[slot]];
            for (unsigned j = 0; j < 8; j++) {
                const unsigned level = (levels >> (2 * j)) & 3u;
                const float value = scale * (float)QW4_IQ2XXS_MAGNITUDE(level);
                out[g * 32 + slot * 8 + j] = (signs >> j) & 1u ? -value : value;
            }
        }
    }
}

static void block_q8_0(const uint8_t *b, float *out) {           /* src/qwen4_packed.c:80-85 */
    const float d = half_at(b);
    for (unsigned j = 0; j < 32; j++) {
        int code = b[2 + j];
        if (code >= 128) code -= 256;
        out[j] = d * (float)code;
    }
}

static void block_mxfp4(const uint8_t *b, float *out) {          /* src/qwen4_packed.c:94-101 */
    static const float e2m1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                   -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
    const float scale = bits_to_float(b[0] ? (uint32_t)b[0] << 23 : 0x00400000u);
    for (unsigned lane = 0; lane < 32; lane++)
        out[lane] = e2m1[(b[1 + lane % 16] >> ((lane / 16) * 4)) & 15u] * scale;
}

/* Decodes one packed row into k_storage floats.  Returns O_NONFINITE if any decoded value
 * is not finite (src/qwen4_packed.c:124-143), after writing the whole row. */
int qw4o_decode_row(uint32_t type, const uint8_t *row, size_t k_storage, float *out) {
    size_t block, bytes;
    if (!format_of(type, &block, &bytes) || k_storage % block) return O_FORMAT;
    const size_t blocks = k_storage / block;
    for (size_t i = 0; i < blocks; i++) {
        const uint8_t *b = row + i * bytes;
        float *o = out + i * block;
        switch (type) {
        case 0:  *o = bits_to_float((uint32_t)b[0] | (uint32_t)b[1] << 8 |
                                    (uint32_t)b[2] << 16 | (uint32_t)b[3] << 24); break;
        case 1:  *o = half_at(b); break;
        case 30: *o = bits_to_float(((uint32_t)b[0] | (uint32_t)b[1] << 8) << 16); break;
        case 8:  block_q8_0(b, o); break;
        case 10: block_q2_k(b, o); break;
        case 12: block_q4_k(b, o); break;
        case 16: block_iq2_xxs(b, o); break;
        default: block_mxfp4(b, o); break;
        }
    }
    for (size_t k = 0; k < k_storage; k++) if (!isfinite(out[k])) return O_NONFINITE;
    return O_OK;
}

/* y[n] = sum over k < k_logical of w[n][k] * x[k], k ascending, product and sum rounded
 * separately; any nonfinite weight, input, product or partial sum is an error
 * (src/qwen4_packed.c:164-178). */
static int dot_serial(const float *w, const float *x, size_t k_logical, float *out) {
    float sum = 0.0f;
    bool bad = false;
    for (size_t k = 0; k < k_logical; k++) {
        const float product = w[k] * x[k];
        sum += product;
        bad |= !isfinite(w[k]) | !isfinite(x[k]) | !isfinite(product) | !isfinite(sum);
    }
    *out = sum;
    return bad ? O_NONFINITE : O_OK;
}

/* y[m][n] for one expert's matrix: weights at `w` ([n_out] rows of row_bytes), x [m_rows]
 * rows with x_pitch floats between rows, y likewise.  Same contract as the reference's
 * packed matmul for one expert (src/qwen4_packed.c:145-180). */
int qw4o_matmul(uint32_t type, const uint8_t *w, size_t k_storage, size_t k_logical,
                size_t n_out, const float *x, size_t x_pitch, size_t m_rows,
                float *y, size_t y_pitch) {
    const size_t row_bytes = qw4o_row_bytes(type, k_storage);
    if (!row_bytes || k_logical > k_storage) return O_FORMAT;
    float *decoded = malloc(k_storage * sizeof *decoded);
    if (!decoded) return O_OOM;
    int status = O_OK;
    for (size_t n = 0; n < n_out && m_rows; n++) {
        qw4o_decode_row(type, w + n * row_bytes, k_storage, decoded);
        for (size_t m = 0; m < m_rows; m++)
            if (dot_serial(decoded, x + m * x_pitch, k_logical, y + m * y_pitch + n)) status = O_NONFINITE;
    }
    free(decoded);
    return status;
}

/* ------------------------------------------------------------------------------------
 * Activations (picoforge src/qwen4_cpu_internal.h:103-107, src/qwen4_base.c:76-99).
 * ---------------------------------------------------------------------------------- */
static float sigmoid_f32(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}
float qw4o_sigmoid(float x) { return sigmoid_f32(x); }
float qw4o_silu(float x) { return x * sigmoid_f32(x); }

/* ------------------------------------------------------------------------------------
 * Router (picoforge src/qwen4_moe.c:188-249).
 * logits [tokens][experts] with `pitch` floats between rows.  Outputs are dense:
 * probs [tokens][experts], ids and weights [tokens][k].  A nonfinite logit anywhere
 * returns O_NONFINITE with *bad_row set and writes nothing.
 * ---------------------------------------------------------------------------------- */
int qw4o_route(uint32_t experts, uint32_t k, int norm, const float *logits, size_t pitch,
               size_t tokens, float *probs, uint32_t *ids, float *weights, uint64_t *bad_row) {
    if (!experts || !k || k > experts) return O_RANGE;
    for (size_t t = 0; t < tokens; t++)
        for (size_t e = 0; e < experts; e++)
            if (!isfinite(logits[t * pitch + e])) { if (bad_row) *bad_row = t; return O_NONFINITE; }
    for (size_t t = 0; t < tokens; t++) {
        const float *z = logits + t * pitch;
        float *p = probs + t * experts, *w = weights + t * k;
        uint32_t *id = ids + t * k;
        float maximum = z[0], sum = 0.0f;
        for (size_t e = 1; e < experts; e++) if (z[e] > maximum) maximum = z[e];
        for (size_t e = 0; e < experts; e++) { p[e] = expf(z[e] - maximum); sum += p[e]; }
        for (size_t e = 0; e < experts; e++) p[e] /= sum;
        float selected = 0.0f;
        for (size_t slot = 0; slot < k; slot++) {
            size_t best = 0;
            bool found = false;
            for (size_t e = 0; e < experts; e++) {
                bool used = false;
                for (size_t j = 0; j < slot; j++) used |= id[j] == e;
                if (!used && (!found || p[e] > p[best])) { best = e; found = true; }
            }
            id[slot] = (uint32_t)best;
            w[slot] = p[best];
            selected += w[slot];
        }
        if (norm) for (size_t slot = 0; slot < k; slot++) w[slot] /= selected;
    }
    return O_OK;
}

/* ------------------------------------------------------------------------------------
 * Dispatch lists (picoforge src/qwen4_moe.c:251-303; contract
 * src/qwen4_moe_internal.h:78-95): stable counting sort of pair = t*k + slot by expert.
 * ---------------------------------------------------------------------------------- */
int qw4o_group(uint32_t experts, uint32_t k, size_t tokens, const uint32_t *ids,
               uint64_t *offsets, uint64_t *pair_to_row, uint64_t *row_to_pair) {
    for (size_t t = 0; t < tokens; t++)
        for (size_t s = 0; s < k; s++) {
            if (ids[t * k + s] >= experts) return O_RANGE;
            for (size_t j = 0; j < s; j++) if (ids[t * k + j] == ids[t * k + s]) return O_INVALID;
        }
    uint64_t *cursor = malloc(((size_t)experts + 1) * sizeof *cursor);
    if (!cursor) return O_OOM;
    memset(offsets, 0, ((size_t)experts + 1) * sizeof *offsets);
    for (size_t p = 0; p < tokens * k; p++) offsets[ids[p] + 1]++;
    for (size_t e = 0; e < experts; e++) { offsets[e + 1] += offsets[e]; cursor[e] = offsets[e]; }
    for (size_t p = 0; p < tokens * k; p++) {
        const uint64_t row = cursor[ids[p]]++;
        pair_to_row[p] = row;
        row_to_pair[row] = p;
    }
    free(cursor);
    return O_OK;
}

/* ------------------------------------------------------------------------------------
 * Whole layer (picoforge src/qwen4_moe.c:318-382): router product, route, per-expert
 * SwiGLU, shared expert with sigmoid gate, slot-order weighted sum.  Token results do not
 * depend on how tokens are batched, so the reference's 32-token microbatching
 * (src/qwen4_moe.c:83,415-416) is not reproduced; experts are evaluated group by group so
 * that each packed row is decoded once.
 * ---------------------------------------------------------------------------------- */
typedef struct {
    uint32_t type;
    const uint8_t *data;
} QW4OTensor;

typedef struct {
    uint32_t hidden, experts, k, inter, shared_inter, down_physical;
    int norm;
    QW4OTensor w[8];              /* router, gate, up, down, sgate, sup, sdown, srouter */
} QW4OLayer;

typedef struct {
    const QW4OLayer *layer;
    const float *x;               /* dense [tokens][hidden] */
    size_t tokens;
    const uint32_t *ids;
    const uint64_t *offsets, *row_to_pair;
    float *down;                  /* [pairs][hidden], grouped-row order */
    float *shared;                /* [tokens][hidden] */
    float *logits;                /* [tokens][experts] */
    float *shared_logit;          /* [tokens] */
    size_t next, total;           /* work cursor */
    int phase;
    pthread_mutex_t lock;
    int status;
} Job;

static size_t take(Job *job) {
    pthread_mutex_lock(&job->lock);
    const size_t item = job->next < job->total ? job->next++ : SIZE_MAX;
    pthread_mutex_unlock(&job->lock);
    return item;
}
static void fail(Job *job, int status) {
    pthread_mutex_lock(&job->lock);
    if (!job->status) job->status = status;
    pthread_mutex_unlock(&job->lock);
}

/* SwiGLU of `rows` gathered tokens through one expert: gate, up, silu, product, down
 * (src/qwen4_moe.c:318-333).  token_of[r] is the x row of gathered row r. */
static int expert_rows(const QW4OLayer *l, bool shared, size_t expert, const float *x,
                       const size_t *token_of, size_t rows, float *out, size_t out_pitch) {
    const size_t h = l->hidden, inter = shared ? l->shared_inter : l->inter;
    const size_t down_k = shared ? inter : l->down_physical;
    const QW4OTensor *gate = &l->w[shared ? 4 : 1], *up = &l->w[shared ? 5 : 2], *down = &l->w[shared ? 6 : 3];
    const size_t gate_row = qw4o_row_bytes(gate->type, h), up_row = qw4o_row_bytes(up->type, h);
    const size_t down_row = qw4o_row_bytes(down->type, down_k);
    if (!gate_row || !up_row || !down_row) return O_FORMAT;
    float *decoded = malloc(((h > down_k ? h : down_k) + rows * inter) * sizeof *decoded);
    if (!decoded) return O_OOM;
    float *act = decoded + (h > down_k ? h : down_k);
    int status = O_OK;
    const uint8_t *gw = gate->data + expert * inter * gate_row, *uw = up->data + expert * inter * up_row;
    for (size_t n = 0; n < inter; n++) {
        qw4o_decode_row(gate->type, gw + n * gate_row, h, decoded);
        for (size_t r = 0; r < rows; r++)
            if (dot_serial(decoded, x + token_of[r] * h, h, &act[r * inter + n])) status = O_NONFINITE;
    }
    for (size_t n = 0; n < inter; n++) {
        qw4o_decode_row(up->type, uw + n * up_row, h, decoded);
        for (size_t r = 0; r < rows; r++) {
            float u;
            if (dot_serial(decoded, x + token_of[r] * h, h, &u)) status = O_NONFINITE;
            const float a = qw4o_silu(act[r * inter + n]);
            if (!isfinite(a)) status = O_NONFINITE;
            act[r * inter + n] = a * u;
            if (!isfinite(act[r * inter + n])) status = O_NONFINITE;
        }
    }
    const uint8_t *dw = down->data + expert * h * down_row;
    for (size_t c = 0; c < h; c++) {
        qw4o_decode_row(down->type, dw + c * down_row, down_k, decoded);
        for (size_t r = 0; r < rows; r++)
            if (dot_serial(decoded, act + r * inter, inter, &out[r * out_pitch + c])) status = O_NONFINITE;
    }
    free(decoded);
    return status;
}

static void *worker(void *arg) {
    Job *job = arg;
    const QW4OLayer *l = job->layer;
    const size_t h = l->hidden, k = l->k;
    for (;;) {
        const size_t item = take(job);
        if (item == SIZE_MAX) break;
        if (job->phase == 0) {                       /* router + shared logits, one token */
            const size_t t = item;
            float *row = malloc(h * sizeof *row);
            if (!row) { fail(job, O_OOM); continue; }
            for (size_t e = 0; e < l->experts; e++) {
                qw4o_decode_row(l->w[0].type, l->w[0].data + e * qw4o_row_bytes(l->w[0].type, h), h, row);
                if (dot_serial(row, job->x + t * h, h, &job->logits[t * l->experts + e])) fail(job, O_NONFINITE);
            }
            qw4o_decode_row(l->w[7].type, l->w[7].data, h, row);
            if (dot_serial(row, job->x + t * h, h, &job->shared_logit[t])) fail(job, O_NONFINITE);
            free(row);
        } else if (item < l->experts) {              /* one routed expert group */
            const size_t first = job->offsets[item], rows = job->offsets[item + 1] - first;
            if (!rows) continue;
            size_t *token_of = malloc(rows * sizeof *token_of);
            if (!token_of) { fail(job, O_OOM); continue; }
            for (size_t r = 0; r < rows; r++) token_of[r] = job->row_to_pair[first + r] / k;
            const int st = expert_rows(l, false, item, job->x, token_of, rows, job->down + first * h, h);
            if (st) fail(job, st);
            free(token_of);
        } else {                                     /* shared expert, 32 tokens at a time */
            const size_t first = (item - l->experts) * 32;
            const size_t rows = job->tokens - first < 32 ? job->tokens - first : 32;
            size_t token_of[32];
            for (size_t r = 0; r < rows; r++) token_of[r] = first + r;
            const int st = expert_rows(l, true, 0, job->x, token_of, rows, job->shared + first * h, h);
            if (st) fail(job, st);
        }
    }
    return NULL;
}

static void run_phase(Job *job, int phase, size_t total, int threads) {
    job->phase = phase; job->next = 0; job->total = total;
    pthread_t tid[256];
    if (threads > 256) threads = 256;
    int started = 0;
    for (int i = 1; i < threads; i++) if (pthread_create(&tid[started], NULL, worker, job) == 0) started++;
    worker(job);
    for (int i = 0; i < started; i++) pthread_join(tid[i], NULL);
}

/* x, y dense [tokens][hidden]; ids, weights dense [tokens][k]; logits_out (optional)
 * [tokens][experts]; routed_out (optional) [tokens][hidden] is the sum before the shared
 * term.  threads >= 1.  Returns O_OK, O_NONFINITE, ... */
int qw4o_forward(const QW4OLayer *l, const float *x, size_t tokens, float *y, uint32_t *ids,
                 float *weights, float *logits_out, float *routed_out, int threads) {
    const size_t h = l->hidden, e = l->experts, k = l->k, pairs = tokens * k;
    if (!tokens) return O_OK;
    for (size_t i = 0; i < tokens * h; i++) if (!isfinite(x[i])) return O_NONFINITE;
    Job job = {.layer = l, .x = x, .tokens = tokens};
    pthread_mutex_init(&job.lock, NULL);
    float *probs = malloc(tokens * e * sizeof *probs);
    uint64_t *offsets = malloc((e + 1) * sizeof *offsets), *p2r = malloc(pairs * sizeof *p2r);
    uint64_t *r2p = malloc(pairs * sizeof *r2p);
    job.logits = malloc(tokens * e * sizeof(float));
    job.shared_logit = malloc(tokens * sizeof(float));
    job.down = malloc(pairs * h * sizeof(float));
    job.shared = malloc(tokens * h * sizeof(float));
    int status = O_OOM;
    uint64_t bad_row = 0;
    if (!probs || !offsets || !p2r || !r2p || !job.logits || !job.shared_logit || !job.down || !job.shared)
        goto done;
    run_phase(&job, 0, tokens, threads);
    if ((status = job.status)) goto done;
    if (logits_out) memcpy(logits_out, job.logits, tokens * e * sizeof(float));
    if ((status = qw4o_route(l->experts, l->k, l->norm, job.logits, e, tokens, probs, ids, weights, &bad_row))) goto done;
    if ((status = qw4o_group(l->experts, l->k, tokens, ids, offsets, p2r, r2p))) goto done;
    job.ids = ids; job.offsets = offsets; job.row_to_pair = r2p;
    run_phase(&job, 1, e + (tokens + 31) / 32, threads);
    if ((status = job.status)) goto done;
    for (size_t t = 0; t < tokens; t++) {            /* src/qwen4_moe.c:362-380 */
        const float gate = sigmoid_f32(job.shared_logit[t]);
        for (size_t c = 0; c < h; c++) {
            float sum = 0.0f;
            for (size_t s = 0; s < k; s++) {
                const float term = weights[t * k + s] * job.down[p2r[t * k + s] * h + c];
                sum += term;
                if (!isfinite(term) || !isfinite(sum)) status = O_NONFINITE;
            }
            if (routed_out) routed_out[t * h + c] = sum;
            const float term = gate * job.shared[t * h + c];
            sum += term;
            if (!isfinite(term) || !isfinite(sum)) status = O_NONFINITE;
            y[t * h + c] = sum;
        }
    }
done:
    free(probs); free(offsets); free(p2r); free(r2p);
    free(job.logits); free(job.shared_logit); free(job.down); free(job.shared);
    pthread_mutex_destroy(&job.lock);
    return status;
}

/* ------------------------------------------------------------------------------------
 * The expf the CUDA kernels use, restated on the CPU so that it can be compared with libm.
 * glibc's expf is the table-driven double-precision routine published in ARM's optimized
 * routines (2^(k/32) table, cubic in r); x86-64 builds with FMA fuse its products and sums.
 * tests/test_oracle.py checks this function against libm expf on a dense sample of the
 * domain the layer uses (arguments <= 0); the exhaustive comparison over all 1 120 927 745
 * binary32 values in [-104, -0] found no difference against glibc 2.39.
 * ---------------------------------------------------------------------------------- */
static const uint64_t exp2_table[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
};
float qw4o_expf_fma(float x) {
    if (x < -0x1.9fe368p6f) return 0.0f;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32, c1 = 0x1.ebfce50fac4f3p-3 / 32 / 32, c2 = 0x1.62e42ff0c52d6p-1 / 32;
    const double xd = (double)x;
    double kd = fma(inv_ln2_n, xd, shift);
    uint64_t ki; memcpy(&ki, &kd, 8);
    kd -= shift;
    const double r = fma(inv_ln2_n, xd, -kd);
    uint64_t t = exp2_table[ki & 31u] + (ki << 47);
    double s; memcpy(&s, &t, 8);
    const double z = fma(c0, r, c1), r2 = r * r;
    double y = fma(c2, r, 1.0);
    y = fma(z, r2, y);
    return (float)(y * s);
}
/* Number of inputs in bit range [first_bits, last_bits) (negative floats, stepping `step`)
 * where qw4o_expf_fma and libm expf differ. */
uint64_t qw4o_expf_mismatches(uint32_t first_bits, uint32_t last_bits, uint32_t step) {
    uint64_t bad = 0;
    for (uint64_t b = first_bits; b < last_bits; b += step ? step : 1) {
        const uint32_t bits = (uint32_t)b;
        float x; memcpy(&x, &bits, 4);
        const float want = expf(x), got = qw4o_expf_fma(x);
        bad += memcmp(&want, &got, 4) != 0;
    }
    return bad;
}
