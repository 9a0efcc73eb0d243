/* The eight MoE tensors of one layer, straight out of a GGUF v3 file.
 *
 * picoforge finds them through its model-wide loader: the container parse (src/gguf.c:31-106), the role table
 * (src/qwen4_weights.c:91-99: blk.<L>.ffn_gate_inp / ffn_gate_inp_shexp / ffn_{gate,up,down}_shexp /
 * ffn_{gate,up,down}_exps) and the packed layout of each tensor (src/qwen4_packed.c:8-32).  This file does the
 * same for ONE layer and nothing else of the model: it walks the header once, keeps the MoE dimensions
 * (src/qwen4_config.c:170-172, :200-211) and the eight descriptors, maps the file read-only, and hands host views
 * of the payload to qwen4_moe_create, which uploads them; the mapping is released before returning.
 *
 * A malformed file is an error status here (the reference's loader ends the process instead): QW4_IO for the
 * file itself, QW4_FORMAT for the container, QW4_MISSING / QW4_TYPE / QW4_SHAPE for keys and tensors.
 */
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "qwen4_moe_b200.h"

void qw4cu_moe_forget_host_weights(Qwen4Moe *m);                        /* moe_host.c */

/* ---- bounded little-endian cursor ------------------------------------------------------------------ */
typedef struct { const unsigned char *data; size_t size, pos; bool bad; } Cursor;

static const unsigned char *take(Cursor *c, size_t n) {
    if (c->bad || n > c->size - c->pos) { c->bad = true; return NULL; }
    const unsigned char *p = c->data + c->pos;
    c->pos += n;
    return p;
}
static uint64_t number(Cursor *c, size_t width) {
    const unsigned char *p = take(c, width);
    uint64_t v = 0;
    if (p) for (size_t i = width; i-- > 0;) v = (v << 8) | p[i];
    return v;
}
/* A GGUF string: u64 length, bytes (not terminated). */
static const unsigned char *string(Cursor *c, size_t *length) {
    const uint64_t n = number(c, 8);
    if (n > c->size) { c->bad = true; return NULL; }
    *length = (size_t)n;
    return take(c, (size_t)n);
}
static void name_into(Cursor *c, char *out, size_t capacity) {
    size_t n = 0;
    const unsigned char *s = string(c, &n);
    if (!s || n >= capacity || memchr(s, 0, n)) { c->bad = true; out[0] = 0; return; }
    memcpy(out, s, n);
    out[n] = 0;
}
/* Width of a scalar metadata type, 0 for strings, arrays and unknown ids (GGUF v3 value types 0-12). */
static size_t scalar_width(uint32_t type) {
    static const unsigned char width[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
    return type < 13 ? width[type] : 0;
}
static void skip_value(Cursor *c, uint32_t type, int depth) {
    size_t n;
    if (type == 8) { (void)string(c, &n); return; }
    if (type == 9) {
        const uint32_t element = (uint32_t)number(c, 4);
        const uint64_t count = number(c, 8);
        if (depth > 2 || (element != 8 && element != 9 && !scalar_width(element))) { c->bad = true; return; }
        if (scalar_width(element)) {
            if (count > c->size / scalar_width(element)) { c->bad = true; return; }
            (void)take(c, (size_t)count * scalar_width(element));
            return;
        }
        for (uint64_t i = 0; i < count && !c->bad; i++) skip_value(c, element, depth + 1);
        return;
    }
    if (!scalar_width(type)) { c->bad = true; return; }
    (void)take(c, scalar_width(type));
}

/* ---- formats (src/gguf.c:12-22) --------------------------------------------------------------------------- */
static bool format_of(uint32_t type, size_t *block, size_t *bytes) {
    static const struct { uint32_t id; size_t block, bytes; } table[] = {
        {0, 1, 4}, {1, 1, 2}, {8, 32, 34}, {10, 256, 84}, {12, 256, 144}, {16, 256, 66}, {30, 1, 2}, {39, 32, 17}};
    for (size_t i = 0; i < sizeof table / sizeof *table; i++)
        if (table[i].id == type) { *block = table[i].block; *bytes = table[i].bytes; return true; }
    return false;
}

static Qwen4Status fail(Qwen4Error *err, Qwen4Status code, const char *subject, const char *detail, int os_errno, uint64_t offset) {
    if (err) {
        memset(err, 0, sizeof *err);
        err->code = code; err->os_errno = os_errno; err->file_offset = offset;
        snprintf(err->subject, sizeof err->subject, "%s", subject);
        snprintf(err->detail, sizeof err->detail, "%s", detail);
    }
    return code;
}

static const char *const ROLE_SUFFIX[8] = {"ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight",
                                           "ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight",
                                           "ffn_gate_inp_shexp.weight"};
static const char *const CONFIG_KEY[5] = {"qwen4exp.embedding_length", "qwen4exp.expert_count", "qwen4exp.expert_used_count",
                                          "qwen4exp.expert_feed_forward_length", "qwen4exp.expert_shared_feed_forward_length"};

typedef struct { int fd; void *map; size_t size; } Mapping;
static void unmap(Mapping *m) {
    if (m->map && m->map != MAP_FAILED) munmap(m->map, m->size);
    if (m->fd >= 0) close(m->fd);
    m->map = NULL; m->fd = -1;
}

/* Header walk.  On success the slice holds the config, descriptors (absolute file offsets) and layouts. */
static Qwen4Status read_slice(const char *path, uint32_t layer, Mapping *m, QW4CuGgufSlice *out, Qwen4Error *err) {
    memset(out, 0, sizeof *out);
    m->fd = -1; m->map = NULL;
    if (!path) return fail(err, QW4_INVALID_ARGUMENT, "gguf", "null path", 0, 0);
    m->fd = open(path, O_RDONLY);
    struct stat st;
    if (m->fd < 0 || fstat(m->fd, &st) || !S_ISREG(st.st_mode)) {
        const int e = errno;
        unmap(m);
        return fail(err, QW4_IO, path, "cannot open a regular file", e, 0);
    }
    if (st.st_size < 24) { unmap(m); return fail(err, QW4_FORMAT, path, "shorter than a GGUF header", 0, 0); }
    m->size = (size_t)st.st_size;
    m->map = mmap(NULL, m->size, PROT_READ, MAP_PRIVATE, m->fd, 0);
    if (m->map == MAP_FAILED) { const int e = errno; m->map = NULL; unmap(m); return fail(err, QW4_IO, path, "mapping failed", e, 0); }

    Cursor c = {m->map, m->size, 0, false};
    const unsigned char *magic = take(&c, 4);
    if (!magic || memcmp(magic, "GGUF", 4) || number(&c, 4) != 3) return fail(err, QW4_FORMAT, path, "expected little-endian GGUF v3", 0, 0);
    const uint64_t tensor_count = number(&c, 8), metadata_count = number(&c, 8);
    if (c.bad || !tensor_count || tensor_count > 100000 || metadata_count > 100000)
        return fail(err, QW4_FORMAT, path, "invalid descriptor counts", 0, c.pos);

    uint64_t alignment = 32;
    uint32_t config[5] = {0, 0, 0, 0, 0}, down_logical = 0, down_physical = 0;
    bool seen[5] = {false, false, false, false, false}, architecture = false;
    for (uint64_t i = 0; i < metadata_count; i++) {
        char key[128];
        name_into(&c, key, sizeof key);
        const uint32_t type = (uint32_t)number(&c, 4);
        const size_t at = c.pos;
        skip_value(&c, type, 0);
        if (c.bad) return fail(err, QW4_FORMAT, path, "truncated or malformed metadata", 0, at);
        Cursor value = {c.data, c.pos, at, false};
        if (!strcmp(key, "general.architecture")) {
            size_t n = 0;
            const unsigned char *s = type == 8 ? string(&value, &n) : NULL;
            architecture = s && n == 8 && !memcmp(s, "qwen4exp", 8);
            continue;
        }
        uint32_t *slot = NULL;
        if (!strcmp(key, "general.alignment")) {
            if (type != 4) return fail(err, QW4_TYPE, key, "alignment must be uint32", 0, at);
            alignment = number(&value, 4);
            continue;
        }
        for (int j = 0; j < 5; j++)
            if (!strcmp(key, CONFIG_KEY[j])) {
                if (seen[j]) return fail(err, QW4_FORMAT, key, "duplicate key", 0, at);
                seen[j] = true; slot = &config[j];
            }
        if (!strcmp(key, "ds4.qwen4.down.logical_input")) slot = &down_logical;
        if (!strcmp(key, "ds4.qwen4.down.physical_input")) slot = &down_physical;
        if (slot) {
            if (type != 4) return fail(err, QW4_TYPE, key, "metadata type: uint32 expected", 0, at);
            *slot = (uint32_t)number(&value, 4);
            if (!*slot) return fail(err, QW4_RANGE, key, "positive dimension", 0, at);
        }
    }
    if (!architecture) return fail(err, QW4_FORMAT, path, "expected qwen4exp architecture", 0, 0);
    if (!alignment || (alignment & (alignment - 1)) || alignment > 128u * 1024 * 1024) return fail(err, QW4_FORMAT, path, "invalid alignment", 0, 0);
    for (int j = 0; j < 5; j++)
        if (!seen[j]) return fail(err, QW4_MISSING, CONFIG_KEY[j], "required metadata", 0, 0);

    char wanted[8][128];
    bool found[8] = {false};
    for (int j = 0; j < 8; j++) snprintf(wanted[j], sizeof wanted[j], "blk.%u.%s", layer, ROLE_SUFFIX[j]);
    for (uint64_t i = 0; i < tensor_count; i++) {
        QW4CuGgufTensor t;
        memset(&t, 0, sizeof t);
        name_into(&c, t.name, sizeof t.name);
        t.rank = (uint32_t)number(&c, 4);
        if (c.bad || !t.rank || t.rank > 4) return fail(err, QW4_FORMAT, path, "invalid tensor rank", 0, c.pos);
        for (uint32_t d = 0; d < t.rank; d++) {
            t.shape[d] = number(&c, 8);
            if (!t.shape[d]) return fail(err, QW4_FORMAT, t.name, "zero tensor dimension", 0, c.pos);
        }
        t.type = (uint32_t)number(&c, 4);
        t.file_offset = number(&c, 8);                                  /* relative to the data section until the header is complete */
        if (c.bad) return fail(err, QW4_FORMAT, path, "truncated tensor table", 0, c.pos);
        for (int j = 0; j < 8; j++)
            if (!strcmp(t.name, wanted[j])) {
                if (found[j]) return fail(err, QW4_FORMAT, t.name, "duplicate tensor name", 0, c.pos);
                size_t block, bytes;
                if (!format_of(t.type, &block, &bytes)) return fail(err, QW4_UNSUPPORTED, t.name, "unsupported tensor format", 0, c.pos);
                if (t.shape[0] % block || t.file_offset % alignment) return fail(err, QW4_FORMAT, t.name, "unaligned tensor row or offset", 0, c.pos);
                uint64_t total = t.shape[0] / block * bytes;
                for (uint32_t d = 1; d < t.rank; d++) {
                    if (t.shape[d] > UINT64_MAX / (total ? total : 1)) return fail(err, QW4_OVERFLOW, t.name, "tensor extent overflow", 0, c.pos);
                    total *= t.shape[d];
                }
                t.bytes = total;
                out->tensor[j] = t;
                found[j] = true;
            }
    }
    for (int j = 0; j < 8; j++)
        if (!found[j]) return fail(err, QW4_MISSING, wanted[j], "tensor absent from the file", 0, 0);
    const uint64_t data_offset = ((uint64_t)c.pos + alignment - 1) & ~(alignment - 1);
    if (data_offset > m->size) return fail(err, QW4_FORMAT, path, "alignment padding runs past the file", 0, c.pos);
    out->data_offset = data_offset;
    out->file_bytes = m->size;

    Qwen4MoeConfig *cfg = &out->config;
    cfg->hidden_size = config[0]; cfg->experts = config[1]; cfg->top_k = config[2];
    cfg->intermediate = config[3]; cfg->shared_intermediate = config[4];
    cfg->norm_topk_prob = true;                                         /* the profile's constant (src/qwen4_config.c:218-220) */
    for (int j = 0; j < 3; j++) cfg->trunk_type[j] = out->tensor[1 + j].type;
    /* stored K of the routed down projection: Q2_K pads the logical K to 256 (src/qwen4_config.c:43-45); the
     * optional ds4 keys must agree with the tensor and with the intermediate size (:203-206) */
    cfg->down_physical = (uint32_t)out->tensor[3].shape[0];
    if (out->tensor[3].shape[0] > UINT32_MAX) return fail(err, QW4_OVERFLOW, wanted[3], "dimension exceeds 32 bits", 0, 0);
    const uint64_t padded = out->tensor[3].type == 10 ? ((uint64_t)cfg->intermediate + 255) / 256 * 256 : cfg->intermediate;
    if (padded != cfg->down_physical) return fail(err, QW4_SHAPE, "down", "physical K must round logical K to 256", 0, 0);
    if ((down_logical && down_logical != cfg->intermediate) || (down_physical && down_physical != cfg->down_physical))
        return fail(err, QW4_SHAPE, "down", "logical / physical K keys disagree with the tensor", 0, 0);

    const uint64_t h = cfg->hidden_size, f = cfg->intermediate, fs = cfg->shared_intermediate, ne = cfg->experts;
    const uint32_t rank[8] = {2, 3, 3, 3, 2, 2, 2, 1};
    const uint64_t shape[8][3] = {{h, ne, 1}, {h, f, ne}, {h, f, ne}, {cfg->down_physical, h, ne}, {h, fs, 1}, {h, fs, 1}, {fs, h, 1}, {h, 1, 1}};
    const uint64_t logical[8] = {h, h, h, f, h, h, fs, h};
    for (int j = 0; j < 8; j++) {
        QW4CuGgufTensor *t = &out->tensor[j];
        if (t->rank != rank[j]) return fail(err, QW4_SHAPE, t->name, "tensor rank", 0, 0);
        for (uint32_t d = 0; d < t->rank; d++)
            if (t->shape[d] != shape[j][d]) return fail(err, QW4_SHAPE, t->name, "tensor shape differs from the metadata", 0, 0);
        if ((j == 0 || j == 7) && t->type != 0) return fail(err, QW4_TYPE, t->name, "router tensors are F32", 0, 0);
        t->file_offset += data_offset;
        if (t->file_offset > m->size || t->bytes > m->size - t->file_offset) return fail(err, QW4_FORMAT, t->name, "tensor runs past the file", 0, t->file_offset);
        size_t block = 1, bytes = 1;
        (void)format_of(t->type, &block, &bytes);
        QW4PackedLayout *l = &out->layout[j];
        l->gguf_type = t->type;
        l->k_storage = (size_t)t->shape[0]; l->k_logical = (size_t)logical[j];
        l->n_out = t->rank > 1 ? (size_t)t->shape[1] : 1; l->n_experts = t->rank > 2 ? (size_t)t->shape[2] : 1;
        l->row_bytes = l->k_storage / block * bytes;
        l->expert_bytes = l->row_bytes * l->n_out;
        l->tensor_bytes = l->expert_bytes * l->n_experts;
        if (l->tensor_bytes != t->bytes) return fail(err, QW4_FORMAT, t->name, "descriptor bytes differ from physical shape", 0, 0);
    }
    /* the eight payloads must not overlap */
    for (int a = 1; a < 8; a++)
        for (int b = 0; b < a; b++) {
            const QW4CuGgufTensor *p = &out->tensor[a], *q = &out->tensor[b];
            if (p->file_offset < q->file_offset + q->bytes && q->file_offset < p->file_offset + p->bytes)
                return fail(err, QW4_FORMAT, p->name, "overlapping tensors", 0, p->file_offset);
        }
    if (err) memset(err, 0, sizeof *err);
    return QW4_OK;
}

Qwen4Status qw4cu_gguf_slice_describe(const char *path, uint32_t layer, QW4CuGgufSlice *out, Qwen4Error *err) {
    if (!out) return fail(err, QW4_INVALID_ARGUMENT, "gguf", "null output", 0, 0);
    Mapping m;
    const Qwen4Status st = read_slice(path, layer, &m, out, err);
    unmap(&m);
    if (st) memset(out, 0, sizeof *out);
    return st;
}

Qwen4Status qw4cu_moe_create_from_gguf(const char *path, uint32_t layer, Qwen4Moe **out, QW4CuGgufSlice *slice, Qwen4Error *err) {
    if (out) *out = NULL;
    if (!out) return fail(err, QW4_INVALID_ARGUMENT, "gguf", "null output", 0, 0);
    Mapping m;
    QW4CuGgufSlice local;
    Qwen4Status st = read_slice(path, layer, &m, &local, err);
    if (st == QW4_OK) {
        QW4PackedCpuView v[8];
        for (int j = 0; j < 8; j++) {
            v[j].span.data = (const unsigned char *)m.map + local.tensor[j].file_offset;
            v[j].span.bytes = (size_t)local.tensor[j].bytes;
            v[j].layout = local.layout[j];
        }
        const Qwen4MoeWeights weights = {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]};
        st = qwen4_moe_create(&local.config, &weights, out, err);           /* uploads: the mapping is not needed afterwards */
        if (st == QW4_OK) qw4cu_moe_forget_host_weights(*out);
    }
    unmap(&m);
    if (slice) { if (st == QW4_OK) *slice = local; else memset(slice, 0, sizeof *slice); }
    return st;
}
