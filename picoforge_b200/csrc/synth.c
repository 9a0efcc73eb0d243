/* Synthetic weights for the Qwen4 MoE layer: seeded FP32 masters N(0, sigma) encoded into
 * GGUF Q4_K, Q2_K or IQ2_XXS blocks (or kept as F32).
 *
 * picoforge ships no quantiser: its tests fabricate random block bytes
 * (picoforge tests/test_qwen4_fast_kernels.py:280-290).  The encoders below are this
 * project's own.  They only have to emit VALID blocks (finite fp16 scales) whose decoded
 * values are close to the masters; parity is defined on what the reference decodes from the
 * bytes, not on how the bytes were chosen.
 *
 * Determinism: row r of a tensor draws from a counter-based generator keyed by
 * (seed, stream, r), so the bytes do not depend on the number of threads.
 *
 * Host-side data preparation only; nothing here is on the measured path.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "iq2xxs_codebook.h"

/* ---- counter-based random numbers ------------------------------------------------- */
static uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
typedef struct { uint64_t key, counter; } Stream;
static Stream stream_for(uint64_t seed, uint64_t stream, uint64_t row) {
    Stream s = { mix64(mix64(seed + 0x9e3779b97f4a7c15ull) ^ mix64(stream * 0xd1342543de82ef95ull + 1) ^
                       mix64(row + 0x632be59bd9b4e019ull)), 0 };
    return s;
}
static uint64_t next64(Stream *s) { return mix64(s->key + 0x9e3779b97f4a7c15ull * ++s->counter); }

/* Two normals per call (Box-Muller on 24-bit uniforms). */
static void normal_pair(Stream *s, float sigma, float *a, float *b) {
    const uint64_t bits = next64(s);
    const float u1 = ((float)((bits >> 40) & 0xffffff) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = (float)((bits >> 8) & 0xffffff) * (1.0f / 16777216.0f);
    const float radius = sigma * sqrtf(-2.0f * logf(u1)), angle = 6.28318530717958647692f * u2;
    *a = radius * cosf(angle);
    *b = radius * sinf(angle);
}
static void normal_row(uint64_t seed, uint64_t stream, uint64_t row, float sigma, float *out, size_t n) {
    Stream s = stream_for(seed, stream, row);
    size_t i = 0;
    for (; i + 1 < n; i += 2) normal_pair(&s, sigma, out + i, out + i + 1);
    if (i < n) { float spare; normal_pair(&s, sigma, out + i, &spare); }
}

/* ---- binary16 ---------------------------------------------------------------------- */
static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, f = h & 1023u;
    uint32_t bits;
    if (!e) {
        float v = (float)f * 5.9604644775390625e-08f;      /* f * 2^-24, exact */
        memcpy(&bits, &v, 4); bits |= sign;
    } else bits = sign | ((e == 31 ? 255u : e + 112u) << 23) | f << 13;
    float out; memcpy(&out, &bits, 4); return out;
}
/* Round to nearest even; values beyond the finite range saturate (never Inf). */
static uint16_t float_to_half(float v) {
    uint32_t bits; memcpy(&bits, &v, 4);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    float a = fabsf(v);
    if (!(a == a)) return sign;                            /* NaN -> 0: keep blocks finite */
    if (a >= 65504.0f) return sign | 0x7bffu;
    if (a < 6.103515625e-05f) {                            /* subnormal half: multiple of 2^-24 */
        const float scaled = a * 16777216.0f;
        uint32_t q = (uint32_t)scaled;
        const float rest = scaled - (float)q;
        if (rest > 0.5f || (rest == 0.5f && (q & 1u))) q++;
        return sign | (uint16_t)q;
    }
    memcpy(&bits, &a, 4);
    uint32_t mantissa = bits & 0x7fffffu, exponent = (bits >> 23) - 112u;
    uint32_t half = exponent << 10 | mantissa >> 13;
    const uint32_t rest = mantissa & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) half++;
    if (half >= 0x7c00u) half = 0x7bffu;
    return sign | (uint16_t)half;
}
static void put16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
static int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

/* ---- Q4_K: 256 weights = 8 sub-blocks of 32, w = (d*sc)*q - dmin*m ------------------- */
static void encode_q4_k(const float *x, uint8_t *b) {
    float scale[8], minimum[8], max_scale = 0, max_min = 0;
    for (int g = 0; g < 8; g++) {
        float lo = 0, hi = 0;                               /* lo <= 0 so that m >= 0 */
        for (int j = 0; j < 32; j++) { const float v = x[g * 32 + j]; if (v < lo) lo = v; if (v > hi) hi = v; }
        scale[g] = (hi - lo) / 15.0f; minimum[g] = -lo;
        if (scale[g] > max_scale) max_scale = scale[g];
        if (minimum[g] > max_min) max_min = minimum[g];
    }
    const uint16_t dh = float_to_half(max_scale / 63.0f), mh = float_to_half(max_min / 63.0f);
    const float d = half_to_float(dh), dmin = half_to_float(mh);
    memset(b, 0, 144);
    put16(b, dh); put16(b + 2, mh);
    uint8_t *sc = b + 4;
    for (int g = 0; g < 8; g++) {
        const int s = d > 0 ? clampi((int)lrintf(scale[g] / d), 0, 63) : 0;
        const int m = dmin > 0 ? clampi((int)lrintf(minimum[g] / dmin), 0, 63) : 0;
        if (g < 4) { sc[g] |= (uint8_t)s; sc[g + 4] |= (uint8_t)m; }
        else {
            sc[g + 4] |= (uint8_t)((s & 15) | (m & 15) << 4);
            sc[g - 4] |= (uint8_t)((s >> 4) << 6);
            sc[g] |= (uint8_t)((m >> 4) << 6);
        }
        const float dl = d * (float)s, ml = dmin * (float)m;
        for (int j = 0; j < 32; j++) {
            const int q = dl > 0 ? clampi((int)lrintf((x[g * 32 + j] + ml) / dl), 0, 15) : 0;
            b[16 + (g / 2) * 32 + j] |= (uint8_t)(q << ((g % 2) * 4));
        }
    }
}

/* ---- Q2_K: 256 weights = 16 sub-blocks of 16, w = (d*(s&15))*q - dmin*(s>>4) ---------- */
static void encode_q2_k(const float *x, uint8_t *b) {
    float scale[16], minimum[16], max_scale = 0, max_min = 0;
    for (int g = 0; g < 16; g++) {
        float lo = 0, hi = 0;
        for (int j = 0; j < 16; j++) { const float v = x[g * 16 + j]; if (v < lo) lo = v; if (v > hi) hi = v; }
        scale[g] = (hi - lo) / 3.0f; minimum[g] = -lo;
        if (scale[g] > max_scale) max_scale = scale[g];
        if (minimum[g] > max_min) max_min = minimum[g];
    }
    const uint16_t dh = float_to_half(max_scale / 15.0f), mh = float_to_half(max_min / 15.0f);
    const float d = half_to_float(dh), dmin = half_to_float(mh);
    memset(b, 0, 84);
    put16(b + 80, dh); put16(b + 82, mh);
    for (int g = 0; g < 16; g++) {
        const int s = d > 0 ? clampi((int)lrintf(scale[g] / d), 0, 15) : 0;
        const int m = dmin > 0 ? clampi((int)lrintf(minimum[g] / dmin), 0, 15) : 0;
        b[g] = (uint8_t)(s | m << 4);
        const float dl = d * (float)s, ml = dmin * (float)m;
        for (int j = 0; j < 16; j++) {
            const int lane = g * 16 + j;
            const int q = dl > 0 ? clampi((int)lrintf((x[lane] + ml) / dl), 0, 3) : 0;
            b[16 + lane / 128 * 32 + lane % 32] |= (uint8_t)(q << (2 * (lane % 128 / 32)));
        }
    }
}

/* ---- IQ2_XXS: 256 weights = 8 groups of 32 = 4 codebook vectors of 8 each ------------- */
static uint8_t nearest_vector[6561];                       /* 3^8 level patterns -> codebook index */
static pthread_once_t nearest_once = PTHREAD_ONCE_INIT;
static void build_nearest(void) {
    static const int magnitude[3] = {8, 25, 43};
    for (int pattern = 0; pattern < 6561; pattern++) {
        int want[8], p = pattern;
        for (int j = 0; j < 8; j++) { want[j] = magnitude[p % 3]; p /= 3; }
        long best = -1; int best_index = 0;
        for (int i = 0; i < 256; i++) {
            long distance = 0;
            for (int j = 0; j < 8; j++) {
                const int level = (QW4_IQ2XXS_LEVELS[i] >> (2 * j)) & 3;
                const int diff = want[j] - (int)QW4_IQ2XXS_MAGNITUDE(level);
                distance += (long)diff * diff;
            }
            if (best < 0 || distance < best) { best = distance; best_index = i; }
        }
        nearest_vector[pattern] = (uint8_t)best_index;
    }
}
static void encode_iq2_xxs(const float *x, uint8_t *b) {
    pthread_once(&nearest_once, build_nearest);
    float group_scale[8], top = 0;
    for (int g = 0; g < 8; g++) {
        float peak = 0;
        for (int j = 0; j < 32; j++) { const float a = fabsf(x[g * 32 + j]); if (a > peak) peak = a; }
        group_scale[g] = peak / 43.0f;
        if (group_scale[g] > top) top = group_scale[g];
    }
    const uint16_t dh = float_to_half(top / 3.875f);        /* largest group scale is d*31/8 */
    const float d = half_to_float(dh);
    put16(b, dh);
    for (int g = 0; g < 8; g++) {
        const int s = d > 0 ? clampi((int)lrintf((group_scale[g] / d * 8.0f - 1.0f) * 0.5f), 0, 15) : 0;
        const float unit = d * (float)(2 * s + 1) * 0.125f;
        uint32_t bits = (uint32_t)s << 28;
        uint8_t *out = b + 2 + 8 * g;
        for (int slot = 0; slot < 4; slot++) {
            const float *v = x + g * 32 + slot * 8;
            int pattern = 0, power = 1, signs = 0, weakest = 0;
            float weakest_size = INFINITY;
            for (int j = 0; j < 8; j++) {
                const float a = fabsf(v[j]), ratio = unit > 0 ? a / unit : 0;
                pattern += (ratio < 16.5f ? 0 : ratio < 34.0f ? 1 : 2) * power; power *= 3;
                if (v[j] < 0) signs |= 1 << j;
                if (a < weakest_size) { weakest_size = a; weakest = j; }
            }
            if (__builtin_popcount((unsigned)signs) & 1) signs ^= 1 << weakest;   /* even parity */
            out[slot] = nearest_vector[pattern];
            bits |= (uint32_t)(signs & 127) << (7 * slot);
        }
        out[4] = (uint8_t)bits; out[5] = (uint8_t)(bits >> 8); out[6] = (uint8_t)(bits >> 16); out[7] = (uint8_t)(bits >> 24);
    }
}

static size_t block_bytes(uint32_t type) { return type == 12 ? 144 : type == 10 ? 84 : type == 16 ? 66 : 0; }

/* Encodes rows of k floats (k a multiple of 256 for the block formats).  Returns 0, or -1
 * for an unsupported type / shape. */
int qw4s_encode_rows(uint32_t type, const float *src, size_t rows, size_t k, uint8_t *out) {
    if (type == 0) { memcpy(out, src, rows * k * 4); return 0; }
    const size_t bytes = block_bytes(type);
    if (!bytes || k % 256) return -1;
    for (size_t i = 0; i < rows * (k / 256); i++) {
        if (type == 12) encode_q4_k(src + i * 256, out + i * bytes);
        else if (type == 10) encode_q2_k(src + i * 256, out + i * bytes);
        else encode_iq2_xxs(src + i * 256, out + i * bytes);
    }
    return 0;
}

/* A row of fabricated blocks: random code, scale and sign bytes with fp16 super-scales chosen so that the decoded
 * weights have a spread of about 0.02 around zero (the reference's own kernel tests fabricate block bytes the same
 * way: it has no quantiser).  Far cheaper than drawing and encoding Gaussians; any such bytes are valid blocks. */
static void fabricated_row(uint32_t type, uint64_t seed, uint64_t stream, uint64_t row, uint8_t *out, size_t k) {
    Stream s = stream_for(seed, stream ^ 0xfab0000000000000ull, row);
    const size_t bytes = block_bytes(type), blocks = k / 256;
    const float base = type == 12 ? 1.1e-4f : type == 10 ? 2.0e-3f : 3.0e-4f, min_ratio = type == 12 ? 7.5f : 1.5f;
    uint16_t d[16], dmin[16];                                   /* sixteen super-scales, 0.75 .. 1.25 of the base */
    for (int j = 0; j < 16; j++) {
        const float scale = base * (0.75f + 0.5f * (float)j / 15.0f);
        d[j] = float_to_half(scale); dmin[j] = float_to_half(scale * min_ratio);
    }
    for (size_t b = 0; b < blocks; b++) {
        uint8_t *p = out + b * bytes;
        size_t i = 0;
        uint64_t v = 0;
        for (; i + 8 <= bytes; i += 8) { v = next64(&s); memcpy(p + i, &v, 8); }
        if (i < bytes) { v = next64(&s); memcpy(p + i, &v, bytes - i); }
        const int pick = (int)(v >> 60);
        if (type == 12) { put16(p, d[pick]); put16(p + 2, dmin[pick]); }
        else if (type == 10) { put16(p + 80, d[pick]); put16(p + 82, dmin[pick]); }
        else put16(p, d[pick]);
    }
}

typedef struct {
    uint32_t type; uint64_t seed, stream; float sigma; size_t rows, k, first, last, row0; uint8_t *out; int status;
} Slice;
static void *slice_worker(void *arg) {
    Slice *s = arg;
    const size_t bytes = s->type == 0 ? s->k * 4 : s->k / 256 * block_bytes(s->type);
    if (s->sigma < 0.0f && s->type != 0) {                     /* fabricated blocks */
        for (size_t r = s->first; r < s->last; r++) fabricated_row(s->type, s->seed, s->stream, r + s->row0, s->out + r * bytes, s->k);
        return NULL;
    }
    float *row = malloc(s->k * sizeof *row);
    if (!row) { s->status = -1; return NULL; }
    for (size_t r = s->first; r < s->last; r++) {
        normal_row(s->seed, s->stream, r + s->row0, s->sigma, row, s->k);
        if (qw4s_encode_rows(s->type, row, 1, s->k, s->out + r * bytes)) { s->status = -1; break; }
    }
    free(row);
    return NULL;
}

/* A whole tensor of `rows` rows (all experts stacked) of k weights ~ N(0, sigma), encoded
 * as `type`, written to out.  threads >= 1. */
int qw4s_tensor_rows(uint32_t type, uint64_t seed, uint64_t stream, float sigma, size_t row0, size_t rows, size_t k,
                     uint8_t *out, int threads);
int qw4s_tensor(uint32_t type, uint64_t seed, uint64_t stream, float sigma, size_t rows, size_t k,
                uint8_t *out, int threads) {
    return qw4s_tensor_rows(type, seed, stream, sigma, 0, rows, k, out, threads);
}
/* Rows [row0, row0 + rows) of the same tensor (an expert shard): identical bytes to the
 * corresponding slice of the whole tensor.  sigma < 0 (block formats): fabricated blocks instead of
 * encoded Gaussians. */
int qw4s_tensor_rows(uint32_t type, uint64_t seed, uint64_t stream, float sigma, size_t row0, size_t rows, size_t k,
                     uint8_t *out, int threads) {
    if (type != 0 && (!block_bytes(type) || k % 256)) return -1;
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if ((size_t)threads > rows) threads = rows ? (int)rows : 1;
    pthread_once(&nearest_once, build_nearest);
    Slice slice[256]; pthread_t tid[256];
    const size_t per = (rows + (size_t)threads - 1) / (size_t)threads;
    int started = 0;
    for (int i = 0; i < threads; i++) {
        const size_t first = per * (size_t)i, last = first + per < rows ? first + per : rows;
        slice[i] = (Slice){type, seed, stream, sigma, rows, k, first < rows ? first : rows, last, row0, out, 0};
        if (i + 1 < threads && pthread_create(&tid[started], NULL, slice_worker, &slice[i]) == 0) started++;
        else slice_worker(&slice[i]);
    }
    for (int i = 0; i < started; i++) pthread_join(tid[i], NULL);
    for (int i = 0; i < threads; i++) if (slice[i].status) return -1;
    return 0;
}

/* n floats ~ N(0, sigma) from (seed, stream), row-keyed in chunks of `k`. */
void qw4s_normal(uint64_t seed, uint64_t stream, float sigma, float *out, size_t rows, size_t k) {
    for (size_t r = 0; r < rows; r++) normal_row(seed, stream, r, sigma, out + r * k, k);
}
