// The observed forward: the layer run stage by stage in the reference's order, for callers that set
// an observer (picoforge src/qwen4_moe_internal.h:9-15, qw4_moe_observe).
//
// The fast kernels fuse gate, up, SiLU, product, down and the combine, so the per-expert stages the
// reference's observer reports (projection stages = weight indices 0-7, 8 SiLU, 9 product, 10 sigmoid,
// 11 routed sum, 12 y) never exist in memory there.  When an observer is set the forward takes this path
// instead: every stage of src/qwen4_moe.c:334-382 is one plain kernel (one thread per output, products and
// sums separately rounded in ascending k, libm-exact expf), in 32-token microbatches like the reference, and
// after every stage the buffers are copied back and handed to the observer with the reference's stage,
// expert and token arguments.  It is a diagnostic path, as in the reference ("never substitutes an
// operator"): slow, exact, and independent of the fast kernels it is compared with.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../../include/qwen4_moe_b200.h"
#include "cuda_shim.h"
#include "formats.cuh"
#include "route.cuh"

extern "C" int qw4sh_note_launch(const char *name);
extern "C" int qw4sh_fail_text(const char *text);
extern "C" int qw4sh_route(uint32_t experts, uint32_t k, int norm, const float *logits, size_t pitch, size_t tokens, float *probs, uint32_t *ids,
                           float *weights, uint32_t *status, void *stream);

namespace qw4 {

// y[r, n] = sum over k < k_logical of weight(expert, n, k) * x[row(r), k], serial in k, no FMA
// (src/qwen4_packed.c:164-173).  row(r) = gather ? gather[r] / divide : r.
__global__ void __launch_bounds__(128) observed_linear_kernel(DevTensor t, uint32_t expert, const float *__restrict__ x, uint32_t x_pitch,
                                                              const uint32_t *__restrict__ gather, uint32_t divide, uint32_t rows,
                                                              float *__restrict__ y, uint32_t *status) {
    const uint32_t n = blockIdx.x * 128 + threadIdx.x, r = blockIdx.y;
    if (n >= t.n_out || r >= rows) return;
    const float *row = x + (uint64_t)(gather ? gather[r] / divide : r) * x_pitch;
    float sum = 0.0f;
    for (uint32_t k = 0; k < t.k_logical; k++) sum = __fadd_rn(sum, __fmul_rn(decode_value(t, expert, n, k), row[k]));
    if (!finite_f32(sum)) atomicOr(status, QW4SH_ERR_NONFINITE);
    y[(uint64_t)r * t.n_out + n] = sum;
}
// mode 0: out = silu(in) (x * sigmoid(x), src/qwen4_cpu_internal.h:103-107); 1: out *= in; 2: out = sigmoid(in)
__global__ void __launch_bounds__(256) observed_map_kernel(int mode, const float *__restrict__ in, float *__restrict__ out, uint32_t n,
                                                           uint32_t *status) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float v;
    if (mode == 0) v = __fmul_rn(in[i], sigmoid_libm(in[i]));
    else if (mode == 1) v = __fmul_rn(out[i], in[i]);
    else v = sigmoid_libm(in[i]);
    if (!finite_f32(v)) atomicOr(status, QW4SH_ERR_NONFINITE);
    out[i] = v;
}
// mode 0: y[t, c] = sum over slots in slot order of weight * down[pair_to_row[pair], c] (src/qwen4_moe.c:362-372);
// mode 1: y[t, c] += gate[t] * shared[t, c] (:374-379)
__global__ void __launch_bounds__(256) observed_combine_kernel(int mode, const float *__restrict__ weights, const float *__restrict__ down,
                                                               const uint32_t *__restrict__ pair_to_row, const float *__restrict__ gate,
                                                               const float *__restrict__ shared, uint32_t k, uint32_t hidden, float *__restrict__ y,
                                                               uint32_t *status) {
    const uint32_t t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= hidden) return;
    float out;
    if (mode == 0) {
        out = 0.0f;
        for (uint32_t s = 0; s < k; s++) out = __fadd_rn(out, __fmul_rn(weights[t * k + s], down[(uint64_t)pair_to_row[t * k + s] * hidden + c]));
    } else out = __fadd_rn(y[(uint64_t)t * hidden + c], __fmul_rn(gate[t], shared[(uint64_t)t * hidden + c]));
    if (!finite_f32(out)) atomicOr(status, QW4SH_ERR_NONFINITE);
    y[(uint64_t)t * hidden + c] = out;
}

}  // namespace qw4

using namespace qw4;

#define CU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { qw4sh_fail_text(cudaGetErrorString(e_)); return (int)e_; } } while (0)

namespace {
DevTensor dev(const QW4ShTensor &s) {
    DevTensor t;
    t.data = s.data; t.type = s.type; t.k_storage = s.k_storage; t.k_logical = s.k_logical;
    t.n_out = s.n_out; t.n_experts = s.n_experts; t.row_bytes = s.row_bytes; t.expert_bytes = s.expert_bytes;
    return t;
}
Qwen4F32 matrix(const float *data, size_t rows, size_t cols, size_t pitch_floats) {
    Qwen4F32 v;
    memset(&v, 0, sizeof v);
    v.data = data; v.capacity_bytes = rows ? ((rows - 1) * pitch_floats + cols) * 4 : 0; v.rank = 2;
    v.dim[0] = rows; v.dim[1] = cols; v.dim[2] = 1; v.dim[3] = 1;
    v.stride_bytes[0] = pitch_floats * 4; v.stride_bytes[1] = 4;
    return v;
}
struct Scratch {                                  // device and host twins of the stage buffers of one microbatch
    float *d = nullptr;
    std::vector<float> h;
    int alloc(size_t floats) {
        h.resize(floats);
        return cudaMalloc(&d, floats * 4 + 16) == cudaSuccess ? 0 : -1;
    }
    int fetch(size_t floats, cudaStream_t s) { return cudaMemcpyAsync(h.data(), d, floats * 4, cudaMemcpyDeviceToHost, s) == cudaSuccess ? 0 : -1; }
    ~Scratch() { cudaFree(d); }
};
int linear(const QW4ShTensor &w, uint32_t expert, const float *x, uint32_t x_pitch, const uint32_t *gather, uint32_t divide, uint32_t rows,
           float *y, uint32_t *status, cudaStream_t s) {
    if (!rows) return 0;
    observed_linear_kernel<<<dim3((w.n_out + 127) / 128, rows), 128, 0, s>>>(dev(w), expert, x, x_pitch, gather, divide, rows, y, status);
    return qw4sh_note_launch("observed_linear_kernel");
}
int map(int mode, const float *in, float *out, size_t n, uint32_t *status, cudaStream_t s) {
    if (!n) return 0;
    observed_map_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(mode, in, out, (uint32_t)n, status);
    return qw4sh_note_launch("observed_map_kernel");
}
}  // namespace

// x, y: device [tokens, hidden] dense; x_host: the caller's rows (what the observer is shown as the stage input);
// token0: index of the first token of this call in the caller's batch.  Writes ids / weights of the workspace too.
// Returns 0, or -1 with the error text set; device-side findings go to work->status as elsewhere.
extern "C" int qw4sh_observed_forward(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens, const float *x_host,
                                      size_t x_host_pitch, size_t token0, void (*observer)(void *, size_t, size_t, size_t, Qwen4F32, Qwen4F32),
                                      void *ctx) {
    cudaStream_t s = (cudaStream_t)work->stream;
    const uint32_t H = layer->hidden, E = layer->experts, k = layer->top_k, I = layer->inter, IS = layer->shared_inter;
    const uint32_t imax = I > IS ? I : IS, MICRO = 32;
    Scratch z, g, u, a, down, shared, sg, sa, yy;
    if (z.alloc((size_t)MICRO * E) || g.alloc((size_t)MICRO * imax) || u.alloc((size_t)MICRO * imax) || a.alloc((size_t)MICRO * imax) ||
        down.alloc((size_t)MICRO * k * H) || shared.alloc((size_t)MICRO * H) || sg.alloc(MICRO) || sa.alloc(MICRO) || yy.alloc((size_t)MICRO * H))
        return qw4sh_fail_text("observed forward: scratch allocation");
    std::vector<uint32_t> ids(MICRO * k), p2r(MICRO * k), r2p(MICRO * k), offsets(E + 1);
    std::vector<float> weights(MICRO * k), gathered((size_t)MICRO * H);
    uint32_t *d_lists = nullptr;                                               // pair_to_row | row_to_pair of the microbatch
    if (cudaMalloc(&d_lists, 2 * MICRO * k * 4 + 16) != cudaSuccess) return qw4sh_fail_text("observed forward: list allocation");
    int rc = 0;
#define STEP(call) do { if (!rc && (call)) rc = -1; } while (0)
#define SYNC() do { if (!rc && cudaStreamSynchronize(s) != cudaSuccess) rc = qw4sh_fail_text("observed forward: synchronize"); } while (0)
    for (size_t first = 0; first < tokens && !rc; first += MICRO) {
        const uint32_t n = (uint32_t)(tokens - first < MICRO ? tokens - first : MICRO), pairs = n * k;
        const float *xb = x + first * H;
        const size_t token = token0 + first;
        const Qwen4F32 x_view = matrix(x_host + first * x_host_pitch, n, H, x_host_pitch);
        // stage 0: router logits; routing; grouping of this microbatch (host, the reference's stable order)
        STEP(linear(layer->w[0], 0, xb, H, nullptr, 1, n, z.d, work->status, s));
        STEP(qw4sh_route(E, k, layer->norm, z.d, E, n, work->probs, work->ids + first * k, work->weights + first * k, work->status, s));
        STEP(z.fetch((size_t)n * E, s));
        if (!rc && (cudaMemcpyAsync(ids.data(), work->ids + first * k, pairs * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
                    cudaMemcpyAsync(weights.data(), work->weights + first * k, pairs * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess)) rc = -1;
        SYNC();
        if (rc) break;
        observer(ctx, 0, 0, token, x_view, matrix(z.h.data(), n, E, E));
        bool routed = true;
        for (uint32_t p = 0; p < pairs; p++) routed &= ids[p] < E;             // a failed routing leaves ids unset: the status word says why
        if (!routed) break;
        std::fill(offsets.begin(), offsets.end(), 0u);
        for (uint32_t p = 0; p < pairs; p++) offsets[ids[p] + 1]++;
        for (uint32_t e = 0; e < E; e++) offsets[e + 1] += offsets[e];
        {
            std::vector<uint32_t> cursor(offsets.begin(), offsets.end() - 1);
            for (uint32_t p = 0; p < pairs; p++) { const uint32_t row = cursor[ids[p]]++; p2r[p] = row; r2p[row] = p; }
        }
        if (cudaMemcpyAsync(d_lists, p2r.data(), pairs * 4, cudaMemcpyHostToDevice, s) != cudaSuccess ||
            cudaMemcpyAsync(d_lists + MICRO * k, r2p.data(), pairs * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = -1; break; }
        const uint32_t *d_p2r = d_lists, *d_r2p = d_lists + MICRO * k;
        // routed experts in ascending order, each on its gathered rows
        for (uint32_t e = 0; e < E && !rc; e++) {
            const uint32_t begin = offsets[e], rows = offsets[e + 1] - begin;
            if (!rows) continue;
            for (uint32_t r = 0; r < rows; r++)
                memcpy(&gathered[(size_t)r * H], x_host + (first + r2p[begin + r] / k) * x_host_pitch, (size_t)H * 4);
            const Qwen4F32 gx = matrix(gathered.data(), rows, H, H);
            STEP(linear(layer->w[1], e, xb, H, d_r2p + begin, k, rows, g.d, work->status, s));
            STEP(linear(layer->w[2], e, xb, H, d_r2p + begin, k, rows, u.d, work->status, s));
            STEP(map(0, g.d, a.d, (size_t)rows * I, work->status, s));
            STEP(g.fetch((size_t)rows * I, s)); STEP(u.fetch((size_t)rows * I, s)); STEP(a.fetch((size_t)rows * I, s));
            SYNC();
            if (rc) break;
            observer(ctx, 1, e, token, gx, matrix(g.h.data(), rows, I, I));
            observer(ctx, 2, e, token, gx, matrix(u.h.data(), rows, I, I));
            observer(ctx, 8, e, token, matrix(g.h.data(), rows, I, I), matrix(a.h.data(), rows, I, I));
            STEP(map(1, u.d, a.d, (size_t)rows * I, work->status, s));
            STEP(linear(layer->w[3], e, a.d, I, nullptr, 1, rows, down.d + (size_t)begin * H, work->status, s));
            STEP(a.fetch((size_t)rows * I, s));
            if (!rc && cudaMemcpyAsync(down.h.data() + (size_t)begin * H, down.d + (size_t)begin * H, (size_t)rows * H * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) rc = -1;
            SYNC();
            if (rc) break;
            observer(ctx, 9, e, token, matrix(u.h.data(), rows, I, I), matrix(a.h.data(), rows, I, I));
            observer(ctx, 3, e, token, matrix(a.h.data(), rows, I, I), matrix(down.h.data() + (size_t)begin * H, rows, H, H));
        }
        if (rc) break;
        // shared expert, shared router, sigmoid
        STEP(linear(layer->w[4], 0, xb, H, nullptr, 1, n, g.d, work->status, s));
        STEP(linear(layer->w[5], 0, xb, H, nullptr, 1, n, u.d, work->status, s));
        STEP(map(0, g.d, a.d, (size_t)n * IS, work->status, s));
        STEP(g.fetch((size_t)n * IS, s)); STEP(u.fetch((size_t)n * IS, s)); STEP(a.fetch((size_t)n * IS, s));
        SYNC();
        if (rc) break;
        observer(ctx, 4, 0, token, x_view, matrix(g.h.data(), n, IS, IS));
        observer(ctx, 5, 0, token, x_view, matrix(u.h.data(), n, IS, IS));
        observer(ctx, 8, SIZE_MAX, token, matrix(g.h.data(), n, IS, IS), matrix(a.h.data(), n, IS, IS));
        STEP(map(1, u.d, a.d, (size_t)n * IS, work->status, s));
        STEP(linear(layer->w[6], 0, a.d, IS, nullptr, 1, n, shared.d, work->status, s));
        STEP(linear(layer->w[7], 0, xb, H, nullptr, 1, n, sg.d, work->status, s));
        STEP(map(2, sg.d, sa.d, n, work->status, s));
        STEP(a.fetch((size_t)n * IS, s)); STEP(shared.fetch((size_t)n * H, s)); STEP(sg.fetch(n, s)); STEP(sa.fetch(n, s));
        SYNC();
        if (rc) break;
        observer(ctx, 9, SIZE_MAX, token, matrix(u.h.data(), n, IS, IS), matrix(a.h.data(), n, IS, IS));
        observer(ctx, 6, 0, token, matrix(a.h.data(), n, IS, IS), matrix(shared.h.data(), n, H, H));
        observer(ctx, 7, 0, token, x_view, matrix(sg.h.data(), n, 1, 1));
        observer(ctx, 10, SIZE_MAX, token, matrix(sg.h.data(), n, 1, 1), matrix(sa.h.data(), n, 1, 1));
        // routed sum in slot order, then the gated shared expert
        float *yb = y + first * H;
        observed_combine_kernel<<<dim3((H + 255) / 256, n), 256, 0, s>>>(0, work->weights + first * k, down.d, d_p2r, nullptr, nullptr, k, H, yb, work->status);
        STEP(qw4sh_note_launch("observed_combine_kernel"));
        if (!rc && cudaMemcpyAsync(yy.h.data(), yb, (size_t)n * H * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) rc = -1;
        SYNC();
        if (rc) break;
        observer(ctx, 11, SIZE_MAX, token, x_view, matrix(yy.h.data(), n, H, H));
        observed_combine_kernel<<<dim3((H + 255) / 256, n), 256, 0, s>>>(1, nullptr, nullptr, nullptr, sa.d, shared.d, k, H, yb, work->status);
        STEP(qw4sh_note_launch("observed_combine_kernel"));
        if (!rc && cudaMemcpyAsync(yy.h.data(), yb, (size_t)n * H * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) rc = -1;
        SYNC();
        if (rc) break;
        observer(ctx, 12, SIZE_MAX, token, x_view, matrix(yy.h.data(), n, H, H));
    }
#undef STEP
#undef SYNC
    cudaFree(d_lists);
    if (rc) qw4sh_fail_text("observed forward: launch or copy failed");
    return rc;
}
