// Expert parallelism inside the library (new design: the reference is a single-device engine).
//
// Experts are cut into contiguous blocks, one per rank; the router and the shared expert are
// replicated; tokens are data-parallel (every rank brings the same number).  One layer step:
//
//   1. a rank routes its own tokens and packs one exchange row per TOKEN: the token's `hidden`
//      activations, its k route ids and its k route weights (ep_pack_kernel); the shared expert of
//      its own tokens starts on a second stream;
//   2. all-gather: every rank now holds every token's row once, whatever the number of experts of a
//      token a rank owns (a row crosses NVLink once per destination, never once per pair);
//   3. a rank runs ITS experts on the tokens that route to them (lists built from the gathered ids with
//      the foreign ones masked out) and forms, per token, the weighted sum of its own experts' outputs,
//      plus the sigmoid-gated shared expert for the tokens it owns (ep_partial_kernel);
//   4. reduce-scatter (sum): a rank receives the finished rows of its own tokens.
//
// Two collectives per layer, both on large contiguous buffers, both issued by this file through NCCL
// (ncclAllGather, ncclReduceScatter) on the stream the library enqueues on.  NCCL is taken from the process
// at run time (dlopen of libnccl.so.2): a program that never makes a communicator needs no NCCL.  Nothing here
// waits on another rank in a kernel of its own: the only cross-rank waits are NCCL's.
//
// The sum over a token's experts runs per rank and then over ranks, not in slot order: y differs from the
// one-GPU result in the last bits (the layer tolerance holds); ids and weights are the router's bits.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "cuda_shim.h"

extern "C" int qw4sh_note_launch(const char *name);
extern "C" int qw4sh_fail_text(const char *text);

namespace qw4 {

// ---- kernels ---------------------------------------------------------------------------------------------
// Row t of the message: x[t, 0..hidden) | ids[t, 0..k) as words | weights[t, 0..k); k padded to a multiple of 4.
__global__ void __launch_bounds__(256) ep_pack_kernel(const float *__restrict__ x, const uint32_t *__restrict__ ids,
                                                      const float *__restrict__ weights, uint32_t hidden, uint32_t k, uint32_t kp,
                                                      float *__restrict__ msg, uint32_t pitch) {
    const uint32_t t = blockIdx.x;
    const float4 *src = reinterpret_cast<const float4 *>(x + (uint64_t)t * hidden);
    float4 *dst = reinterpret_cast<float4 *>(msg + (uint64_t)t * pitch);
    for (uint32_t i = threadIdx.x; i < hidden / 4; i += 256) dst[i] = src[i];
    uint32_t *tail = reinterpret_cast<uint32_t *>(msg + (uint64_t)t * pitch + hidden);
    for (uint32_t s = threadIdx.x; s < 2 * kp; s += 256) {
        uint32_t word = 0xffffffffu;
        if (s < kp) { if (s < k) word = ids[t * k + s]; }
        else { const uint32_t j = s - kp; word = j < k ? __float_as_uint(weights[t * k + j]) : 0u; }
        tail[s] = word;
    }
}

// Pair p = token * k + slot of the gathered rows: its expert's index inside this rank's block, or 0xffffffff.
__global__ void __launch_bounds__(256) ep_local_ids_kernel(const float *__restrict__ msg, uint32_t pitch, uint32_t hidden, uint32_t k,
                                                           uint32_t pairs, uint32_t experts, uint32_t first, uint32_t count,
                                                           uint32_t *__restrict__ local, uint32_t *status) {
    const uint32_t p = blockIdx.x * 256 + threadIdx.x;
    if (p >= pairs) return;
    const uint32_t id = __float_as_uint(msg[(uint64_t)(p / k) * pitch + hidden + p % k]);
    if (id >= experts) atomicOr(status, QW4SH_ERR_BOUNDS);
    local[p] = id >= first && id - first < count ? id - first : 0xffffffffu;
}

// partial[t, c] = sum over the slots of token t whose expert this rank owns of weight * out[pair, c]
// (+ sigmoid(shared logit) * shared_out for the tokens this rank owns: [own_first, own_first + own)).
__global__ void __launch_bounds__(256) ep_partial_kernel(const float *__restrict__ msg, uint32_t pitch, uint32_t hidden, uint32_t k, uint32_t kp,
                                                         const uint32_t *__restrict__ local, const float *__restrict__ out,
                                                         const float *__restrict__ shared_out, const float *__restrict__ shared_logit,
                                                         uint32_t own_first, uint32_t own, float *__restrict__ partial, uint32_t *status) {
    const uint32_t t = blockIdx.y, c = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (c >= hidden) return;
    const float *weights = msg + (uint64_t)t * pitch + hidden + kp;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t s = 0; s < k; s++) {
        if (local[t * k + s] == 0xffffffffu) continue;
        const float w = weights[s];
        const float4 v = *reinterpret_cast<const float4 *>(out + ((uint64_t)t * k + s) * hidden + c);
        sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y); sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
    }
    if (t >= own_first && t - own_first < own) {
        const uint32_t tl = t - own_first;
        const float sl = shared_logit[tl], e = __expf(-fabsf(sl));
        const float gate = sl >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
        const float4 v = *reinterpret_cast<const float4 *>(shared_out + (uint64_t)tl * hidden + c);
        sum.x = fmaf(gate, v.x, sum.x); sum.y = fmaf(gate, v.y, sum.y); sum.z = fmaf(gate, v.z, sum.z); sum.w = fmaf(gate, v.w, sum.w);
    }
    if ((__float_as_uint(sum.x) & 0x7f800000u) == 0x7f800000u || (__float_as_uint(sum.y) & 0x7f800000u) == 0x7f800000u ||
        (__float_as_uint(sum.z) & 0x7f800000u) == 0x7f800000u || (__float_as_uint(sum.w) & 0x7f800000u) == 0x7f800000u)
        atomicOr(status, QW4SH_ERR_NONFINITE);
    *reinterpret_cast<float4 *>(partial + (uint64_t)t * hidden + c) = sum;
}

// The non-empty experts of the block [first, first + count) out of the ascending list of all non-empty experts
// (active[0] entries from active[1]), as indices inside the block: active_local[0] = how many, then the indices.
__global__ void __launch_bounds__(1024) ep_active_slice_kernel(const uint32_t *__restrict__ active, uint32_t first, uint32_t count,
                                                               uint32_t *__restrict__ active_local) {
    const uint32_t n = active[0];
    __shared__ uint32_t below, inside;
    if (threadIdx.x == 0) { below = 0; inside = 0; }
    __syncthreads();
    uint32_t b = 0, in = 0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t e = active[1 + i];
        b += e < first ? 1u : 0u;
        in += e >= first && e - first < count ? 1u : 0u;
    }
    atomicAdd(&below, b); atomicAdd(&inside, in);
    __syncthreads();
    if (threadIdx.x == 0) active_local[0] = inside;
    for (uint32_t i = threadIdx.x; i < inside; i += blockDim.x) active_local[1 + i] = active[1 + below + i] - first;   // ascending: the block is contiguous
}

}  // namespace qw4

using namespace qw4;

#define CU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { qw4sh_fail_text(cudaGetErrorString(e_)); return (int)e_; } } while (0)

extern "C" uint32_t qw4sh_ep_row_floats(uint32_t hidden, uint32_t k) { return hidden + 2 * ((k + 3) & ~3u); }

extern "C" int qw4sh_ep_pack_rows(const float *x, const uint32_t *ids, const float *weights, uint32_t tokens, uint32_t hidden, uint32_t k,
                                  float *msg, void *stream) {
    if (!tokens) return 0;
    ep_pack_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(x, ids, weights, hidden, k, (k + 3) & ~3u, msg, qw4sh_ep_row_floats(hidden, k));
    return qw4sh_note_launch("ep_pack_kernel");
}
extern "C" int qw4sh_ep_local_ids(const float *msg, uint32_t hidden, uint32_t k, uint32_t tokens, uint32_t experts, uint32_t first,
                                  uint32_t count, uint32_t *local, uint32_t *status, void *stream) {
    const uint32_t pairs = tokens * k;
    if (!pairs) return 0;
    ep_local_ids_kernel<<<(pairs + 255) / 256, 256, 0, (cudaStream_t)stream>>>(msg, qw4sh_ep_row_floats(hidden, k), hidden, k, pairs, experts, first,
                                                                              count, local, status);
    return qw4sh_note_launch("ep_local_ids_kernel");
}
extern "C" int qw4sh_ep_active_slice(const uint32_t *active, uint32_t first, uint32_t count, uint32_t *active_local, void *stream) {
    ep_active_slice_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(active, first, count, active_local);
    return qw4sh_note_launch("ep_active_slice_kernel");
}
extern "C" int qw4sh_ep_partial(const float *msg, uint32_t hidden, uint32_t k, uint32_t tokens, const uint32_t *local, const float *out,
                                const float *shared_out, const float *shared_logit, uint32_t own_first, uint32_t own, float *partial,
                                uint32_t *status, void *stream) {
    if (!tokens) return 0;
    ep_partial_kernel<<<dim3((hidden / 4 + 255) / 256, tokens), 256, 0, (cudaStream_t)stream>>>(
        msg, qw4sh_ep_row_floats(hidden, k), hidden, k, (k + 3) & ~3u, local, out, shared_out, shared_logit, own_first, own, partial, status);
    return qw4sh_note_launch("ep_partial_kernel");
}

// ---- NCCL, bound at run time -------------------------------------------------------------------------------
// The few entry points used, with the types of nccl.h (2.x ABI): results are ints (0 = success), ncclFloat = 7,
// ncclSum = 0, the unique id is 128 opaque bytes passed by value.
namespace {
struct NcclId { char bytes[128]; };
typedef void *NcclComm;
struct NcclApi {
    void *handle;
    int (*get_unique_id)(NcclId *);
    int (*comm_init_rank)(NcclComm *, int, NcclId, int);
    int (*comm_destroy)(NcclComm);
    int (*all_gather)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
    int (*reduce_scatter)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t);
    const char *(*error_string)(int);
};
NcclApi g_nccl = {};
const int NCCL_FLOAT = 7, NCCL_SUM = 0;

int nccl_bind() {
    if (g_nccl.handle) return 0;
    const char *names[] = {getenv("QW4CU_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    void *h = nullptr;
    for (const char *name : names) if (name && *name && (h = dlopen(name, RTLD_NOW | RTLD_GLOBAL))) break;
    if (!h) return qw4sh_fail_text("libnccl.so.2 not found (set QW4CU_NCCL_LIBRARY)");
    NcclApi api = {};
    api.handle = h;
    *(void **)&api.get_unique_id = dlsym(h, "ncclGetUniqueId");
    *(void **)&api.comm_init_rank = dlsym(h, "ncclCommInitRank");
    *(void **)&api.comm_destroy = dlsym(h, "ncclCommDestroy");
    *(void **)&api.all_gather = dlsym(h, "ncclAllGather");
    *(void **)&api.reduce_scatter = dlsym(h, "ncclReduceScatter");
    *(void **)&api.error_string = dlsym(h, "ncclGetErrorString");
    if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_gather || !api.reduce_scatter || !api.error_string)
        return qw4sh_fail_text("libnccl.so.2 lacks an expected entry point");
    g_nccl = api;
    return 0;
}
int nccl_check(int rc, const char *what) {
    if (rc == 0) return 0;
    char text[200];
    snprintf(text, sizeof text, "%s: %s", what, g_nccl.error_string ? g_nccl.error_string(rc) : "NCCL error");
    qw4sh_fail_text(text);
    return rc;
}
}  // namespace

struct QW4ShEp {
    NcclComm comm;
    int rank, world;
    float *msg_local, *msg_all, *partial;            // grown on demand, owned here
    size_t msg_local_floats, msg_all_floats, partial_floats;
};

extern "C" int qw4sh_ep_unique_id(unsigned char id[128]) {
    if (nccl_bind()) return -1;
    NcclId nid;
    if (nccl_check(g_nccl.get_unique_id(&nid), "ncclGetUniqueId")) return -1;
    memcpy(id, nid.bytes, 128);
    return 0;
}
extern "C" int qw4sh_ep_create(const unsigned char id[128], int rank, int world, QW4ShEp **out) {
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return qw4sh_fail_text("rank outside the world");
    QW4ShEp *ep = new QW4ShEp();
    memset(ep, 0, sizeof *ep);
    ep->rank = rank; ep->world = world;
    if (world > 1) {
        if (nccl_bind()) { delete ep; return -1; }
        NcclId nid;
        memcpy(nid.bytes, id, 128);
        if (nccl_check(g_nccl.comm_init_rank(&ep->comm, world, nid, rank), "ncclCommInitRank")) { delete ep; return -1; }
    }
    *out = ep;
    return 0;
}
extern "C" void qw4sh_ep_destroy(QW4ShEp *ep) {
    if (!ep) return;
    if (ep->comm) g_nccl.comm_destroy(ep->comm);
    cudaFree(ep->msg_local); cudaFree(ep->msg_all); cudaFree(ep->partial);
    delete ep;
}
extern "C" int qw4sh_ep_rank(const QW4ShEp *ep) { return ep ? ep->rank : -1; }
extern "C" int qw4sh_ep_world(const QW4ShEp *ep) { return ep ? ep->world : 0; }

static int grow(float **buffer, size_t *have, size_t want) {
    if (*have >= want) return 0;
    cudaFree(*buffer);
    *buffer = nullptr; *have = 0;
    CU(cudaMalloc(buffer, want * sizeof(float)));
    *have = want;
    return 0;
}
// Buffers for `tokens_local` tokens per rank (allocates when they grow: call once outside any capture).
extern "C" int qw4sh_ep_reserve(QW4ShEp *ep, uint32_t hidden, uint32_t k, size_t tokens_local) {
    const size_t pitch = qw4sh_ep_row_floats(hidden, k), total = tokens_local * (size_t)ep->world;
    int rc;
    if ((rc = grow(&ep->msg_local, &ep->msg_local_floats, tokens_local * pitch + 4))) return rc;
    if ((rc = grow(&ep->msg_all, &ep->msg_all_floats, total * pitch + 4))) return rc;
    return grow(&ep->partial, &ep->partial_floats, total * hidden + 4);
}
extern "C" float *qw4sh_ep_msg_local(QW4ShEp *ep) { return ep->msg_local; }
extern "C" float *qw4sh_ep_msg_all(QW4ShEp *ep) { return ep->msg_all; }
extern "C" float *qw4sh_ep_partial_buffer(QW4ShEp *ep) { return ep->partial; }

// all-gather of the packed rows: msg_local [tokens_local, pitch] -> msg_all [world * tokens_local, pitch]
extern "C" int qw4sh_ep_all_gather(QW4ShEp *ep, size_t floats_per_rank, void *stream) {
    if (ep->world == 1) { CU(cudaMemcpyAsync(ep->msg_all, ep->msg_local, floats_per_rank * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)); return 0; }
    return nccl_check(g_nccl.all_gather(ep->msg_local, ep->msg_all, floats_per_rank, NCCL_FLOAT, ep->comm, (cudaStream_t)stream), "ncclAllGather");
}
// reduce-scatter (sum) of the partial rows: partial [world * tokens_local, hidden] -> y [tokens_local, hidden]
extern "C" int qw4sh_ep_reduce_scatter(QW4ShEp *ep, float *y, size_t floats_per_rank, void *stream) {
    if (ep->world == 1) { CU(cudaMemcpyAsync(y, ep->partial, floats_per_rank * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)); return 0; }
    return nccl_check(g_nccl.reduce_scatter(ep->partial, y, floats_per_rank, NCCL_FLOAT, NCCL_SUM, ep->comm, (cudaStream_t)stream), "ncclReduceScatter");
}
