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
// Two exchanges per layer, both on large contiguous buffers.  Their default transport is this file's own kernels
// over NVLink peer memory: every rank maps the other ranks' gather and partial-sum buffers (CUDA IPC handles,
// handed round once through the communicator) and
//   - the all-gather is a PUSH: ep_push_kernel stores the rank's rows into every rank's gather buffer with plain
//     128-bit peer stores, fences, and the CTA that finishes last raises this rank's epoch in every peer's flag row;
//   - the reduce-scatter is a PULL: after its partial sums are written a rank raises its second epoch at the peers;
//     ep_pull_sum_kernel reads the partial rows of its own tokens from every rank (uncached peer loads) and adds
//     them in rank order, which also makes the sum's order fixed.
// A rank waits for its peers' epochs in small kernels of its own (ep_wait_kernel): acquire loads, a bounded
// number of polls (about eight seconds), then QW4SH_ERR_STATE in the workspace's status word and the step goes on
// with whatever arrived; nothing spins without a limit.  Buffers need no double buffering: a rank can only push
// rows of the next layer after it has seen every peer's partial-sum epoch of this one, and a peer raises that only
// after its last read of the gathered rows; and a rank overwrites its partial sums only after it has seen every
// peer's next push, which a peer issues after its pull.  No multicast, no TMA, no library kernel on peer memory.
// NCCL (ncclAllGather / ncclReduceScatter, bound at run time by dlopen of libnccl.so.2) hands the IPC handles
// round and remains the transport when peer mapping is not possible or QW4CU_EP_TRANSPORT=nccl is set.
//
// The sum over a token's experts runs per rank and then over ranks (rank order with the peer transport, NCCL's
// order otherwise), not in slot order: y differs from the one-GPU result in the last bits (the layer tolerance
// holds); ids and weights are the router's bits.
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

// ---- peer-memory transport --------------------------------------------------------------------------------
constexpr int EP_MAX_WORLD = 8;
constexpr uint32_t EP_FLAG_ROWS = 0, EP_FLAG_PARTIAL = EP_MAX_WORLD;         // flag row: [2][EP_MAX_WORLD] epochs, indexed by the writer's rank
struct PeerTable {
    float *msg_all[EP_MAX_WORLD];            // every rank's gather buffer (own entry: the local pointer)
    const float *partial[EP_MAX_WORLD];      // every rank's partial sums
    uint32_t *flags[EP_MAX_WORLD];           // every rank's flag row
};
struct EpState { uint32_t done, epoch_rows, epoch_partial, pad; };          // local: CTA counter of the push, this rank's two epochs

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// This rank's rows -> slot `rank` of every rank's gather buffer; the last CTA to finish raises the rows epoch.
__global__ void __launch_bounds__(256) ep_push_kernel(const float *__restrict__ msg_local, uint32_t quads, PeerTable pt, uint32_t rank,
                                                      uint32_t world, EpState *state) {
    const float4 *src = reinterpret_cast<const float4 *>(msg_local);
    for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < quads; i += gridDim.x * 256) {
        const float4 v = src[i];
        for (uint32_t r = 0; r < world; r++) reinterpret_cast<float4 *>(pt.msg_all[r])[(uint64_t)rank * quads + i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&state->done, 1u) == gridDim.x - 1) {
        state->done = 0;
        const uint32_t epoch = state->epoch_rows + 1;
        state->epoch_rows = epoch;
        __threadfence_system();
        for (uint32_t r = 0; r < world; r++) if (r != rank) st_release_sys(pt.flags[r] + EP_FLAG_ROWS + rank, epoch);
    }
}
// Raises this rank's partial-sum epoch at the peers (after the kernels that wrote the sums, in stream order).
__global__ void ep_signal_partial_kernel(PeerTable pt, uint32_t rank, uint32_t world, EpState *state) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const uint32_t epoch = state->epoch_partial + 1;
    state->epoch_partial = epoch;
    __threadfence_system();
    for (uint32_t r = 0; r < world; r++) if (r != rank) st_release_sys(pt.flags[r] + EP_FLAG_PARTIAL + rank, epoch);
}
// Lane r waits until rank r's epoch in this rank's flag row has reached this rank's own (the ranks step together).
constexpr uint32_t EP_WAIT_POLLS = 1u << 22;                                  // about eight seconds with the sleeps below
__global__ void __launch_bounds__(32) ep_wait_kernel(const uint32_t *flags_local, uint32_t base, const uint32_t *own_epoch, uint32_t rank,
                                                     uint32_t world, uint32_t limit, uint32_t *status) {
    const uint32_t r = threadIdx.x;
    if (r >= world || r == rank) return;
    const uint32_t want = *own_epoch;
    for (uint32_t polls = 0; polls < limit; polls++) {
        if ((int32_t)(ld_acquire_sys(flags_local + base + r) - want) >= 0) return;
        __nanosleep(polls < 64 ? 20 : polls < 4096 ? 200 : 2000);
    }
    atomicOr(status, QW4SH_ERR_STATE);
}
// y[i] = sum over ranks, in rank order, of that rank's partial row of this rank's token.
__global__ void __launch_bounds__(256) ep_pull_sum_kernel(PeerTable pt, float *__restrict__ y, uint32_t quads, uint32_t rank, uint32_t world) {
    for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < quads; i += gridDim.x * 256) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < world; r++) {
            const float4 v = __ldcv(reinterpret_cast<const float4 *>(pt.partial[r]) + (uint64_t)rank * quads + i);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        reinterpret_cast<float4 *>(y)[i] = sum;
    }
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
    float *msg_local;                                // grown on demand, owned here
    size_t msg_local_floats;
    // ONE allocation holds what the peers touch, so that one IPC handle per rank covers it:
    // flag row [2][EP_MAX_WORLD] | gather buffer | partial sums
    unsigned char *pool;
    size_t pool_bytes, msg_all_floats, partial_floats, partial_offset;
    float *msg_all, *partial;                        // into the pool
    uint32_t *flags;
    // peer-memory transport
    int peer;                                        // 1: the table below is valid on every rank
    EpState *state;
    unsigned char *handles;                          // device staging for the exchange of IPC handles
    PeerTable table;
    void *mapped[EP_MAX_WORLD];                      // what cudaIpcOpenMemHandle returned (to close)
};
constexpr size_t EP_POOL_HEAD = 256;                 // bytes of the flag row at the head of the pool

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
// ---- peer mapping ------------------------------------------------------------------------------------------
static void peer_close(QW4ShEp *ep) {
    for (void *&m : ep->mapped) if (m) { cudaIpcCloseMemHandle(m); m = nullptr; }
    ep->peer = 0;
}
// A tiny all-gather through NCCL on the default stream: `bytes` per rank from ep->handles[rank * bytes] in place.
static int tiny_all_gather(QW4ShEp *ep, size_t bytes) {
    if (nccl_check(g_nccl.all_gather(ep->handles + ep->rank * bytes, ep->handles, bytes, 0 /* ncclInt8 */, ep->comm, (cudaStream_t)0), "ncclAllGather"))
        return -1;
    CU(cudaStreamSynchronize((cudaStream_t)0));
    return 0;
}
// Collective over the communicator: every rank exports its gather buffer, partial sums and flag row and maps the
// others'.  Peer transport is on only when EVERY rank mapped everything (agreed by a second tiny all-gather).
static int peer_open(QW4ShEp *ep) {
    const char *transport = getenv("QW4CU_EP_TRANSPORT");
    const bool wanted = !(transport && !strcmp(transport, "nccl")) && ep->world <= EP_MAX_WORLD;
    constexpr size_t RECORD = sizeof(cudaIpcMemHandle_t);
    if (!ep->handles) {
        CU(cudaMalloc(&ep->handles, EP_MAX_WORLD * RECORD));
        CU(cudaMalloc(&ep->state, sizeof(EpState)));
    }
    CU(cudaMemset(ep->state, 0, sizeof(EpState)));                              // epochs restart with the (zeroed) flag rows
    unsigned char mine[RECORD], all[EP_MAX_WORLD * RECORD];
    memset(mine, 0, sizeof mine);
    bool ok = wanted && cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(mine), ep->pool) == cudaSuccess;
    (void)cudaGetLastError();
    CU(cudaMemcpy(ep->handles + ep->rank * RECORD, mine, RECORD, cudaMemcpyHostToDevice));
    if (tiny_all_gather(ep, RECORD)) return -1;                                 // also: every rank has zeroed its new pool by now
    CU(cudaMemcpy(all, ep->handles, ep->world * RECORD, cudaMemcpyDeviceToHost));
    for (int r = 0; r < ep->world; r++) {
        void *base = ep->pool;
        if (r != ep->rank) {
            base = nullptr;
            if (ok) ok = cudaIpcOpenMemHandle(&base, *reinterpret_cast<cudaIpcMemHandle_t *>(all + r * RECORD), cudaIpcMemLazyEnablePeerAccess) == cudaSuccess && base;
            if (ok) ep->mapped[r] = base;
        }
        unsigned char *bytes = (unsigned char *)base;                           // every rank lays its pool out alike (same token counts)
        ep->table.flags[r] = (uint32_t *)bytes;
        ep->table.msg_all[r] = (float *)(bytes ? bytes + EP_POOL_HEAD : nullptr);
        ep->table.partial[r] = (const float *)(bytes ? bytes + ep->partial_offset : nullptr);
    }
    (void)cudaGetLastError();
    // agreement: one byte per rank
    const unsigned char vote = ok ? 1 : 0;
    unsigned char votes[EP_MAX_WORLD];
    CU(cudaMemcpy(ep->handles + ep->rank, &vote, 1, cudaMemcpyHostToDevice));
    if (tiny_all_gather(ep, 1)) return -1;
    CU(cudaMemcpy(votes, ep->handles, ep->world, cudaMemcpyDeviceToHost));
    for (int r = 0; r < ep->world; r++) ok = ok && votes[r];
    if (!ok) peer_close(ep);
    ep->peer = ok ? 1 : 0;
    return 0;
}

// Collective when the peer transport is on (the peers may still be reading this rank's buffers): every rank calls it.
extern "C" void qw4sh_ep_destroy(QW4ShEp *ep) {
    if (!ep) return;
    if (ep->peer) {
        cudaDeviceSynchronize();
        unsigned char zero = 0;
        cudaMemcpy(ep->handles + ep->rank, &zero, 1, cudaMemcpyHostToDevice);
        tiny_all_gather(ep, 1);                                                  // nobody lets go before everybody has finished its last step
        peer_close(ep);
        tiny_all_gather(ep, 1);                                                  // nobody frees what a peer still has mapped
    }
    if (ep->comm) g_nccl.comm_destroy(ep->comm);
    cudaFree(ep->msg_local); cudaFree(ep->pool);
    cudaFree(ep->state); cudaFree(ep->handles);
    delete ep;
}
extern "C" int qw4sh_ep_transport(const QW4ShEp *ep) { return ep ? ep->peer : 0; }
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
    const size_t gather_floats = total * pitch + 4, partial_floats = total * hidden + 4;
    if (ep->msg_all_floats >= gather_floats && ep->partial_floats >= partial_floats) return 0;
    if (ep->world > 1) {
        // the peers hold mappings of the pool about to be replaced: everybody lets go first (the ranks take this
        // branch together: every rank brings the same token count)
        CU(cudaDeviceSynchronize());
        if (ep->peer) {
            unsigned char zero = 0;
            CU(cudaMemcpy(ep->handles + ep->rank, &zero, 1, cudaMemcpyHostToDevice));
            if (tiny_all_gather(ep, 1)) return -1;
            peer_close(ep);
            if (tiny_all_gather(ep, 1)) return -1;                             // nobody frees what a peer still has mapped
        }
    }
    cudaFree(ep->pool);
    ep->pool = nullptr; ep->pool_bytes = 0; ep->msg_all_floats = ep->partial_floats = 0;
    const size_t partial_offset = (EP_POOL_HEAD + gather_floats * sizeof(float) + 255) & ~(size_t)255;
    const size_t bytes = partial_offset + partial_floats * sizeof(float);
    CU(cudaMalloc(&ep->pool, bytes));
    CU(cudaMemset(ep->pool, 0, EP_POOL_HEAD));
    CU(cudaDeviceSynchronize());
    ep->pool_bytes = bytes; ep->partial_offset = partial_offset;
    ep->flags = (uint32_t *)ep->pool;
    ep->msg_all = (float *)(ep->pool + EP_POOL_HEAD); ep->msg_all_floats = gather_floats;
    ep->partial = (float *)(ep->pool + partial_offset); ep->partial_floats = partial_floats;
    return ep->world > 1 ? peer_open(ep) : 0;
}
extern "C" float *qw4sh_ep_msg_local(QW4ShEp *ep) { return ep->msg_local; }
extern "C" float *qw4sh_ep_msg_all(QW4ShEp *ep) { return ep->msg_all; }
extern "C" float *qw4sh_ep_partial_buffer(QW4ShEp *ep) { return ep->partial; }

// all-gather of the packed rows: msg_local [tokens_local, pitch] -> msg_all [world * tokens_local, pitch]
extern "C" int qw4sh_ep_all_gather(QW4ShEp *ep, size_t floats_per_rank, uint32_t *status, void *stream) {
    if (ep->world == 1) { CU(cudaMemcpyAsync(ep->msg_all, ep->msg_local, floats_per_rank * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)); return 0; }
    if (ep->peer && floats_per_rank % 4 == 0 && floats_per_rank / 4 < (1u << 31)) {
        const uint32_t quads = (uint32_t)(floats_per_rank / 4), blocks = (quads + 255) / 256;
        ep_push_kernel<<<blocks < 296 ? blocks : 296, 256, 0, (cudaStream_t)stream>>>(ep->msg_local, quads, ep->table, (uint32_t)ep->rank, (uint32_t)ep->world, ep->state);
        qw4sh_note_launch("ep_push_kernel");
        ep_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ep->flags, EP_FLAG_ROWS, &ep->state->epoch_rows, (uint32_t)ep->rank, (uint32_t)ep->world, EP_WAIT_POLLS, status);
        return qw4sh_note_launch("ep_wait_kernel");
    }
    return nccl_check(g_nccl.all_gather(ep->msg_local, ep->msg_all, floats_per_rank, NCCL_FLOAT, ep->comm, (cudaStream_t)stream), "ncclAllGather");
}
// reduce-scatter (sum) of the partial rows: partial [world * tokens_local, hidden] -> y [tokens_local, hidden]
extern "C" int qw4sh_ep_reduce_scatter(QW4ShEp *ep, float *y, size_t floats_per_rank, uint32_t *status, void *stream) {
    if (ep->world == 1) { CU(cudaMemcpyAsync(y, ep->partial, floats_per_rank * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)); return 0; }
    if (ep->peer && floats_per_rank % 4 == 0 && floats_per_rank / 4 < (1u << 31) && ((uintptr_t)y & 15u) == 0) {
        const uint32_t quads = (uint32_t)(floats_per_rank / 4), blocks = (quads + 255) / 256;
        ep_signal_partial_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ep->table, (uint32_t)ep->rank, (uint32_t)ep->world, ep->state);
        qw4sh_note_launch("ep_signal_partial_kernel");
        ep_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ep->flags, EP_FLAG_PARTIAL, &ep->state->epoch_partial, (uint32_t)ep->rank, (uint32_t)ep->world, EP_WAIT_POLLS, status);
        qw4sh_note_launch("ep_wait_kernel");
        ep_pull_sum_kernel<<<blocks < 592 ? blocks : 592, 256, 0, (cudaStream_t)stream>>>(ep->table, y, quads, (uint32_t)ep->rank, (uint32_t)ep->world);
        return qw4sh_note_launch("ep_pull_sum_kernel");
    }
    return nccl_check(g_nccl.reduce_scatter(ep->partial, y, floats_per_rank, NCCL_FLOAT, NCCL_SUM, ep->comm, (cudaStream_t)stream), "ncclReduceScatter");
}

// Test aid: the wait kernel on a flag row that nothing raises, as rank 0 of two, with a short poll limit (at most
// 65536 polls, about a tenth of a second).  Returns the status bits the kernel left (QW4SH_ERR_STATE when the wait
// ran out, as it must) or a negative value on a CUDA error; the context stays usable either way.
extern "C" int qw4sh_ep_wait_probe(uint32_t polls, int raise_first) {
    uint32_t *words = nullptr;                                                  // [0..15] flag row, [16] own epoch, [17] status
    CU(cudaMalloc(&words, 32 * sizeof(uint32_t)));
    uint32_t host[32] = {0};
    host[16] = 1;                                                               // this rank is at epoch 1
    if (raise_first) host[EP_FLAG_ROWS + 1] = 1;                                // ... and so is the peer (the wait returns at once)
    cudaError_t e = cudaMemcpy(words, host, sizeof host, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) {
        ep_wait_kernel<<<1, 32>>>(words, EP_FLAG_ROWS, words + 16, 0u, 2u, polls < 65536u ? polls : 65536u, words + 17);
        qw4sh_note_launch("ep_wait_kernel");
        e = cudaDeviceSynchronize();
    }
    if (e == cudaSuccess) e = cudaMemcpy(host, words, sizeof host, cudaMemcpyDeviceToHost);
    cudaFree(words);
    if (e != cudaSuccess) { qw4sh_fail_text(cudaGetErrorString(e)); return -1; }
    return (int)host[17];
}
